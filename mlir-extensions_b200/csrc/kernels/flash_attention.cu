// Attention forward, O = softmax(sm_scale * Q K^T) V, one pass over K and V with the
// running-max / running-sum recurrence, on the 5th-generation tensor cores.
//
// Reference: test/Integration/Dialect/XeGPU/WG/flash_attention_fwd.mlir (gpu_impl :254-330,
// the per-tile recurrence :111-250, and the CPU check :334-432 that the oracle restates):
// Q, K, V, O are [heads * n_ctx, 64] 16-bit arrays, heads one after the other.
//
// One CTA per (head, block of 128 query rows):
//   warp 0      TMA producer: the Q tile once, then K and V tiles of 128 keys through a
//               three-stage ring (all tiles are 128 rows x 64 d = one 128B-swizzled box).
//   warp 1      one thread issues tcgen05.mma: S_j = Q K_j^T (M128 N128 K64; both operands
//               K-major) into one of two TMEM S buffers, one block ahead of the softmax;
//               then PV_j = P_j V_j (M128 N64 K128; P K-major from shared memory, V
//               MN-major exactly as it lies in its tile) into a third TMEM buffer.
//   warps 2-    SPLIT (4, or 2) threads per query row, each with its share of the block's keys
//               and of the output columns: read the
//               scores of S_j from TMEM once (tcgen05.ld), free the S buffer, exchange the
//               two partial row maxima through shared memory, keep m and a partial l,
//               write P_j as 16-bit values into shared memory in the swizzled K-major
//               layout the MMA expects (two P buffers, two PV buffers in TMEM), then fold
//               PV_{j-1} into their f32 output registers while the tensor core works on
//               S_{j+1} and PV_j.  No shuffles.
// Every wait is bounded; a wait that runs out records a status code, the roles leave
// their loops, the CTA syncs and frees its TMEM.
#include "kernels.h"
#include "tcgen05_host.h"
#include "tcgen05_ptx.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <string>

namespace imex {
namespace {

using namespace tc;
using namespace tc_host;

constexpr int BQ = 128;        // query rows per CTA
constexpr int BKV = 128;       // keys per block
constexpr int DH = 64;         // head dimension
constexpr int KV_STAGES = 3;  // 144 KB of shared memory: one CTA per SM, which owns all 512 TMEM columns
constexpr int TILE_BYTES = 128 * DH * 2;        // 16 KB: any of the Q / K / V tiles
constexpr int P_BYTES = BQ * BKV * 2;           // 32 KB: two 128 x 64-key boxes; two such buffers
// threads: producer warp, MMA warp, 4 * SPLIT softmax warps (SPLIT threads per query row)
constexpr int num_threads(int split) { return 64 + 128 * split; }
constexpr int TMEM_COLS = 512;  // S0 [0,128) S1 [128,256) PV0 [256,320) PV1 [320,384) P0 [384,448) P1 [448,512)
constexpr int PV_COL = 256;
constexpr int P_COL = 384;      // P as the A operand of P.V: 128 keys = 64 columns of two 16-bit values
constexpr int XCH_BYTES = 2 * 4 * BQ * 4;           // partial row maxima / sums of the threads of a row
constexpr int SMEM_BYTES = TILE_BYTES + KV_STAGES * 2 * TILE_BYTES + 2 * P_BYTES + 1024 + 256 + XCH_BYTES;

struct AttnParams {
  long long *stats;   // optional cycle counters (nullptr = off), 8 per CTA
  void *O;
  unsigned *status;
  int n_ctx;
  int heads;
  float scale_log2e;  // sm_scale * log2(e)
  int is_bf16;
  uint32_t idesc_s, idesc_pv;
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// two f32 -> one 32-bit word of two 16-bit values (a in the low half), round to nearest even
__device__ __forceinline__ uint32_t pack2(float a, float b, int is_bf16) {
  uint32_t w;
  if (is_bf16) asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(w) : "f"(b), "f"(a));
  else asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(w) : "f"(b), "f"(a));
  return w;
}
// ---- packed arithmetic of sm_100: two f32 per 64-bit register, two f16 per 32-bit register
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
  uint64_t w;
  asm("mov.b64 %0, {%1, %2};" : "=l"(w) : "f"(lo), "f"(hi));
  return w;
}
__device__ __forceinline__ uint64_t pack_u32x2(uint32_t lo, uint32_t hi) {
  uint64_t w;
  asm("mov.b64 %0, {%1, %2};" : "=l"(w) : "r"(lo), "r"(hi));
  return w;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t w, float &lo, float &hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(w));
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// 2^x of two f16 values at once: one trip through the special-function unit for two keys, and
// the result is already the packed 16-bit pair the P tile holds
__device__ __forceinline__ uint32_t ex2_f16x2(uint32_t x) {
  uint32_t y;
  asm("ex2.approx.f16x2 %0, %1;" : "=r"(y) : "r"(x));
  return y;
}
__device__ __forceinline__ uint32_t add_f16x2(uint32_t a, uint32_t b) {
  uint32_t y;
  asm("add.rn.f16x2 %0, %1, %2;" : "=r"(y) : "r"(a), "r"(b));
  return y;
}
__device__ __forceinline__ float sum_halves_f16x2(uint32_t w) {
  float lo, hi;
  asm("{\n\t.reg .b16 l, h;\n\tmov.b32 {l, h}, %2;\n\tcvt.f32.f16 %0, l;\n\tcvt.f32.f16 %1, h;\n\t}"
      : "=f"(lo), "=f"(hi)
      : "r"(w));
  return lo + hi;
}
__device__ __forceinline__ void st_shared_f32(uint32_t addr, float v) {
  asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ float ld_shared_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}

__device__ __forceinline__ void st_shared_v4_u32(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// 16 consecutive 32-bit columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_st_16cols(uint32_t taddr, const uint32_t *r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// D (TMEM) (+)= A (TMEM: row = lane, two 16-bit values of consecutive k per column) . B (shared memory)
__device__ __forceinline__ void tcgen05_mma_f16_a_tmem(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                                       uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

template <int N> __device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t (&r)[N]);
template <> __device__ __forceinline__ void tmem_ld_cols<32>(uint32_t taddr, uint32_t (&r)[32]) {
  tmem_ld_32x32(taddr, r);
}
template <> __device__ __forceinline__ void tmem_ld_cols<16>(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

// FAST16 (f16 only): the exponentials run as ex2.approx.f16x2 on the 16-bit rounded exponent
// (x = s' - m <= 0, so its absolute rounding error is largest where 2^x is smallest) and the
// row sums are added up from the packed P values themselves.
// PTMEM: P goes from the softmax threads' registers into TMEM (tcgen05.st) and the second MMA
// takes it from there; otherwise through the swizzled shared-memory tile.
template <int SPLIT, bool STATS, bool FAST16, bool PTMEM>
__global__ void __launch_bounds__(num_threads(SPLIT), 1)
flash_attention_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                           const __grid_constant__ CUtensorMap tmap_v, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_smem = smem_base;
  auto k_smem = [&](int s) { return smem_base + TILE_BYTES + s * 2 * TILE_BYTES; };
  auto v_smem = [&](int s) { return k_smem(s) + TILE_BYTES; };
  auto p_smem = [&](int b) { return smem_base + TILE_BYTES + KV_STAGES * 2 * TILE_BYTES + b * P_BYTES; };
  const uint32_t bars = p_smem(2);
  const uint32_t q_full = bars;
  auto kv_full = [&](int s) { return bars + 8u * (1 + s); };
  auto kv_empty = [&](int s) { return bars + 8u * (1 + KV_STAGES + s); };
  auto s_full = [&](int b) { return bars + 8u * (1 + 2 * KV_STAGES + b); };
  auto s_empty = [&](int b) { return bars + 8u * (3 + 2 * KV_STAGES + b); };
  auto p_full = [&](int b) { return bars + 8u * (5 + 2 * KV_STAGES + b); };
  auto pv_full = [&](int b) { return bars + 8u * (7 + 2 * KV_STAGES + b); };
  auto pv_empty = [&](int b) { return bars + 8u * (9 + 2 * KV_STAGES + b); };
  auto xch_bar_of = [&](int g) { return bars + 8u * (11 + 2 * KV_STAGES + g); };   // one per lane group
  const uint32_t tmem_slot = bars + 8u * (15 + 2 * KV_STAGES);
  const uint32_t xch = bars + 256;
  uint8_t *smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
  volatile uint32_t *tmem_slot_ptr = reinterpret_cast<volatile uint32_t *>(
      smem_aligned + TILE_BYTES + KV_STAGES * 2 * TILE_BYTES + 2 * P_BYTES + 8 * (15 + 2 * KV_STAGES));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int head = blockIdx.y;
  const int q0 = blockIdx.x * BQ;                 // first query row of this CTA inside the head
  const int head_row0 = head * p.n_ctx;           // first row of the head in the arrays
  const int num_blocks = (p.n_ctx + BKV - 1) / BKV;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(kv_full(s), 1);
      mbar_init(kv_empty(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(s_full(b), 1);
      mbar_init(s_empty(b), 4 * SPLIT);   // lane 0 of each softmax warp
      mbar_init(p_full(b), 4 * SPLIT);
      mbar_init(pv_full(b), 1);
      mbar_init(pv_empty(b), 4 * SPLIT);
    }
    for (int g = 0; g < 4; ++g) mbar_init(xch_bar_of(g), SPLIT);   // the SPLIT warps that share rows
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_q) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_k) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_v) : "memory");
      mbar_expect_tx(q_full, TILE_BYTES);
      tma_load_3d(q_smem, &tmap_q, 0, q0, head, q_full);
      int filled = 0;
      for (int j = 0; j < num_blocks; ++j) {
        const int s = j % KV_STAGES;
        if (!mbar_wait(kv_empty(s), ((j / KV_STAGES) & 1) ^ 1u)) {
          report(p.status, kStatusTmaWaitTimeout);
          break;
        }
        mbar_expect_tx(kv_full(s), 2 * TILE_BYTES);
        tma_load_3d(k_smem(s), &tmap_k, 0, j * BKV, head, kv_full(s));
        tma_load_3d(v_smem(s), &tmap_v, 0, j * BKV, head, kv_full(s));
        filled = j + 1;
      }
      // every tile this thread asked for has been consumed before the CTA may go
      for (int j = filled; j < filled + KV_STAGES && filled >= KV_STAGES; ++j) {
        if (!mbar_wait(kv_empty(j % KV_STAGES), ((j / KV_STAGES) & 1) ^ 1u)) break;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      long long w_kv = 0, w_se = 0, w_pf = 0, w_pe = 0;
      const long long t_begin = STATS ? clock64() : 0;
      bool ok = mbar_wait(q_full, 0);
      if (!ok) report(p.status, kStatusMmaWaitTimeout);
      const uint64_t q_desc = make_smem_desc(q_smem, 16, 1024);
      const uint64_t p_desc = make_smem_desc(p_smem(0), 16, 1024);
      auto issue_s = [&](int j) -> bool {
        const int s = j % KV_STAGES, b = j & 1;
        long long t0 = STATS ? clock64() : 0;
        if (!mbar_wait(kv_full(s), (j / KV_STAGES) & 1)) return false;
        if (STATS) { const long long t1 = clock64(); w_kv += t1 - t0; t0 = t1; }
        if (!mbar_wait(s_empty(b), ((j >> 1) & 1) ^ 1u)) return false;
        if (STATS) w_se += clock64() - t0;
        tcgen05_fence_after();
        // a step of 16 along d is 32 bytes inside the swizzled rows: +2 in the address field
        const uint64_t kd = make_smem_desc(k_smem(s), 16, 1024);
#pragma unroll
        for (int k = 0; k < DH / 16; ++k)
          tcgen05_mma_f16(tmem_base + b * BKV, q_desc + 2 * k, kd + 2 * k, p.idesc_s, k ? 1u : 0u);
        tcgen05_commit(s_full(b));
        return true;
      };
      auto issue_pv = [&](int j) -> bool {
        const int s = j % KV_STAGES, b = j & 1;
        long long t0 = STATS ? clock64() : 0;
        if (!mbar_wait(p_full(b), (j >> 1) & 1)) return false;
        if (STATS) { const long long t1 = clock64(); w_pf += t1 - t0; t0 = t1; }
        if (!mbar_wait(pv_empty(b), ((j >> 1) & 1) ^ 1u)) return false;
        if (STATS) w_pe += clock64() - t0;
        tcgen05_fence_after();
        // P: 16 keys are 32 bytes (+2) inside a box of 64 keys, the second box 16 KB on (+1024);
        // V: 16 keys are 16 rows of 128 bytes (+128)
        const uint64_t pd = p_desc + static_cast<uint64_t>(b) * (P_BYTES >> 4);
        const uint64_t vd = make_smem_desc(v_smem(s), TILE_BYTES, 1024);
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k) {
          if constexpr (PTMEM)
            tcgen05_mma_f16_a_tmem(tmem_base + PV_COL + b * DH, tmem_base + P_COL + b * (BKV / 2) + k * 8,
                                   vd + k * 128, p.idesc_pv, k ? 1u : 0u);
          else
            tcgen05_mma_f16(tmem_base + PV_COL + b * DH, pd + (k >> 2) * (TILE_BYTES >> 4) + (k & 3) * 2,
                            vd + k * 128, p.idesc_pv, k ? 1u : 0u);
        }
        tcgen05_commit(pv_full(b));   // PV_j is complete: P buffer b and this K/V stage are free again
        tcgen05_commit(kv_empty(s));
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; j < num_blocks && ok; ++j) {
        if (j + 1 < num_blocks) ok = issue_s(j + 1);
        if (ok) ok = issue_pv(j);
      }
      if (!ok) report(p.status, kStatusMmaWaitTimeout);
      if (STATS && p.stats) {
        long long *st = p.stats + 8 * (blockIdx.y * gridDim.x + blockIdx.x);
        st[0] = clock64() - t_begin;  // MMA thread, total
        st[1] = w_kv;                 // ... waiting for K/V tiles
        st[2] = w_se;                 // ... for a free S buffer
        st[3] = w_pf;                 // ... for P
        st[4] = w_pe;                 // ... for a free PV buffer
      }
    }
  } else {
    // ------------------------------------------------------------ softmax + output
    // SPLIT threads per query row: warp w takes the TMEM lanes 32 * (w % 4) ... (a warp can
    // reach no others), so warps w, w + 4, ... see the same rows; part = (w - 2) / 4 takes
    // keys [part * 128 / SPLIT, ...) of every block and the same share of the output
    // columns.  The parts of a row exchange their partial maxima through shared memory
    // once per block.
    const int lane_group = warp & 3;
    const int part = (warp - 2) >> 2;
    const int r = lane_group * 32 + lane;                       // row of the tile = TMEM lane
    constexpr int HC = BKV / SPLIT;   // keys per thread and block
    constexpr int HO = DH / SPLIT;    // output columns per thread
    const uint32_t t_row = tmem_base + (static_cast<uint32_t>(lane_group * 32) << 16);
    // this thread's keys lie in box (part * HC) / 64 of P, from 16-byte chunk ((part * HC) % 64) / 8 on
    const uint32_t p_row_off = ((part * HC) >> 6) * TILE_BYTES + r * 128;
    const uint32_t chunk0 = static_cast<uint32_t>(((part * HC) & 63) >> 3);
    const uint32_t swz = static_cast<uint32_t>(r & 7);
    const uint32_t xch_bar = xch_bar_of(lane_group);
    uint64_t o2[HO / 2];   // output accumulators, two f32 per register (fma.rn.f32x2)
#pragma unroll
    for (int i = 0; i < HO / 2; ++i) o2[i] = 0ull;
    float m = -INFINITY, l = 0.0f, alpha_prev = 0.0f;
    const float neg_inf = -INFINITY;
    bool ok = true;
    // partial results of the threads of a row meet here: xch[parity][part][row]
    auto xch_addr = [&](int parity, int h) { return xch + static_cast<uint32_t>(((parity * 4 + h) * BQ + r) * 4); };
    // every thread of the row gets max (is_max) or sum of all parts' values
    auto exchange = [&](int round, float mine, bool is_max, float &all) -> bool {
      st_shared_f32(xch_addr(round & 1, part), mine);
      __syncwarp();
      if (lane == 0) mbar_arrive(xch_bar);
      bool w = mbar_wait(xch_bar, round & 1);
      w = __all_sync(0xffffffffu, w);
      if (!w) return false;
      all = mine;
#pragma unroll
      for (int h = 1; h < SPLIT; ++h) {
        const float other = ld_shared_f32(xch_addr(round & 1, (part + h) % SPLIT));
        all = is_max ? fmaxf(all, other) : all + other;
      }
      return true;
    };
    auto fold_pv = [&](int j, float alpha) -> bool {
      // O = O * alpha + PV_j (this thread's columns)
      bool w = mbar_wait(pv_full(j & 1), (j >> 1) & 1);
      w = __all_sync(0xffffffffu, w);
      if (!w) return false;
      tcgen05_fence_after();
      uint32_t v[HO];
      tmem_ld_cols<HO>(t_row + PV_COL + (j & 1) * DH + part * HO, v);
      tmem_ld_wait();
      const uint64_t alpha2 = pack_f32x2(alpha, alpha);
#pragma unroll
      for (int i = 0; i < HO / 2; ++i) o2[i] = fma_f32x2(o2[i], alpha2, pack_u32x2(v[2 * i], v[2 * i + 1]));
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(pv_empty(j & 1));
      return true;
    };
    long long w_sf = 0;
    const long long t_begin = STATS ? clock64() : 0;
    for (int j = 0; j < num_blocks; ++j) {
      const int b = j & 1;
      const long long t0 = STATS ? clock64() : 0;
      bool w = mbar_wait(s_full(b), (j >> 1) & 1);
      if (STATS) w_sf += clock64() - t0;
      w = __all_sync(0xffffffffu, w);
      if (!w) { ok = false; break; }
      tcgen05_fence_after();
      // this thread's scores, read once; the S buffer is free again right away
      uint32_t sc[HC];
      if constexpr (HC == 64) {
        uint32_t lo[32], hi[32];
        tmem_ld_32x32(t_row + b * BKV + part * HC, lo);
        tmem_ld_32x32(t_row + b * BKV + part * HC + 32, hi);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) { sc[i] = lo[i]; sc[32 + i] = hi[i]; }
      } else {
        tmem_ld_cols<HC>(t_row + b * BKV + part * HC, sc);
        tmem_ld_wait();
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_empty(b));
      const int valid = p.n_ctx - j * BKV - part * HC;  // this thread's keys that exist (>= HC: all)
      // all keys present and a positive scale (every block but a ragged last one): the
      // maximum is taken on the raw scores and scaled once, nothing is masked
      const bool plain = valid >= HC && p.scale_log2e > 0.0f;
      float mx = neg_inf;   // in units of log2: s * sm_scale * log2 e
      if (plain) {
#pragma unroll
        for (int i = 0; i < HC; i += 2) mx = max3(mx, __uint_as_float(sc[i]), __uint_as_float(sc[i + 1]));
        mx *= p.scale_log2e;
      } else {
#pragma unroll
        for (int i = 0; i < HC; ++i) mx = fmaxf(mx, (i < valid) ? __uint_as_float(sc[i]) * p.scale_log2e : neg_inf);
      }
      float row_max;
      if (!exchange(j, mx, true, row_max)) { ok = false; break; }
      const float m_new = fmaxf(m, row_max);
      const float alpha = ex2(m - m_new);  // 0 on the first block (m = -inf)
      // p = 2^(s' - m_new), rounded to 16 bits into the swizzled K-major P tile; buffer b was
      // last read by PV_{j-2}, whose completion this thread saw when it folded it in
      const uint32_t p_row = p_smem(b) + p_row_off;
      float rowsum = 0.0f;
      const float neg_m = -m_new;
      uint32_t pw[HC / 2];   // this thread's keys of P, two 16-bit values per word
      if (FAST16 && plain) {
        const uint64_t scale2 = pack_f32x2(p.scale_log2e, p.scale_log2e);
        const uint64_t neg_m2 = pack_f32x2(neg_m, neg_m);
#pragma unroll
        for (int i = 0; i < HC / 2; ++i) {
          float x0, x1;
          unpack_f32x2(fma_f32x2(pack_u32x2(sc[2 * i], sc[2 * i + 1]), scale2, neg_m2), x0, x1);
          pw[i] = ex2_f16x2(pack2(x0, x1, 0));
        }
        uint32_t acc[HC / 4];
#pragma unroll
        for (int i = 0; i < HC / 4; ++i) acc[i] = add_f16x2(pw[2 * i], pw[2 * i + 1]);
#pragma unroll
        for (int n = HC / 4; n > 1; n >>= 1)
#pragma unroll
          for (int q = 0; q < n / 2; ++q) acc[q] = add_f16x2(acc[q], acc[q + n / 2]);
        rowsum = sum_halves_f16x2(acc[0]);
      } else {
#pragma unroll
        for (int q = 0; q < HC / 8; ++q) {  // 8 keys at a time
          float e[8];
          if (plain) {
#pragma unroll
            for (int i = 0; i < 8; ++i) e[i] = ex2(fmaf(__uint_as_float(sc[8 * q + i]), p.scale_log2e, neg_m));
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float pe = ex2(fmaf(__uint_as_float(sc[8 * q + i]), p.scale_log2e, neg_m));
              e[i] = (8 * q + i < valid) ? pe : 0.0f;
            }
          }
          rowsum += ((e[0] + e[1]) + (e[2] + e[3])) + ((e[4] + e[5]) + (e[6] + e[7]));
#pragma unroll
          for (int i = 0; i < 4; ++i) pw[4 * q + i] = pack2(e[2 * i], e[2 * i + 1], p.is_bf16);
        }
      }
      if constexpr (PTMEM) {
        // buffer b was last read by PV_{j-2}, whose completion this thread saw when it folded it in
#pragma unroll
        for (int c = 0; c < HC / 2; c += 16)
          tmem_st_16cols(t_row + P_COL + b * (BKV / 2) + part * (HC / 2) + c, pw + c);
        tmem_st_wait();
        tcgen05_fence_before();
      } else {
#pragma unroll
        for (int q = 0; q < HC / 8; ++q)
          st_shared_v4_u32(p_row + (((chunk0 + static_cast<uint32_t>(q)) ^ swz) << 4), pw[4 * q], pw[4 * q + 1],
                           pw[4 * q + 2], pw[4 * q + 3]);
        fence_async_smem();  // P (generic-proxy stores) visible to the tensor core's reads
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full(b));
      l = fmaf(l, alpha, rowsum);
      m = m_new;
      // the previous block's P.V, off the path that feeds the tensor core
      if (j > 0) {
        if (!fold_pv(j - 1, alpha_prev)) { ok = false; break; }
      }
      alpha_prev = alpha;
    }
    if (STATS && p.stats && warp == 2 && lane == 0) {
      long long *st = p.stats + 8 * (blockIdx.y * gridDim.x + blockIdx.x);
      st[5] = clock64() - t_begin;  // a softmax thread, all blocks
      st[6] = w_sf;                 // ... waiting for S
    }
    if (ok && num_blocks > 0) ok = fold_pv(num_blocks - 1, alpha_prev);
    float l_row = 0.0f;
    if (ok) ok = exchange(num_blocks, l, false, l_row);
    if (!ok) {
      if (lane == 0) report(p.status, kStatusEpiWaitTimeout);
    } else if (q0 + r < p.n_ctx) {
      const float inv = 1.0f / l_row;
      float o[HO];
#pragma unroll
      for (int i = 0; i < HO / 2; ++i) unpack_f32x2(o2[i], o[2 * i], o[2 * i + 1]);
      uint16_t *orow = static_cast<uint16_t *>(p.O) + static_cast<size_t>(head_row0 + q0 + r) * DH + part * HO;
#pragma unroll
      for (int c = 0; c < HO; c += 8) {
        const uint4 out = make_uint4(pack2(o[c] * inv, o[c + 1] * inv, p.is_bf16),
                                     pack2(o[c + 2] * inv, o[c + 3] * inv, p.is_bf16),
                                     pack2(o[c + 4] * inv, o[c + 5] * inv, p.is_bf16),
                                     pack2(o[c + 6] * inv, o[c + 7] * inv, p.is_bf16));
        *reinterpret_cast<uint4 *>(orow + c) = out;
      }
    }
  }

  __syncwarp();
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS)
                 : "memory");
  }
}

} // namespace

bool flash_attention_supported(int64_t heads, int64_t n_ctx, int64_t d_head, int dtype, const void *q,
                               const void *k, const void *v, const void *o) {
  if (dtype != kF16 && dtype != kBF16) return false;
  if (d_head != DH || heads <= 0 || n_ctx <= 0) return false;
  if (heads > 65535 || heads * n_ctx > INT32_MAX) return false;
  auto al = [](const void *x) { return (reinterpret_cast<uintptr_t>(x) & 15) == 0; };
  return al(q) && al(k) && al(v) && al(o);
}

cudaError_t launch_flash_attention_fwd(const void *q, const void *k, const void *v, void *o, int64_t heads,
                                       int64_t n_ctx, int64_t d_head, float sm_scale, int dtype,
                                       unsigned *status, cudaStream_t stream) {
  if (!flash_attention_supported(heads, n_ctx, d_head, dtype, q, k, v, o)) return cudaErrorNotSupported;
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  static bool with_stats = false, exp_f32 = false, p_smem = false;
  using Kernel = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const AttnParams);
  // [stats][fast16][p in TMEM]
  static const Kernel kernels[2][2][2] = {
      {{flash_attention_fwd_kernel<4, false, false, false>, flash_attention_fwd_kernel<4, false, false, true>},
       {flash_attention_fwd_kernel<4, false, true, false>, flash_attention_fwd_kernel<4, false, true, true>}},
      {{flash_attention_fwd_kernel<4, true, false, false>, flash_attention_fwd_kernel<4, true, false, true>},
       {flash_attention_fwd_kernel<4, true, true, false>, flash_attention_fwd_kernel<4, true, true, true>}}};
  std::call_once(once, [] {
    with_stats = getenv("IMEX_ATTN_STATS") != nullptr;  // development aid: where the roles wait
    if (const char *e = getenv("IMEX_ATTN_EXP")) exp_f32 = std::string(e) == "f32";  // f16: every exponential in f32
    if (const char *e = getenv("IMEX_ATTN_P")) p_smem = std::string(e) == "smem";   // P through shared memory
    for (int i = 0; i < 8; ++i) {
      cudaError_t x = cudaFuncSetAttribute(kernels[i >> 2][(i >> 1) & 1][i & 1],
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
      if (x != cudaSuccess) attr_err = x;
    }
  });
  if (attr_err != cudaSuccess) return attr_err;
  // heads are a dimension of the tensor maps: a tile that runs past the last key (or query) of
  // its head is filled with zeros, not with the next head's first rows (whose values, were they
  // Inf or NaN, would reach this head's output through 0 x V)
  CUtensorMap tq, tk, tv;
  if (!make_map_batched(&tq, q, dtype, n_ctx, heads, BQ) || !make_map_batched(&tk, k, dtype, n_ctx, heads, BKV) ||
      !make_map_batched(&tv, v, dtype, n_ctx, heads, BKV))
    return cudaErrorNotSupported;
  AttnParams p;
  p.O = o;
  p.status = status;
  p.n_ctx = static_cast<int>(n_ctx);
  p.heads = static_cast<int>(heads);
  p.scale_log2e = sm_scale * 1.4426950408889634f;
  p.is_bf16 = dtype == kBF16 ? 1 : 0;
  const uint32_t fmt = dtype == kBF16 ? 1u : 0u;
  // c = f32; a, b formats; bit 16: B is MN-major (the V tile) ; N >> 3 ; M >> 4
  p.idesc_s = (1u << 4) | (fmt << 7) | (fmt << 10) | (0u << 16) | (static_cast<uint32_t>(BKV >> 3) << 17) |
              (static_cast<uint32_t>(BQ >> 4) << 24);
  p.idesc_pv = (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 16) | (static_cast<uint32_t>(DH >> 3) << 17) |
               (static_cast<uint32_t>(BQ >> 4) << 24);
  const dim3 grid(static_cast<unsigned>((n_ctx + BQ - 1) / BQ), static_cast<unsigned>(heads));
  p.stats = nullptr;
  static long long *stats_buf = nullptr;
  const int ctas = static_cast<int>(grid.x * grid.y);
  if (with_stats && ctas <= 4096) {
    if (!stats_buf) cudaMallocManaged(&stats_buf, 8 * 4096 * sizeof(long long));
    p.stats = stats_buf;
  }
  const bool fast16 = dtype == kF16 && !exp_f32;
  kernels[p.stats ? 1 : 0][fast16 ? 1 : 0][p_smem ? 0 : 1]<<<grid, num_threads(4), SMEM_BYTES, stream>>>(tq, tk, tv, p);
  if (p.stats) {
    cudaStreamSynchronize(stream);
    double a[8] = {0};
    for (int c = 0; c < ctas; ++c)
      for (int i = 0; i < 8; ++i) a[i] += static_cast<double>(stats_buf[8 * c + i]);
    fprintf(stderr,
            "[attention stats, mean cycles per CTA, %d key blocks] mma total %.0f wait_kv %.0f wait_s_free %.0f "
            "wait_p %.0f wait_pv_free %.0f | softmax total %.0f wait_s %.0f\n",
            static_cast<int>((n_ctx + BKV - 1) / BKV), a[0] / ctas, a[1] / ctas, a[2] / ctas, a[3] / ctas,
            a[4] / ctas, a[5] / ctas, a[6] / ctas);
  }
  return cudaGetLastError();
}

} // namespace imex
