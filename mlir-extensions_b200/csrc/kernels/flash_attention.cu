// Attention forward, O = softmax(sm_scale * Q K^T) V, one pass over K and V with the
// running-max / running-sum recurrence, on the 5th-generation tensor cores.
//
// Reference: test/Integration/Dialect/XeGPU/WG/flash_attention_fwd.mlir (gpu_impl :254-330,
// the per-tile recurrence :111-250, and the CPU check :334-432 that the oracle restates):
// Q, K, V, O are [heads * n_ctx, 64] 16-bit arrays, heads one after the other.
//
// One CTA per (head, block of 128 query rows):
//   warp 0      TMA producer: the Q tile once, then K and V tiles of 128 keys through a
//               four-stage ring (all tiles are 128 rows x 64 d = one 128B-swizzled box of a
//               3-D tensor map whose outer dimension is the head, so a ragged last tile is
//               filled with zeros, never with the next head's rows).
//   warp 1      one thread issues tcgen05.mma: S_j = Q K_j^T (M128 N128 K64; both operands
//               K-major in shared memory) into one of two TMEM S buffers, two blocks ahead of
//               the softmax; then O += P_j V_j (M128 N64 K128; P as the A operand from TMEM,
//               V MN-major exactly as it lies in its tile), accumulating in TMEM over all
//               blocks.
//   warps 2-17  four threads per query row, each with 32 of the block's keys and 16 of the
//               output columns, software-pipelined: while the exponentials of block j run,
//               the scores of block j + 1 come from TMEM (tcgen05.ld) into a second register
//               array; P_j goes back into TMEM as 16-bit pairs (tcgen05.st); the four partial
//               row maxima meet through shared memory once per block.  The reference maximum
//               of a row moves only when the row's maximum outgrows it by more than 2^8; only
//               then are O (in TMEM) and the running sum rescaled.  No shuffles.
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
constexpr int KV_STAGES = 4;  // 144 KB of shared memory: one CTA per SM, which owns all 512 TMEM columns
constexpr int TILE_BYTES = 128 * DH * 2;        // 16 KB: any of the Q / K / V tiles
// threads: producer warp, MMA warp, 4 * SPLIT softmax warps (SPLIT threads per query row)
constexpr int num_threads(int split) { return 64 + 128 * split; }
constexpr int TMEM_COLS = 512;  // S0 [0,128) S1 [128,256) O [256,320) P0 [384,448) P1 [448,512)
constexpr int PV_COL = 256;
// the producer and the MMA thread sleep between polls of a barrier: a spinning warp takes issue
// slots from the softmax warps of its scheduler, and neither is on the critical path
constexpr unsigned kPollSleepNs = 40;
constexpr int P_COL = 384;      // P as the A operand of P.V: 128 keys = 64 columns of two 16-bit values
constexpr int XCH_BYTES = 2 * 4 * BQ * 4;           // partial row maxima / sums of the threads of a row
constexpr int SMEM_BYTES = TILE_BYTES + KV_STAGES * 2 * TILE_BYTES + 1024 + 256 + XCH_BYTES;

struct AttnParams {
  long long *stats;   // optional cycle counters (nullptr = off), 24 per CTA
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
__device__ __forceinline__ void st_shared_f32(uint32_t addr, float v) {
  asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ float ld_shared_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
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
__device__ __forceinline__ void tmem_st_8cols(uint32_t taddr, const uint32_t *r) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr),
               "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
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

// P goes from the softmax threads' registers into TMEM (tcgen05.st) and the second MMA takes its
// A operand from there; O accumulates in TMEM.
template <int SPLIT, bool STATS, bool BF16>
__global__ void __launch_bounds__(num_threads(SPLIT), 1)
flash_attention_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                           const __grid_constant__ CUtensorMap tmap_v, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_smem = smem_base;
  auto k_smem = [&](int s) { return smem_base + TILE_BYTES + s * 2 * TILE_BYTES; };
  auto v_smem = [&](int s) { return k_smem(s) + TILE_BYTES; };
  const uint32_t bars = smem_base + TILE_BYTES + KV_STAGES * 2 * TILE_BYTES;
  const uint32_t q_full = bars;
  auto kv_full = [&](int s) { return bars + 8u * (1 + s); };
  auto kv_empty = [&](int s) { return bars + 8u * (1 + KV_STAGES + s); };
  auto s_full = [&](int b) { return bars + 8u * (1 + 2 * KV_STAGES + b); };
  auto s_empty = [&](int b) { return bars + 8u * (3 + 2 * KV_STAGES + b); };
  auto p_full = [&](int b) { return bars + 8u * (5 + 2 * KV_STAGES + b); };
  auto pv_full = [&](int b) { return bars + 8u * (7 + 2 * KV_STAGES + b); };
  auto xch_bar_of = [&](int g) { return bars + 8u * (11 + 2 * KV_STAGES + g); };   // one per lane group
  const uint32_t tmem_slot = bars + 8u * (15 + 2 * KV_STAGES);
  const uint32_t xch = bars + 256;
  uint8_t *smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
  volatile uint32_t *tmem_slot_ptr = reinterpret_cast<volatile uint32_t *>(
      smem_aligned + TILE_BYTES + KV_STAGES * 2 * TILE_BYTES + 8 * (15 + 2 * KV_STAGES));

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
        if (!mbar_wait_relaxed(kv_empty(s), ((j / KV_STAGES) & 1) ^ 1u, kPollSleepNs)) {
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
        if (!mbar_wait_relaxed(kv_empty(j % KV_STAGES), ((j / KV_STAGES) & 1) ^ 1u, kPollSleepNs)) break;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      long long w_kv = 0, w_se = 0, w_pf = 0, w_pe = 0, w_is = 0, w_ip = 0;
      const long long t_begin = STATS ? clock64() : 0;
      bool ok = mbar_wait_relaxed(q_full, 0, kPollSleepNs);
      if (!ok) report(p.status, kStatusMmaWaitTimeout);
      const uint64_t q_desc = make_smem_desc(q_smem, 16, 1024);
      auto issue_s = [&](int j) -> bool {
        const int s = j % KV_STAGES, b = j & 1;
        long long t0 = STATS ? clock64() : 0;
        if (!mbar_wait_relaxed(kv_full(s), (j / KV_STAGES) & 1, kPollSleepNs)) return false;
        if (STATS) { const long long t1 = clock64(); w_kv += t1 - t0; t0 = t1; }
        if (!mbar_wait_relaxed(s_empty(b), ((j >> 1) & 1) ^ 1u, kPollSleepNs)) return false;
        if (STATS) w_se += clock64() - t0;
        tcgen05_fence_after();
        // a step of 16 along d is 32 bytes inside the swizzled rows: +2 in the address field
        const uint64_t kd = make_smem_desc(k_smem(s), 16, 1024);
        const long long t2 = STATS ? clock64() : 0;
#pragma unroll
        for (int k = 0; k < DH / 16; ++k)
          tcgen05_mma_f16(tmem_base + b * BKV, q_desc + 2 * k, kd + 2 * k, p.idesc_s, k ? 1u : 0u);
        tcgen05_commit(s_full(b));
        if (STATS) w_is += clock64() - t2;
        return true;
      };
      auto issue_pv = [&](int j) -> bool {
        const int s = j % KV_STAGES, b = j & 1;
        long long t0 = STATS ? clock64() : 0;
        if (!mbar_wait_relaxed(p_full(b), (j >> 1) & 1, kPollSleepNs)) return false;
        if (STATS) { const long long t1 = clock64(); w_pf += t1 - t0; t0 = t1; }
        tcgen05_fence_after();
        // P: 16 keys are 8 TMEM columns; V: 16 keys are 16 rows of 128 bytes (+128)
        const uint64_t vd = make_smem_desc(v_smem(s), TILE_BYTES, 1024);
        const long long t2 = STATS ? clock64() : 0;
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k) {
          tcgen05_mma_f16_a_tmem(tmem_base + PV_COL, tmem_base + P_COL + b * (BKV / 2) + k * 8, vd + k * 128,
                                 p.idesc_pv, (j | k) ? 1u : 0u);   // O += P_j V_j; the first one starts it
        }
        tcgen05_commit(pv_full(b));   // P_j V_j has been added: P buffer b and this K/V stage are free again
        tcgen05_commit(kv_empty(s));
        if (STATS) w_ip += clock64() - t2;
        return true;
      };
      // S runs two blocks ahead of P.V: the softmax threads take the scores of block j + 1 into
      // registers while they work on block j, so the S buffer of block j + 2 is free by then
      if (ok) ok = issue_s(0);
      if (ok && num_blocks > 1) ok = issue_s(1);
      for (int j = 0; j < num_blocks && ok; ++j) {
        if (j + 2 < num_blocks) ok = issue_s(j + 2);
        if (ok) ok = issue_pv(j);
      }
      if (!ok) report(p.status, kStatusMmaWaitTimeout);
      if (STATS && p.stats) {
        long long *st = p.stats + 24 * (blockIdx.y * gridDim.x + blockIdx.x);
        st[0] = clock64() - t_begin;  // MMA thread, total
        st[1] = w_kv;                 // ... waiting for K/V tiles
        st[2] = w_se;                 // ... for a free S buffer
        st[3] = w_pf;                 // ... for P
        st[4] = w_pe;                 // ... for a free PV buffer
        st[7] = w_is;                 // ... issuing the MMAs of S (4 per block) and their commit
        st[16] = w_ip;                // ... issuing the MMAs of P V (8 per block) and their commits
      }
    }
  } else {
    // ------------------------------------------------------------ softmax + output
    // Four threads per query row: warp w takes the TMEM lanes 32 * (w % 4) ... (a warp can
    // reach no others), so warps w, w + 4, ... see the same rows; part = (w - 2) / 4 takes
    // keys [32 * part, 32 * part + 32) of every block and 16 of the output columns.  The
    // parts of a row exchange their partial maxima through shared memory once per block.
    //
    // The loop is software-pipelined over the key blocks: the exponentials of block j keep
    // the special-function unit busy (16 results per clock and SM: 1024 clocks per block, the
    // longest single item) while the same threads fetch the scores of block j + 1 from TMEM.
    // O accumulates in TMEM over all blocks (the tensor core adds P_j V_j onto it); the
    // reference maximum m only moves when a row's maximum outgrows it by more than 2^8, and
    // only then are O (in TMEM) and l rescaled: P values stay below 2^8 = 256, well inside
    // the range of f16 and bf16, and the final O / l does not depend on the reference.
    static_assert(SPLIT == 4, "the pipelined loop is written for four threads per row");
    const int lane_group = warp & 3;
    const int part = (warp - 2) >> 2;
    const int r = lane_group * 32 + lane;                       // row of the tile = TMEM lane
    constexpr int HC = BKV / SPLIT;   // keys per thread and block (32)
    constexpr int HO = DH / SPLIT;    // output columns per thread (16)
    const uint32_t t_row = tmem_base + (static_cast<uint32_t>(lane_group * 32) << 16);
    const uint32_t xch_bar = xch_bar_of(lane_group);
    float m = -INFINITY, l = 0.0f;   // m: the reference maximum the exponents are taken against
    const float neg_inf = -INFINITY;
    bool ok = true;
    // partial results of the threads of a row meet here: xch[parity][part][row]
    auto xch_addr = [&](int parity, int h) { return xch + static_cast<uint32_t>(((parity * 4 + h) * BQ + r) * 4); };
    // the exchange in two halves, so that other work can stand between them
    auto exchange_post = [&](int round, float mine) {
      st_shared_f32(xch_addr(round & 1, part), mine);
      __syncwarp();
      if (lane == 0) mbar_arrive(xch_bar);
    };
    auto exchange_collect = [&](int round, float mine, bool is_max, float &all) -> bool {
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
    long long ph[8] = {0, 0, 0, 0, 0, 0, 0, 0};   // cycles per phase of the loop body (STATS)
    long long t_last = 0;
    auto tick = [&](int slot) {
      if (STATS) {
        const long long t = clock64();
        ph[slot] += t - t_last;
        t_last = t;
      }
    };
    // this thread's keys of block j that exist (>= HC: all of them)
    auto valid_keys = [&](int j) { return p.n_ctx - j * BKV - part * HC; };
    // maximum of the 32 scores of part `prt` of block j, in units of log2: s * sm_scale * log2 e.
    // With all keys present and a positive scale (every block but a ragged last one) the
    // maximum is taken on the raw scores and scaled once, nothing is masked.
    auto block_max = [&](const uint32_t (&sc)[HC], int j, int prt) __attribute__((always_inline)) -> float {
      const int valid = p.n_ctx - j * BKV - prt * HC;
      if (valid >= HC && p.scale_log2e > 0.0f) {
        float a = neg_inf, c = neg_inf;   // two chains
#pragma unroll
        for (int i = 0; i < HC; i += 4) {
          a = max3(a, __uint_as_float(sc[i]), __uint_as_float(sc[i + 1]));
          c = max3(c, __uint_as_float(sc[i + 2]), __uint_as_float(sc[i + 3]));
        }
        return fmaxf(a, c) * p.scale_log2e;
      }
      float mx = neg_inf;
#pragma unroll
      for (int i = 0; i < HC; ++i) mx = fmaxf(mx, (i < valid) ? __uint_as_float(sc[i]) * p.scale_log2e : neg_inf);
      return mx;
    };
    // P values of keys [8 * q0, 8 * q1) of block j from the scores: p = 2^(s' - m), rounded
    // to 16 bits, two per word; their f32 sum goes into sum2 (two partial sums side by side).
    // `plain` (a literal at every call, folded when the lambda is inlined: the choice is made once
    // per block, outside) says that all 32 keys exist, so nothing is masked and the whole half
    // is one straight line of code.
    auto exp_keys = [&](const bool plain, const uint32_t (&sc)[HC], uint32_t (&pw)[HC / 2], int q0, int q1, int j,
                        float neg_m, uint64_t &sum2) __attribute__((always_inline)) {
      const int valid = valid_keys(j);
      const uint64_t scale2 = pack_f32x2(p.scale_log2e, p.scale_log2e);
      const uint64_t neg_m2 = pack_f32x2(neg_m, neg_m);
#pragma unroll
      for (int q = q0; q < q1; ++q) {
        float e[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float x0, x1;
          unpack_f32x2(fma_f32x2(pack_u32x2(sc[8 * q + 2 * i], sc[8 * q + 2 * i + 1]), scale2, neg_m2), x0, x1);
          e[2 * i] = ex2(x0);
          e[2 * i + 1] = ex2(x1);
        }
        if (!plain) {
#pragma unroll
          for (int i = 0; i < 8; ++i) e[i] = (8 * q + i < valid) ? e[i] : 0.0f;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          sum2 = add_f32x2(sum2, pack_f32x2(e[2 * i], e[2 * i + 1]));
          pw[4 * q + i] = pack2(e[2 * i], e[2 * i + 1], BF16);
        }
      }
    };
    // O (this thread's 16 columns, all blocks so far) and l times 2^(m - m_to) for the rows
    // whose reference maximum moves; the other rows of the warp are multiplied by 1.
    auto rescale = [&](int j_done, bool move, float m_to) -> bool {
      // every P.V issued so far has been added: the last one is PV_{j_done}
      bool w = mbar_wait(pv_full(j_done & 1), (j_done >> 1) & 1);
      w = __all_sync(0xffffffffu, w);
      if (!w) return false;
      tcgen05_fence_after();
      const float a = move ? ex2(m - m_to) : 1.0f;   // m = -inf never comes here
      uint32_t v[HO];
      tmem_ld_cols<HO>(t_row + PV_COL + part * HO, v);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < HO; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * a);
      tmem_st_16cols(t_row + PV_COL + part * HO, v);
      tmem_st_wait();
      tcgen05_fence_before();
      l *= a;
      if (move) m = m_to;
      return true;
    };
    // One turn of the pipelined loop: block j's scores are in `cur` and the reference maximum m
    // covers them (every score of the row is at most m + 8); `nxt` receives the scores of
    // block j + 1.
    long long w_sf = 0;
    auto turn = [&](uint32_t (&cur)[HC], uint32_t (&nxt)[HC], int j) __attribute__((always_inline)) -> bool {
      const int b = j & 1;
      const bool have_next = j + 1 < num_blocks;
      if (STATS) t_last = clock64();
      uint32_t pw[HC / 2];
      uint64_t sum2 = 0ull;
      const float neg_m = -m;
      const uint32_t p_addr = t_row + P_COL + b * (BKV / 2) + part * (HC / 2);
      const bool plain = valid_keys(j) >= HC;
      if (plain) exp_keys(true, cur, pw, 0, HC / 16, j, neg_m, sum2);   // first half of the exponentials
      else exp_keys(false, cur, pw, 0, HC / 16, j, neg_m, sum2);
      tick(0);
      if (j >= 2) {
        // P buffer b was read by PV_{j-2}: finished long ago, but the order must be seen
        bool w = mbar_wait(pv_full(b), ((j - 2) >> 1) & 1);
        w = __all_sync(0xffffffffu, w);
        if (!w) return false;
        tcgen05_fence_after();
      }
      tmem_st_8cols(p_addr, pw);
      if (have_next) {
        // S_{j+1} was issued a whole block ago: it is there
        const long long t0 = STATS ? clock64() : 0;
        bool w = mbar_wait(s_full(b ^ 1), ((j + 1) >> 1) & 1);
        if (STATS) w_sf += clock64() - t0;
        w = __all_sync(0xffffffffu, w);
        if (!w) return false;
        tcgen05_fence_after();
        tmem_ld_cols<HC>(t_row + (b ^ 1) * BKV + part * HC, nxt);   // lands while the second half runs
      }
      tick(1);
      if (plain) exp_keys(true, cur, pw, HC / 16, HC / 8, j, neg_m, sum2);   // second half
      else exp_keys(false, cur, pw, HC / 16, HC / 8, j, neg_m, sum2);
      tick(2);
      tmem_st_8cols(p_addr + 8, pw + 8);
      if (have_next) tmem_ld_wait();
      tmem_st_wait();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(p_full(b));
        if (have_next) mbar_arrive(s_empty(b ^ 1));   // the scores of block j + 1 are in registers
      }
      float s_lo, s_hi;
      unpack_f32x2(sum2, s_lo, s_hi);
      l += s_lo + s_hi;
      tick(3);
      if (have_next) {
        const float mx = block_max(nxt, j + 1, part);
        exchange_post(j + 1, mx);
        tick(4);
        float row_max;
        if (!exchange_collect(j + 1, mx, true, row_max)) return false;
        tick(5);
        // the reference maximum stays while the row's maximum is within 2^8 of it
        const bool move = row_max > m + 8.0f;
        if (__any_sync(0xffffffffu, move)) {
          if (!rescale(j, move, row_max)) return false;
        }
        tick(6);
      }
      return true;
    };
    const long long t_begin = STATS ? clock64() : 0;
    uint32_t sc_a[HC], sc_b[HC];
    if (num_blocks > 0) {
      // prologue: the scores of block 0; their row maximum is the first reference maximum
      bool w = mbar_wait(s_full(0), 0);
      w = __all_sync(0xffffffffu, w);
      if (!w) {
        ok = false;
      } else {
        tcgen05_fence_after();
        tmem_ld_cols<HC>(t_row + part * HC, sc_a);
        tmem_ld_wait();
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(s_empty(0));
        const float mx = block_max(sc_a, 0, part);
        exchange_post(0, mx);
        ok = exchange_collect(0, mx, true, m);
      }
    }
    for (int j = 0; j < num_blocks && ok; j += 2) {
      ok = turn(sc_a, sc_b, j);
      if (ok && j + 1 < num_blocks) ok = turn(sc_b, sc_a, j + 1);
    }
    if (STATS && p.stats && warp == 2 && lane == 0) {
      long long *st = p.stats + 24 * (blockIdx.y * gridDim.x + blockIdx.x);
      st[5] = clock64() - t_begin;  // a softmax thread, all blocks
      st[6] = w_sf;                 // ... waiting for S
      for (int i = 0; i < 8; ++i) st[8 + i] = ph[i];
    }
    float l_row = 0.0f;
    if (ok) {
      exchange_post(num_blocks, l);
      ok = exchange_collect(num_blocks, l, false, l_row);
    }
    if (ok && num_blocks > 0) {
      // O is complete when the last P.V has been added
      bool w = mbar_wait(pv_full((num_blocks - 1) & 1), ((num_blocks - 1) >> 1) & 1);
      ok = __all_sync(0xffffffffu, w);
    }
    if (!ok) {
      if (lane == 0) report(p.status, kStatusEpiWaitTimeout);
    } else {
      tcgen05_fence_after();
      uint32_t v[HO];
      tmem_ld_cols<HO>(t_row + PV_COL + part * HO, v);
      tmem_ld_wait();
      if (q0 + r < p.n_ctx) {
        const float inv = 1.0f / l_row;
        float o[HO];
#pragma unroll
        for (int i = 0; i < HO; ++i) o[i] = __uint_as_float(v[i]) * inv;
        uint16_t *orow = static_cast<uint16_t *>(p.O) + static_cast<size_t>(head_row0 + q0 + r) * DH + part * HO;
#pragma unroll
        for (int c = 0; c < HO; c += 8) {
          const uint4 out = make_uint4(pack2(o[c], o[c + 1], BF16), pack2(o[c + 2], o[c + 3], BF16),
                                       pack2(o[c + 4], o[c + 5], BF16), pack2(o[c + 6], o[c + 7], BF16));
          *reinterpret_cast<uint4 *>(orow + c) = out;
        }
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

// ---------------------------------------------------------------------------------------
// The same computation with the key blocks of a CTA shared out between TWO groups of softmax
// warps that work half a period apart (group 0: blocks [0, nA), group 1: blocks [nA, nb)).
// While one group runs its exponentials the other fetches scores, takes maxima and hands P
// over, so the special-function unit and the tensor core see work from one group or the other
// all the time, which a single group in lock step cannot give them.  Each group keeps its own
// reference maxima, sums and its own O accumulator in TMEM; the two are merged at the end
// (O = (O_0 a_0 + O_1 a_1) / (l_0 a_0 + l_1 a_1) with a_g = 2^(m_g - max(m_0, m_1))).
//
//   warp 0      TMA producer: Q once, then K/V tiles into two stages per group, whichever
//               group has a free stage.
//   warp 1      one thread issues tcgen05.mma, serving whichever group is ready: S of a group's
//               next block as soon as its threads hold the previous scores in registers (one S
//               buffer per group), O_g += P V as soon as the group has handed over P.
//   warps 2-17  group g = (warp - 2) / 8: two threads per query row, 64 keys each.
// TMEM: S_0 [0,128) S_1 [128,256) O_0 [256,320) O_1 [320,384) P_0 [384,448) P_1 [448,512).
constexpr int PP_FIN_BYTES = 2 * 2 * BQ * 8;   // (m, l) of every group / part / row for the merge
constexpr int PP_SMEM_BYTES = SMEM_BYTES + PP_FIN_BYTES;

template <bool BF16>
__global__ void __launch_bounds__(num_threads(4), 1)
flash_attention_fwd_pp_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                              const __grid_constant__ CUtensorMap tmap_v, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_smem = smem_base;
  auto k_smem = [&](int s) { return smem_base + TILE_BYTES + s * 2 * TILE_BYTES; };
  auto v_smem = [&](int s) { return k_smem(s) + TILE_BYTES; };
  const uint32_t bars = smem_base + TILE_BYTES + KV_STAGES * 2 * TILE_BYTES;
  const uint32_t q_full = bars;
  auto kv_full = [&](int s) { return bars + 8u * (1 + s); };
  auto kv_empty = [&](int s) { return bars + 8u * (1 + KV_STAGES + s); };
  auto s_full = [&](int g) { return bars + 8u * (1 + 2 * KV_STAGES + g); };
  auto s_empty = [&](int g) { return bars + 8u * (3 + 2 * KV_STAGES + g); };
  auto p_full = [&](int g) { return bars + 8u * (5 + 2 * KV_STAGES + g); };
  auto pv_done = [&](int g) { return bars + 8u * (7 + 2 * KV_STAGES + g); };
  auto xch_bar_of = [&](int g, int lg) { return bars + 8u * (9 + 2 * KV_STAGES + g * 4 + lg); };
  const uint32_t fin_bar = bars + 8u * (17 + 2 * KV_STAGES);
  const uint32_t tmem_slot = bars + 8u * (18 + 2 * KV_STAGES);
  static_assert(8 * (19 + 2 * KV_STAGES) <= 256, "the barriers fit in front of the exchange area");
  const uint32_t xch = bars + 256;
  const uint32_t fin = xch + XCH_BYTES;
  uint8_t *smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
  volatile uint32_t *tmem_slot_ptr = reinterpret_cast<volatile uint32_t *>(
      smem_aligned + TILE_BYTES + KV_STAGES * 2 * TILE_BYTES + 8 * (18 + 2 * KV_STAGES));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int head = blockIdx.y;
  const int q0 = blockIdx.x * BQ;
  const int head_row0 = head * p.n_ctx;
  const int num_blocks = (p.n_ctx + BKV - 1) / BKV;
  const int n_a = (num_blocks + 1) / 2, n_b = num_blocks / 2;   // blocks of group 0 / group 1
  auto block_of = [&](int g, int jl) { return g ? n_a + jl : jl; };

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(kv_full(s), 1);
      mbar_init(kv_empty(s), 1);
    }
    for (int g = 0; g < 2; ++g) {
      mbar_init(s_full(g), 1);
      mbar_init(s_empty(g), 8);   // lane 0 of each of the group's softmax warps
      mbar_init(p_full(g), 8);
      mbar_init(pv_done(g), 1);
      for (int lg = 0; lg < 4; ++lg) mbar_init(xch_bar_of(g, lg), 2);   // the two warps that share rows
    }
    mbar_init(fin_bar, 16);
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

  // K/V stages: two per group (stage 2 g + (jl & 1) holds the group's block jl), so that a group
  // that runs ahead never waits for a stage the other group still holds.
  auto stage_of = [&](int g, int jl) { return 2 * g + (jl & 1); };
  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    // serves whichever group has a free stage; sleeps when neither has
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_q) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_k) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_v) : "memory");
      mbar_expect_tx(q_full, TILE_BYTES);
      tma_load_3d(q_smem, &tmap_q, 0, q0, head, q_full);
      int next[2] = {0, 0};
      const int n_of[2] = {n_a, n_b};
      long long idle_since = 0;
      while (next[0] < n_a || next[1] < n_b) {
        bool progressed = false;
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          const int jl = next[g];
          if (jl >= n_of[g]) continue;
          const int s = stage_of(g, jl);
          if (!mbar_try_wait(kv_empty(s), ((jl >> 1) & 1) ^ 1u)) continue;
          const int row = block_of(g, jl) * BKV;
          mbar_expect_tx(kv_full(s), 2 * TILE_BYTES);
          tma_load_3d(k_smem(s), &tmap_k, 0, row, head, kv_full(s));
          tma_load_3d(v_smem(s), &tmap_v, 0, row, head, kv_full(s));
          next[g] = jl + 1;
          progressed = true;
        }
        if (progressed) {
          idle_since = 0;
        } else {
          if (idle_since == 0) idle_since = clock64();
          else if (clock64() - idle_since > WAIT_LIMIT_CYCLES) {
            report(p.status, kStatusTmaWaitTimeout);
            break;
          }
          __nanosleep(kPollSleepNs);
        }
      }
      // every tile this thread asked for has been consumed before the CTA may go
#pragma unroll
      for (int g = 0; g < 2; ++g)
        for (int jl = next[g]; jl < next[g] + 2 && next[g] >= 2; ++jl)
          if (!mbar_wait_relaxed(kv_empty(stage_of(g, jl)), ((jl >> 1) & 1) ^ 1u, kPollSleepNs)) break;
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    // serves whichever group has handed over P (then O_g += P V) or is owed the scores of its
    // next block; never blocks on one group while the other could go on
    if (lane == 0) {
      bool ok = mbar_wait_relaxed(q_full, 0, kPollSleepNs);
      const uint64_t q_desc = make_smem_desc(q_smem, 16, 1024);
      const int n_of[2] = {n_a, n_b};
      int next_s[2] = {0, 0};    // next block whose S is to be issued
      int next_pv[2] = {0, 0};   // next block whose P V is to be issued
      long long idle_since = 0;
      while (ok && (next_pv[0] < n_a || next_pv[1] < n_b)) {
        bool progressed = false;
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          // S of block jl: its K tile has landed and the group has taken the previous scores out
          int jl = next_s[g];
          if (jl < n_of[g]) {
            const int s = stage_of(g, jl);
            if (mbar_try_wait(kv_full(s), (jl >> 1) & 1) && (jl == 0 || mbar_try_wait(s_empty(g), (jl - 1) & 1))) {
              tcgen05_fence_after();
              const uint64_t kd = make_smem_desc(k_smem(s), 16, 1024);
#pragma unroll
              for (int k = 0; k < DH / 16; ++k)
                tcgen05_mma_f16(tmem_base + g * BKV, q_desc + 2 * k, kd + 2 * k, p.idesc_s, k ? 1u : 0u);
              tcgen05_commit(s_full(g));
              next_s[g] = jl + 1;
              progressed = true;
            }
          }
          // P V of block jl: the group has handed over P
          jl = next_pv[g];
          if (jl < n_of[g] && jl < next_s[g] && mbar_try_wait(p_full(g), jl & 1)) {
            const int s = stage_of(g, jl);
            tcgen05_fence_after();
            const uint64_t vd = make_smem_desc(v_smem(s), TILE_BYTES, 1024);
#pragma unroll
            for (int k = 0; k < BKV / 16; ++k)
              tcgen05_mma_f16_a_tmem(tmem_base + PV_COL + g * DH, tmem_base + P_COL + g * (BKV / 2) + k * 8,
                                     vd + k * 128, p.idesc_pv, (jl | k) ? 1u : 0u);   // the group's first one starts O_g
            tcgen05_commit(pv_done(g));    // P buffer and O_g may be touched again, this K/V stage is free
            tcgen05_commit(kv_empty(s));
            next_pv[g] = jl + 1;
            progressed = true;
          }
        }
        if (progressed) {
          idle_since = 0;
        } else {
          if (idle_since == 0) idle_since = clock64();
          else if (clock64() - idle_since > WAIT_LIMIT_CYCLES) ok = false;
          __nanosleep(kPollSleepNs);
        }
      }
      if (!ok) report(p.status, kStatusMmaWaitTimeout);
    }
  } else {
    // ------------------------------------------------------------ softmax + output
    const int grp = (warp - 2) >> 3;                 // which group of key blocks
    const int lane_group = warp & 3;                 // TMEM lanes 32 * (warp % 4) ...
    const int part = ((warp - 2) & 7) >> 2;          // which 64 of a block's 128 keys
    const int r = lane_group * 32 + lane;            // row of the tile = TMEM lane
    constexpr int HC = BKV / 2;                      // keys per thread and block (64)
    const int n_mine = grp ? n_b : n_a;
    const uint32_t t_row = tmem_base + (static_cast<uint32_t>(lane_group * 32) << 16);
    const uint32_t s_addr = t_row + grp * BKV + part * HC;
    const uint32_t p_addr = t_row + P_COL + grp * (BKV / 2) + part * (HC / 2);
    const uint32_t o_addr = t_row + PV_COL + grp * DH;
    const uint32_t xch_bar = xch_bar_of(grp, lane_group);
    // partial maxima of the two threads of a row meet here: xch[parity][group * 2 + part][row]
    auto xch_addr = [&](int parity, int prt) {
      return xch + static_cast<uint32_t>(((parity * 4 + grp * 2 + prt) * BQ + r) * 4);
    };
    float m = -INFINITY, l = 0.0f;   // m: the reference maximum the exponents are taken against
    const float neg_inf = -INFINITY;
    bool ok = true;
    for (int jl = 0; jl < n_mine && ok; ++jl) {
      const int j = block_of(grp, jl);
      bool w = mbar_wait(s_full(grp), jl & 1);
      w = __all_sync(0xffffffffu, w);
      if (!w) { ok = false; break; }
      tcgen05_fence_after();
      uint32_t sc[HC];
      {
        uint32_t lo[32], hi[32];
        tmem_ld_32x32(s_addr, lo);
        tmem_ld_32x32(s_addr + 32, hi);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) { sc[i] = lo[i]; sc[32 + i] = hi[i]; }
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_empty(grp));   // the scores are in registers: S of the next block may come
      const int valid = p.n_ctx - j * BKV - part * HC;   // this thread's keys that exist (>= HC: all)
      const bool plain = valid >= HC && p.scale_log2e > 0.0f;
      float mx;
      if (plain) {
        float a = neg_inf, c = neg_inf;
#pragma unroll
        for (int i = 0; i < HC; i += 4) {
          a = max3(a, __uint_as_float(sc[i]), __uint_as_float(sc[i + 1]));
          c = max3(c, __uint_as_float(sc[i + 2]), __uint_as_float(sc[i + 3]));
        }
        mx = fmaxf(a, c) * p.scale_log2e;
      } else {
        mx = neg_inf;
#pragma unroll
        for (int i = 0; i < HC; ++i) mx = fmaxf(mx, (i < valid) ? __uint_as_float(sc[i]) * p.scale_log2e : neg_inf);
      }
      // the other thread of the row
      st_shared_f32(xch_addr(jl & 1, part), mx);
      __syncwarp();
      if (lane == 0) mbar_arrive(xch_bar);
      w = mbar_wait(xch_bar, jl & 1);
      w = __all_sync(0xffffffffu, w);
      if (!w) { ok = false; break; }
      const float row_max = fmaxf(mx, ld_shared_f32(xch_addr(jl & 1, part ^ 1)));
      // P buffer and O_g are free once P V of the previous block has been added
      if (jl > 0) {
        w = mbar_wait(pv_done(grp), (jl - 1) & 1);
        w = __all_sync(0xffffffffu, w);
        if (!w) { ok = false; break; }
        tcgen05_fence_after();
      }
      if (jl == 0) {
        m = row_max;
      } else {
        // the reference maximum stays while the row's maximum is within 2^8 of it
        const bool move = row_max > m + 8.0f;
        if (__any_sync(0xffffffffu, move)) {
          const float a = move ? ex2(m - row_max) : 1.0f;
#pragma unroll
          for (int c = 0; c < 2; ++c) {   // this thread's 32 columns of O_g, 16 at a time
            uint32_t v[16];
            tmem_ld_cols<16>(o_addr + part * 32 + c * 16, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * a);
            tmem_st_16cols(o_addr + part * 32 + c * 16, v);
          }
          tmem_st_wait();
          l *= a;
          if (move) m = row_max;
        }
      }
      // p = 2^(s' - m), 16 keys at a time into TMEM
      const uint64_t scale2 = pack_f32x2(p.scale_log2e, p.scale_log2e);
      const uint64_t neg_m2 = pack_f32x2(-m, -m);
      uint64_t sum2 = 0ull;
#pragma unroll
      for (int q = 0; q < HC / 16; ++q) {
        uint32_t pw[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float x0, x1;
          unpack_f32x2(fma_f32x2(pack_u32x2(sc[16 * q + 2 * i], sc[16 * q + 2 * i + 1]), scale2, neg_m2), x0, x1);
          float e0 = ex2(x0), e1 = ex2(x1);
          if (!plain) {
            e0 = (16 * q + 2 * i < valid) ? e0 : 0.0f;
            e1 = (16 * q + 2 * i + 1 < valid) ? e1 : 0.0f;
          }
          sum2 = add_f32x2(sum2, pack_f32x2(e0, e1));
          pw[i] = pack2(e0, e1, BF16);
        }
        tmem_st_8cols(p_addr + 8 * q, pw);
      }
      tmem_st_wait();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full(grp));
      float s_lo, s_hi;
      unpack_f32x2(sum2, s_lo, s_hi);
      l += s_lo + s_hi;
    }
    // O_g is complete when the group's last P V has been added
    if (ok && n_mine > 0) {
      bool w = mbar_wait(pv_done(grp), (n_mine - 1) & 1);
      ok = __all_sync(0xffffffffu, w);
    }
    // merge: every thread of the row learns both groups' (m, l)
    {
      const uint32_t mine = fin + static_cast<uint32_t>((((grp * 2 + part) * BQ) + r) * 8);
      st_shared_f32(mine, m);
      st_shared_f32(mine + 4, l);
      __syncwarp();
      if (lane == 0) mbar_arrive(fin_bar);
      bool w = ok && mbar_wait(fin_bar, 0);
      ok = __all_sync(0xffffffffu, w);
    }
    if (!ok) {
      if (lane == 0) report(p.status, kStatusEpiWaitTimeout);
    } else {
      tcgen05_fence_after();
      auto fin_at = [&](int g, int prt, int which) {
        return ld_shared_f32(fin + static_cast<uint32_t>((((g * 2 + prt) * BQ) + r) * 8 + which * 4));
      };
      const float m0 = fin_at(0, 0, 0), l0 = fin_at(0, 0, 1) + fin_at(0, 1, 1);
      const float m1 = n_b > 0 ? fin_at(1, 0, 0) : neg_inf;
      const float l1 = n_b > 0 ? fin_at(1, 0, 1) + fin_at(1, 1, 1) : 0.0f;
      const float mm = fmaxf(m0, m1);
      const float a0 = ex2(m0 - mm), a1 = n_b > 0 ? ex2(m1 - mm) : 0.0f;
      const float inv = 1.0f / fmaf(l0, a0, l1 * a1);
      // this thread's 16 of the 64 output columns
      const int c0 = (grp * 2 + part) * 16;
      uint32_t v0[16], v1[16];
      tmem_ld_cols<16>(t_row + PV_COL + c0, v0);
      if (n_b > 0) tmem_ld_cols<16>(t_row + PV_COL + DH + c0, v1);
      tmem_ld_wait();
      if (q0 + r < p.n_ctx) {
        float o[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float x = __uint_as_float(v0[i]) * a0;
          if (n_b > 0) x = fmaf(__uint_as_float(v1[i]), a1, x);
          o[i] = x * inv;
        }
        uint16_t *orow = static_cast<uint16_t *>(p.O) + static_cast<size_t>(head_row0 + q0 + r) * DH + c0;
#pragma unroll
        for (int c = 0; c < 16; c += 8) {
          const uint4 out = make_uint4(pack2(o[c], o[c + 1], BF16), pack2(o[c + 2], o[c + 3], BF16),
                                       pack2(o[c + 4], o[c + 5], BF16), pack2(o[c + 6], o[c + 7], BF16));
          *reinterpret_cast<uint4 *>(orow + c) = out;
        }
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
  static bool with_stats = false;
  using Kernel = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const AttnParams);
  // [stats][bf16]
  static const Kernel kernels[2][2] = {
      {flash_attention_fwd_kernel<4, false, false>, flash_attention_fwd_kernel<4, false, true>},
      {flash_attention_fwd_kernel<4, true, false>, flash_attention_fwd_kernel<4, true, true>}};
  std::call_once(once, [] {
    with_stats = getenv("IMEX_ATTN_STATS") != nullptr;  // development aid: where the roles wait
    for (int i = 0; i < 4; ++i) {
      cudaError_t x = cudaFuncSetAttribute(kernels[i >> 1][i & 1], cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           SMEM_BYTES);
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
    if (!stats_buf) cudaMallocManaged(&stats_buf, 24 * 4096 * sizeof(long long));
    p.stats = stats_buf;
  }
  // IMEX_ATTN_KERNEL=pipelined: one group of softmax warps, software-pipelined over the blocks;
  // default: two groups half a period apart
  static const bool one_group = getenv("IMEX_ATTN_KERNEL") && std::string(getenv("IMEX_ATTN_KERNEL")) == "pipelined";
  if (one_group || p.stats) {
    kernels[p.stats ? 1 : 0][dtype == kBF16 ? 1 : 0]<<<grid, num_threads(4), SMEM_BYTES, stream>>>(tq, tk, tv, p);
  } else {
    static std::once_flag pp_once;
    static cudaError_t pp_err = cudaSuccess;
    std::call_once(pp_once, [] {
      cudaError_t a = cudaFuncSetAttribute(flash_attention_fwd_pp_kernel<false>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, PP_SMEM_BYTES);
      cudaError_t b = cudaFuncSetAttribute(flash_attention_fwd_pp_kernel<true>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, PP_SMEM_BYTES);
      pp_err = a != cudaSuccess ? a : b;
    });
    if (pp_err != cudaSuccess) return pp_err;
    if (dtype == kBF16)
      flash_attention_fwd_pp_kernel<true><<<grid, num_threads(4), PP_SMEM_BYTES, stream>>>(tq, tk, tv, p);
    else
      flash_attention_fwd_pp_kernel<false><<<grid, num_threads(4), PP_SMEM_BYTES, stream>>>(tq, tk, tv, p);
  }
  if (p.stats) {
    cudaStreamSynchronize(stream);
    double a[24] = {0};
    for (int c = 0; c < ctas; ++c)
      for (int i = 0; i < 24; ++i) a[i] += static_cast<double>(stats_buf[24 * c + i]);
    for (double &x : a) x /= ctas;
    fprintf(stderr,
            "[attention stats, mean cycles per CTA, %d key blocks] mma total %.0f wait_kv %.0f wait_s_free %.0f "
            "wait_p %.0f wait_pv_free %.0f issue_s %.0f issue_pv %.0f | softmax total %.0f wait_s %.0f | softmax phases: exp_a %.0f "
            "get_s %.0f exp_b %.0f store_p %.0f max_post %.0f wait_pv %.0f fold_pv %.0f collect %.0f\n",
            static_cast<int>((n_ctx + BKV - 1) / BKV), a[0], a[1], a[2], a[3], a[4], a[7], a[16], a[5], a[6], a[8], a[9], a[10],
            a[11], a[12], a[13], a[14], a[15]);
  }
  return cudaGetLastError();
}

} // namespace imex
