// Attention forward, O = softmax(sm_scale * Q K^T) V, one pass over K and V with the
// running-max / running-sum recurrence, on the 5th-generation tensor cores.
//
// Reference: test/Integration/Dialect/XeGPU/WG/flash_attention_fwd.mlir (gpu_impl :254-330,
// the per-tile recurrence :111-250, and the CPU check :334-432 that the oracle restates):
// Q, K, V, O are [heads * n_ctx, 64] 16-bit arrays, heads one after the other.
//
// One CTA per (head, block of 128 query rows).  Its key blocks (128 keys each) are shared out
// between TWO groups of softmax warps that work half a period apart (group 0: blocks
// [0, nA), group 1: blocks [nA, nb)).  While one group runs its exponentials the other fetches
// scores, takes maxima and hands P over, so the special-function unit and the tensor core see
// work from one group or the other all the time, which a single group in lock step cannot
// give them.  Each group keeps its own reference maxima, sums and its own O accumulator in
// TMEM; the two are merged at the end (O = (O_0 a_0 + O_1 a_1) / (l_0 a_0 + l_1 a_1) with
// a_g = 2^(m_g - max(m_0, m_1))).
//
//   warp 0      TMA producer: Q once, then K/V tiles into two stages per group, whichever
//               group has a free stage (all tiles are 128 rows x 64 d = one 128B-swizzled box
//               of a 3-D tensor map whose outer dimension is the head, so a ragged last tile
//               is filled with zeros, never with the next head's rows).
//   warp 1      one thread issues tcgen05.mma, serving whichever group is ready: S_g = Q K^T
//               of a group's next block (M128 N128 K64, both operands K-major in shared
//               memory) as soon as its threads hold the previous scores in registers (one S
//               buffer per group), O_g += P V (M128 N64 K128; P as the A operand from TMEM, V
//               MN-major exactly as it lies in its tile) as soon as the group has handed over P.
//   warps 2-17  group g = (warp - 2) / 8: two threads per query row, 64 keys each; the scores
//               come from TMEM (tcgen05.ld), the two partial row maxima meet through shared
//               memory, P goes back into TMEM as 16-bit pairs (tcgen05.st).  The reference
//               maximum of a row moves only when the row's maximum outgrows it by more than
//               2^8; only then are O_g (in TMEM) and the running sum rescaled.  No shuffles.
// TMEM: S_0 [0,128) S_1 [128,256) O_0 [256,320) O_1 [320,384) P_0 [384,448) P_1 [448,512).
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
constexpr int KV_STAGES = 4;  // two per group; 150 KB of shared memory: one CTA per SM, which owns all 512 TMEM columns
constexpr int TILE_BYTES = 128 * DH * 2;        // 16 KB: any of the Q / K / V tiles
// threads: producer warp, MMA warp, 16 softmax warps
constexpr int num_threads(int split) { return 64 + 128 * split; }
constexpr int TMEM_COLS = 512;  // S_0 [0,128) S_1 [128,256) O_0 [256,320) O_1 [320,384) P_0 [384,448) P_1 [448,512)
constexpr int PV_COL = 256;
// the producer and the MMA thread sleep between polls of a barrier: a spinning warp takes issue
// slots from the softmax warps of its scheduler, and neither is on the critical path
constexpr unsigned kPollSleepNs = 40;
constexpr int P_COL = 384;      // P as the A operand of P.V: 128 keys = 64 columns of two 16-bit values
constexpr int XCH_BYTES = 2 * 4 * BQ * 4;           // partial row maxima of the two threads of a row, double buffered
constexpr int FIN_BYTES = 2 * 2 * BQ * 8;           // (m, l) of every group / part / row for the merge
constexpr int SMEM_BYTES = TILE_BYTES + KV_STAGES * 2 * TILE_BYTES + 1024 + 256 + XCH_BYTES + FIN_BYTES;

struct AttnParams {
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
template <> __device__ __forceinline__ void tmem_ld_cols<16>(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}


template <bool BF16>
__global__ void __launch_bounds__(num_threads(4), 1)
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
  std::call_once(once, [] {
    cudaError_t a = cudaFuncSetAttribute(flash_attention_fwd_kernel<false>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    cudaError_t b = cudaFuncSetAttribute(flash_attention_fwd_kernel<true>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    attr_err = a != cudaSuccess ? a : b;
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
  if (dtype == kBF16)
    flash_attention_fwd_kernel<true><<<grid, num_threads(4), SMEM_BYTES, stream>>>(tq, tk, tv, p);
  else
    flash_attention_fwd_kernel<false><<<grid, num_threads(4), SMEM_BYTES, stream>>>(tq, tk, tv, p);
  return cudaGetLastError();
}

} // namespace imex
