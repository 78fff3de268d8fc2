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
//   warps 2-9   two threads per query row (64 keys and 32 output columns each): read the
//               scores of S_j from TMEM once (tcgen05.ld), free the S buffer, exchange the
//               two partial row maxima through shared memory, keep m and a partial l,
//               write P_j as 16-bit values into shared memory in the swizzled K-major
//               layout the MMA expects, and fold PV_{j-1} into 32 f32 output registers
//               while the tensor core works on S_{j+1} and PV_j.  No shuffles.
// Every wait is bounded; a wait that runs out records a status code, the roles leave
// their loops, the CTA syncs and frees its TMEM.
#include "kernels.h"
#include "tcgen05_host.h"
#include "tcgen05_ptx.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <mutex>

namespace imex {
namespace {

using namespace tc;
using namespace tc_host;

constexpr int BQ = 128;        // query rows per CTA
constexpr int BKV = 128;       // keys per block
constexpr int DH = 64;         // head dimension
constexpr int KV_STAGES = 3;  // 144 KB of shared memory: one CTA per SM, which owns all 512 TMEM columns
constexpr int TILE_BYTES = 128 * DH * 2;        // 16 KB: any of the Q / K / V tiles
constexpr int P_BYTES = BQ * BKV * 2;           // 32 KB: two 128 x 64-key boxes
constexpr int NUM_THREADS = 320;  // producer warp, MMA warp, eight softmax warps
constexpr int TMEM_COLS = 512;                  // S0 [0,128) S1 [128,256) PV [256,320)
constexpr int PV_COL = 256;
constexpr int XCH_BYTES = 2 * 2 * BQ * 4;           // partial row maxima / sums of the two half-rows
constexpr int SMEM_BYTES = TILE_BYTES + KV_STAGES * 2 * TILE_BYTES + P_BYTES + 1024 + 256 + XCH_BYTES;

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

__global__ void __launch_bounds__(NUM_THREADS, 1)
flash_attention_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                           const __grid_constant__ CUtensorMap tmap_v, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_smem = smem_base;
  auto k_smem = [&](int s) { return smem_base + TILE_BYTES + s * 2 * TILE_BYTES; };
  auto v_smem = [&](int s) { return k_smem(s) + TILE_BYTES; };
  const uint32_t p_smem = smem_base + TILE_BYTES + KV_STAGES * 2 * TILE_BYTES;
  const uint32_t bars = p_smem + P_BYTES;
  const uint32_t q_full = bars;
  auto kv_full = [&](int s) { return bars + 8u * (1 + s); };
  auto kv_empty = [&](int s) { return bars + 8u * (1 + KV_STAGES + s); };
  auto s_full = [&](int b) { return bars + 8u * (1 + 2 * KV_STAGES + b); };
  auto s_empty = [&](int b) { return bars + 8u * (3 + 2 * KV_STAGES + b); };
  const uint32_t p_full = bars + 8u * (5 + 2 * KV_STAGES);
  const uint32_t pv_full = bars + 8u * (6 + 2 * KV_STAGES);
  const uint32_t pv_empty = bars + 8u * (7 + 2 * KV_STAGES);
  const uint32_t xch_bar = bars + 8u * (8 + 2 * KV_STAGES);
  const uint32_t tmem_slot = bars + 8u * (9 + 2 * KV_STAGES);
  const uint32_t xch = bars + 256;
  uint8_t *smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
  volatile uint32_t *tmem_slot_ptr = reinterpret_cast<volatile uint32_t *>(
      smem_aligned + TILE_BYTES + KV_STAGES * 2 * TILE_BYTES + P_BYTES + 8 * (9 + 2 * KV_STAGES));

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
      mbar_init(s_empty(b), 8);   // lane 0 of each softmax warp
    }
    mbar_init(p_full, 8);
    mbar_init(pv_full, 1);
    mbar_init(pv_empty, 8);
    mbar_init(xch_bar, 8);
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
      tma_load_2d(q_smem, &tmap_q, 0, head_row0 + q0, q_full);
      int filled = 0;
      for (int j = 0; j < num_blocks; ++j) {
        const int s = j % KV_STAGES;
        if (!mbar_wait(kv_empty(s), ((j / KV_STAGES) & 1) ^ 1u)) {
          report(p.status, kStatusTmaWaitTimeout);
          break;
        }
        mbar_expect_tx(kv_full(s), 2 * TILE_BYTES);
        tma_load_2d(k_smem(s), &tmap_k, 0, head_row0 + j * BKV, kv_full(s));
        tma_load_2d(v_smem(s), &tmap_v, 0, head_row0 + j * BKV, kv_full(s));
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
      bool ok = mbar_wait(q_full, 0);
      if (!ok) report(p.status, kStatusMmaWaitTimeout);
      auto issue_s = [&](int j) -> bool {
        const int s = j % KV_STAGES, b = j & 1;
        if (!mbar_wait(kv_full(s), (j / KV_STAGES) & 1)) return false;
        if (!mbar_wait(s_empty(b), ((j >> 1) & 1) ^ 1u)) return false;
        tcgen05_fence_after();
#pragma unroll
        for (int k = 0; k < DH / 16; ++k)
          tcgen05_mma_f16(tmem_base + b * BKV, make_smem_desc(q_smem + k * 32, 16, 1024),
                          make_smem_desc(k_smem(s) + k * 32, 16, 1024), p.idesc_s, k ? 1u : 0u);
        tcgen05_commit(s_full(b));
        return true;
      };
      auto issue_pv = [&](int j) -> bool {
        const int s = j % KV_STAGES;
        if (!mbar_wait(p_full, j & 1)) return false;
        if (!mbar_wait(pv_empty, (j & 1) ^ 1u)) return false;
        tcgen05_fence_after();
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k)
          tcgen05_mma_f16(tmem_base + PV_COL,
                          make_smem_desc(p_smem + (k >> 2) * TILE_BYTES + (k & 3) * 32, 16, 1024),
                          make_smem_desc(v_smem(s) + k * 2048, TILE_BYTES, 1024), p.idesc_pv, k ? 1u : 0u);
        tcgen05_commit(pv_full);      // PV_j is complete: P and this K/V stage are free again
        tcgen05_commit(kv_empty(s));
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; j < num_blocks && ok; ++j) {
        if (j + 1 < num_blocks) ok = issue_s(j + 1);
        if (ok) ok = issue_pv(j);
      }
      if (!ok) report(p.status, kStatusMmaWaitTimeout);
    }
  } else {
    // ------------------------------------------------------------ softmax + output
    // Two threads per query row: warps 2-5 take keys 0-63 of every block and output
    // columns 0-31, warps 6-9 keys 64-127 and columns 32-63 (a warp reaches the TMEM
    // lanes 32 * (warp % 4) ..., so warps w and w + 4 see the same rows).  The two halves
    // of a row exchange their partial maxima through shared memory once per block.
    const int lane_group = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = lane_group * 32 + lane;                       // row of the tile = TMEM lane
    const uint32_t t_row = tmem_base + (static_cast<uint32_t>(lane_group * 32) << 16);
    const uint32_t p_row = p_smem + half * TILE_BYTES + r * 128; // box `half` holds this thread's keys
    const uint32_t swz = static_cast<uint32_t>(r & 7);
    constexpr int HC = BKV / 2;   // keys per thread and block
    constexpr int HO = DH / 2;    // output columns per thread
    float o[HO];
#pragma unroll
    for (int i = 0; i < HO; ++i) o[i] = 0.0f;
    float m = -INFINITY, l = 0.0f, alpha_prev = 0.0f;
    const float neg_inf = -INFINITY;
    bool ok = true;
    // partial results of the two halves of a row meet here: xch[parity][half][row]
    auto xch_addr = [&](int parity, int h) { return xch + static_cast<uint32_t>(((parity * 2 + h) * BQ + r) * 4); };
    auto exchange = [&](int round, float mine, float &other) -> bool {
      st_shared_f32(xch_addr(round & 1, half), mine);
      __syncwarp();
      if (lane == 0) mbar_arrive(xch_bar);
      bool w = mbar_wait(xch_bar, round & 1);
      w = __all_sync(0xffffffffu, w);
      if (!w) return false;
      other = ld_shared_f32(xch_addr(round & 1, half ^ 1));
      return true;
    };
    auto fold_pv = [&](int j, float alpha) -> bool {
      // O = O * alpha + PV_j (this thread's 32 columns)
      bool w = mbar_wait(pv_full, j & 1);
      w = __all_sync(0xffffffffu, w);
      if (!w) return false;
      tcgen05_fence_after();
      uint32_t v[32];
      tmem_ld_32x32(t_row + PV_COL + half * HO, v);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < HO; ++i) o[i] = fmaf(o[i], alpha, __uint_as_float(v[i]));
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(pv_empty);
      return true;
    };
    for (int j = 0; j < num_blocks; ++j) {
      const int b = j & 1;
      bool w = mbar_wait(s_full(b), (j >> 1) & 1);
      w = __all_sync(0xffffffffu, w);
      if (!w) { ok = false; break; }
      tcgen05_fence_after();
      // this thread's 64 scores, read once; the S buffer is free again right away
      uint32_t sc[HC];
      {
        uint32_t lo[32], hi[32];
        tmem_ld_32x32(t_row + b * BKV + half * HC, lo);
        tmem_ld_32x32(t_row + b * BKV + half * HC + 32, hi);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) { sc[i] = lo[i]; sc[32 + i] = hi[i]; }
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_empty(b));
      const int valid = p.n_ctx - j * BKV - half * HC;  // this thread's keys that exist (>= 64: all)
      float mx = neg_inf;   // in units of log2: s * sm_scale * log2 e
#pragma unroll
      for (int i = 0; i < HC; ++i) mx = fmaxf(mx, (i < valid) ? __uint_as_float(sc[i]) * p.scale_log2e : neg_inf);
      float other;
      if (!exchange(j, mx, other)) { ok = false; break; }
      const float m_new = fmaxf(m, fmaxf(mx, other));
      const float alpha = ex2(m - m_new);  // 0 on the first block (m = -inf)
      // the previous block's P.V: its completion also frees the P buffer
      if (j > 0) {
        if (!fold_pv(j - 1, alpha_prev)) { ok = false; break; }
      }
      // p = 2^(s' - m_new), rounded to 16 bits into the swizzled K-major P tile
      float rowsum = 0.0f;
#pragma unroll
      for (int q = 0; q < HC / 8; ++q) {  // 16-byte chunks of 8 keys
        float e[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float pe = ex2(fmaf(__uint_as_float(sc[8 * q + i]), p.scale_log2e, -m_new));
          e[i] = (8 * q + i < valid) ? pe : 0.0f;
          rowsum += e[i];
        }
        st_shared_v4_u32(p_row + ((static_cast<uint32_t>(q) ^ swz) << 4), pack2(e[0], e[1], p.is_bf16),
                         pack2(e[2], e[3], p.is_bf16), pack2(e[4], e[5], p.is_bf16),
                         pack2(e[6], e[7], p.is_bf16));
      }
      l = fmaf(l, alpha, rowsum);
      m = m_new;
      alpha_prev = alpha;
      fence_async_smem();  // P (generic-proxy stores) visible to the tensor core's reads
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    if (ok && num_blocks > 0) ok = fold_pv(num_blocks - 1, alpha_prev);
    float l_other = 0.0f;
    if (ok) ok = exchange(num_blocks, l, l_other);
    if (!ok) {
      if (lane == 0) report(p.status, kStatusEpiWaitTimeout);
    } else if (q0 + r < p.n_ctx) {
      const float inv = 1.0f / (l + l_other);
      uint16_t *orow = static_cast<uint16_t *>(p.O) + static_cast<size_t>(head_row0 + q0 + r) * DH + half * HO;
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
  std::call_once(once, [] {
    attr_err = cudaFuncSetAttribute(flash_attention_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    SMEM_BYTES);
  });
  if (attr_err != cudaSuccess) return attr_err;
  const int64_t rows = heads * n_ctx;
  CUtensorMap tq, tk, tv;
  if (!make_map(&tq, q, dtype, DH, rows, BQ) || !make_map(&tk, k, dtype, DH, rows, BKV) ||
      !make_map(&tv, v, dtype, DH, rows, BKV))
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
  flash_attention_fwd_kernel<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(tq, tk, tv, p);
  return cudaGetLastError();
}

} // namespace imex
