// bf16/f16 -> f32 GEMM on the 5th-generation tensor cores of sm_100a, with
// the bias / relu / silu epilogue fused.
//
// Reference op: linalg.matmul, C = C0 + A.B with A[M,K], B[K,N] row-major
// 16-bit and an f32 accumulator (test/SPIRV/OpTest.GEMM_BF16_ACC_F32.mlir:126-141,
// test/PlaidML/CppEdsl.DotF16_AccF32.mlir:19-47); epilogues are the relu and
// silu generics (benchmarks/relu/relu_gpu.mlir.in:6-11,
// benchmarks/silu/silu_gpu.mlir.in:6-18); bias is the row-vector add of
// test/Integration/Dialect/XeGPU/WG/gemm_4kx4kx4k_f16_f16_f32_bias.mlir:91-113.
// The reference's GPU lowering of this op is one work-group per C element
// with a scalar k loop; its tuned Xe kernels tile 256x256 per work-group with
// DPAS.  Nothing of either is reused here.
//
// Structure (one CTA per SM, persistent over 128x256 output tiles):
//   warp 0      TMA producer: cp.async.bulk.tensor loads of the A tile
//               (128 x 64, K-major) and the B tile (64 x 256, N-major, as four
//               64x64 boxes) into a 4-stage 128B-swizzled smem ring, completion
//               on mbarriers (expect-tx).  No cluster multicast.
//   warp 1      allocates 512 TMEM columns (two 128x256 f32 accumulators) and
//               issues tcgen05.mma.cta_group::1.kind::f16 (M128 N256 K16) from
//               one thread; tcgen05.commit releases smem stages and publishes
//               finished accumulators.
//   warps 2-5   epilogue: tcgen05.ld the accumulator (32 lanes x 32 columns per
//               warp and step), add C0 / bias, apply relu or silu, store f32 with
//               128-bit stores.  Runs on accumulator i while the MMA warp fills
//               accumulator i^1.
// Every wait is bounded: when one runs out the warp records a status code in
// the host-visible status word and leaves its loop; the kernel still drains
// its loads, frees TMEM and returns.
#include "epilogue.cuh"
#include "tcgen05_ptx.cuh"
#include "tcgen05_host.h"

#include <cuda.h>
#include <cuda_bf16.h>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <mutex>
#include <tuple>

namespace imex {
namespace {

constexpr int BM = 128;        // tile rows   (UMMA M)
constexpr int BN = 256;        // tile cols   (UMMA N)
constexpr int BK = 64;         // k per stage (one 128-byte swizzle row of 16-bit elements)
constexpr int UMMA_K = 16;     // k per tcgen05.mma for 16-bit inputs
constexpr int STAGES = 4;
constexpr int NUM_ACC = 2;     // TMEM accumulators (2 x 256 columns)
constexpr int TMEM_COLS = 512;
constexpr int A_STAGE_BYTES = BM * BK * 2;   // 16 KB
constexpr int B_STAGE_BYTES = BK * BN * 2;   // 32 KB
constexpr int B_BOX_BYTES = BK * 64 * 2;     // one 64(k) x 64(n) box = 8 KB
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int NUM_THREADS = 192;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;

struct KernelParams {
  float *C;
  const float *bias;
  unsigned *status;
  int M, N, K;
  long long ldc;
  int tiles_m, tiles_n, num_tiles, group_m;
  int k_blocks;
  int epilogue;
  int accumulate;
  uint32_t idesc;
};

using namespace tc;
using namespace tc_host;

// Tile order: bands of `group_m` row-blocks; inside a band the column-block
// index moves slowest, so the CTAs in flight share a band of A and a few
// column-blocks of B through L2.
__device__ __forceinline__ void tile_coords(int tile, const KernelParams &p, int &mb, int &nb) {
  const int band_tiles = p.group_m * p.tiles_n;
  const int band = tile / band_tiles;
  const int first_m = band * p.group_m;
  const int rows_in_band = min(p.group_m, p.tiles_m - first_m);
  const int t = tile - band * band_tiles;
  nb = t / rows_in_band;
  mb = first_m + t % rows_in_band;
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a,
                    const __grid_constant__ CUtensorMap tmap_b, const KernelParams p) {
  extern __shared__ uint8_t smem_raw[];
  // 128B-swizzled tiles need 1024-byte aligned bases
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bars = smem_base + STAGES * STAGE_BYTES;
  // barrier layout (8 bytes each): full[STAGES], empty[STAGES], acc_full[2], acc_empty[2], tmem slot
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
  auto acc_full_bar = [&](int a) { return bars + 8u * (2 * STAGES + a); };
  auto acc_empty_bar = [&](int a) { return bars + 8u * (2 * STAGES + NUM_ACC + a); };
  const uint32_t tmem_slot = bars + 8u * (2 * STAGES + 2 * NUM_ACC);
  uint8_t *smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
  volatile uint32_t *tmem_slot_ptr =
      reinterpret_cast<volatile uint32_t *>(smem_aligned + STAGES * STAGE_BYTES +
                                            8 * (2 * STAGES + 2 * NUM_ACC));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < NUM_ACC; ++a) {
      mbar_init(acc_full_bar(a), 1);
      mbar_init(acc_empty_bar(a), 4);  // one arrival per epilogue warp
    }
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
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_a) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_b) : "memory");
      int stage = 0;
      uint32_t phase = 0;
      uint32_t armed = 0;         // stages whose full barrier was armed at least once
      uint32_t armed_parity = 0;  // phase parity of the latest arming, per stage
      bool ok = true;
      for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x) {
        int mb, nb;
        tile_coords(tile, p, mb, nb);
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u)) {
            report(p.status, kStatusTmaWaitTimeout);
            ok = false;
            break;
          }
          const uint32_t a_dst = smem_base + stage * STAGE_BYTES;
          const uint32_t b_dst = a_dst + A_STAGE_BYTES;
          mbar_expect_tx(full_bar(stage), STAGE_BYTES);
          armed |= 1u << stage;
          armed_parity = (armed_parity & ~(1u << stage)) | (phase << stage);
          tma_load_2d(a_dst, &tmap_a, kb * BK, mb * BM, full_bar(stage));
#pragma unroll
          for (int j = 0; j < BN / 64; ++j)
            tma_load_2d(b_dst + j * B_BOX_BYTES, &tmap_b, nb * BN + j * 64, kb * BK,
                        full_bar(stage));
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        // let the loads already in flight land before the CTA can exit
        for (int s = 0; s < STAGES; ++s)
          if (armed & (1u << s)) mbar_wait(full_bar(s), (armed_parity >> s) & 1u);
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x) {
        if (!mbar_wait(acc_empty_bar(acc), acc_phase ^ 1u)) {
          report(p.status, kStatusMmaWaitTimeout);
          break;
        }
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(full_bar(stage), phase)) {
            report(p.status, kStatusMmaWaitTimeout);
            ok = false;
            break;
          }
          tcgen05_fence_after();
          const uint32_t a_addr = smem_base + stage * STAGE_BYTES;
          const uint32_t b_addr = a_addr + A_STAGE_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // A (K-major): 8-row groups 1024 B apart; +32 B per 16 k inside the swizzle row.
            // B (N-major): 8-k groups 1024 B apart (SBO), 64-column groups one box apart (LBO);
            //              +2048 B per 16 k.
            const uint64_t a_desc = make_smem_desc(a_addr + k * (UMMA_K * 2), 16, 1024);
            const uint64_t b_desc = make_smem_desc(b_addr + k * (UMMA_K * 128), B_BOX_BYTES, 1024);
            tcgen05_mma_f16(d_tmem, a_desc, b_desc, p.idesc, (kb | k) ? 1u : 0u);
          }
          tcgen05_commit(empty_bar(stage));  // smem stage reusable once these MMAs finish
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) tcgen05_commit(acc_full_bar(acc));  // accumulator ready for the epilogue
        if (++acc == NUM_ACC) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    // -------------------------------- epilogue --------------------------------
    const int lane_group = warp & 3;  // TMEM lanes this warp may read: 32*lane_group ..
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x) {
      int mb, nb;
      tile_coords(tile, p, mb, nb);
      bool ok = mbar_wait(acc_full_bar(acc), acc_phase);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) report(p.status, kStatusEpiWaitTimeout);
        break;
      }
      tcgen05_fence_after();
      const int row = mb * BM + lane_group * 32 + lane;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(lane_group * 32) << 16) + acc * BN;
      float *c_row = p.C + static_cast<size_t>(row) * p.ldc;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(t_row + c0, r);
        tmem_ld_wait();
        const int col0 = nb * BN + c0;
        if (row < p.M && col0 < p.N) {
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            const int col = col0 + j;
            if (col < p.N) {  // N % 8 == 0, so a group of 4 is inside or outside as a whole
              float4 v = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                     __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
              if (p.accumulate) {
                const float4 c = *reinterpret_cast<const float4 *>(c_row + col);
                v.x += c.x; v.y += c.y; v.z += c.z; v.w += c.w;
              }
              if (p.bias) {
                const float4 b = *reinterpret_cast<const float4 *>(p.bias + col);
                v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
              }
              v.x = apply_epilogue(v.x, p.epilogue);
              v.y = apply_epilogue(v.y, p.epilogue);
              v.z = apply_epilogue(v.z, p.epilogue);
              v.w = apply_epilogue(v.w, p.epilogue);
              *reinterpret_cast<float4 *>(c_row + col) = v;
            }
          }
        }
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty_bar(acc));
      if (++acc == NUM_ACC) { acc = 0; acc_phase ^= 1u; }
    }
  }

  __syncwarp();  // lanes of the producer / MMA warps rejoin their elected lane
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(TMEM_COLS)
                 : "memory");
  }
}

} // namespace

bool gemm_tcgen05_supported(const GemmProblem &p) {
  if (p.in_dtype != kBF16 && p.in_dtype != kF16) return false;
  if (p.trans_a || p.trans_b || p.out_dtype != kF32) return false;  // the pair kernel takes those
  if (p.M <= 0 || p.N <= 0 || p.K <= 0) return false;
  if (p.K % 8 || p.N % 8) return false;  // TMA row pitch must be a multiple of 16 bytes
  if (p.lda % 8 || p.ldb % 8 || p.ldc % 4) return false;
  if ((p.lda && p.lda < p.K) || (p.ldb && p.ldb < p.N) || (p.ldc && p.ldc < p.N)) return false;
  if (p.M > INT32_MAX || p.N > INT32_MAX || p.K > INT32_MAX) return false;
  auto al = [](const void *q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  return al(p.A) && al(p.B) && al(p.C) && (!p.bias || al(p.bias));
}

cudaError_t launch_gemm_tcgen05(const GemmProblem &g, unsigned *status, cudaStream_t stream) {
  if (!gemm_tcgen05_supported(g)) return cudaErrorInvalidValue;
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [] {
    attr_err = cudaFuncSetAttribute(gemm_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    SMEM_BYTES);
  });
  if (attr_err != cudaSuccess) return attr_err;

  CUtensorMap ta, tb;
  // cudaErrorNotSupported: the driver refused this shape for a tensor map; the
  // caller falls back to the SIMT kernel
  if (!make_map(&ta, g.A, g.in_dtype, g.K, g.M, BM, g.lda)) return cudaErrorNotSupported;
  if (!make_map(&tb, g.B, g.in_dtype, g.N, g.K, BK, g.ldb)) return cudaErrorNotSupported;

  KernelParams p;
  p.C = g.C;
  p.bias = g.bias;
  p.status = status;
  p.M = static_cast<int>(g.M);
  p.N = static_cast<int>(g.N);
  p.K = static_cast<int>(g.K);
  p.ldc = g.ldc > 0 ? g.ldc : g.N;
  p.tiles_m = (p.M + BM - 1) / BM;
  p.tiles_n = (p.N + BN - 1) / BN;
  p.num_tiles = p.tiles_m * p.tiles_n;
  p.group_m = 16;
  if (const char *e = getenv("IMEX_GEMM_GROUP_M")) {
    int v = atoi(e);
    if (v > 0) p.group_m = v;
  }
  p.k_blocks = (p.K + BK - 1) / BK;
  p.epilogue = g.epilogue;
  p.accumulate = g.accumulate ? 1 : 0;
  const uint32_t fmt = g.in_dtype == kBF16 ? 1u : 0u;
  // instruction descriptor: D f32, A/B format, A K-major, B N-major, N>>3, M>>4
  p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (0u << 15) | (1u << 16) |
            (static_cast<uint32_t>(BN >> 3) << 17) | (static_cast<uint32_t>(BM >> 4) << 24);

  int usable = sm_count() - (g.sm_margin > 0 ? g.sm_margin : 0);
  if (usable < 1) usable = 1;
  int grid = p.num_tiles < usable ? p.num_tiles : usable;
  gemm_tcgen05_kernel<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb, p);
  return cudaGetLastError();
}

} // namespace imex
