// bf16/f16 -> f32 GEMM on CTA pairs: tcgen05.mma.cta_group::2 (M256 N256 K16).
//
// Same op, epilogues and reference citations as gemm_tcgen05.cu.  Two CTAs of a
// 2-CTA cluster share one 256x256 output tile: CTA r owns rows [128r, 128r+128)
// of it (its own 128-lane TMEM accumulator, double buffered: 2 x 256 columns)
// and loads, per k block of BKT elements, its own 128 x BKT slice of A and HALF
// of the B block (BKT x 128 columns).  The pair's tensor cores read both halves
// of B from both CTAs' shared memory, so every byte of B is fetched from L2
// once per pair instead of once per CTA.  There is no TMA multicast: each CTA
// issues plain tile loads into its own shared memory; only the completion
// barrier lives in the leader CTA.
//
//   warp 0 (both CTAs)   TMA producer: waits its own `empty[s]`, loads A and its
//                        B half, completion bytes go to the LEADER's `full[s]`.
//   warp 1 (leader only) waits `full[s]`, issues BKT/16 MMAs per k block,
//                        tcgen05.commit multicast to `empty[s]` of both CTAs; after
//                        the last k block commits to `acc_full[a]` of both.
//   warps 2-5 (both)     epilogue on the CTA's own 128 rows: tcgen05.ld, + bias,
//                        relu / silu, 128B-swizzled smem staging, TMA tile stores
//                        (C read-modify-written with 128-bit accesses when it is an
//                        input); then arrive on the leader's `acc_empty[a]`
//                        (8 arrivals: 4 warps x 2 CTAs).
//
// Default: 3 stages of BKT = 128 (64 KB per CTA and stage).  The MMA thread pays
// a fixed cost per k block (barrier wait, fence, commit); with 64-wide blocks
// that cost left the tensor pipe idle 12 % of the cycles even for a single pair
// running alone, with 128-wide blocks 6 %.  In-kernel cycle counters (template
// flag STATS, IMEX_GEMM_STATS=1) report where each role waits.
// Waits are bounded; a wait that runs out records a status code and the role
// leaves its loop, after which the pair drains, syncs and frees TMEM.
#include "epilogue.cuh"
#include "tcgen05_host.h"
#include "tcgen05_ptx.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdio>
#include <cstdlib>
#include <mutex>

namespace imex {
namespace {

using namespace tc;
using namespace tc_host;

constexpr int BM = 128;       // rows per CTA
constexpr int PAIR_M = 256;   // rows per CTA pair (UMMA M)
constexpr int BN = 256;       // tile columns (UMMA N)
constexpr int BN_HALF = 128;  // columns of B each CTA loads
constexpr int UMMA_K = 16;
constexpr int NUM_ACC = 2;
constexpr int TMEM_COLS = 512;
// BKT = k elements per stage: 64 (one 128-byte swizzle row of A per box) or 128.
constexpr int A_BOX_BYTES = BM * 64 * 2;                                // 16 KB: 128 rows x 64 k
__host__ __device__ constexpr int a_stage_bytes(int bkt) { return BM * bkt * 2; }           // bkt/64 boxes
__host__ __device__ constexpr int b_box_bytes(int bkt) { return bkt * 64 * 2; }             // bkt k x 64 columns
__host__ __device__ constexpr int b_stage_bytes(int bkt) { return 2 * b_box_bytes(bkt); }   // this CTA's 128 columns
__host__ __device__ constexpr int stage_bytes(int bkt) { return a_stage_bytes(bkt) + b_stage_bytes(bkt); }
constexpr int NUM_THREADS = 192;
constexpr int EPI_CHUNK_BYTES = 32 * 32 * 4;              // 32 rows x 32 f32 columns
constexpr int EPI_BYTES = 4 * 2 * EPI_CHUNK_BYTES;        // 4 epilogue warps, double buffered
constexpr int smem_bytes(int stages, int bkt) {
  return stages * stage_bytes(bkt) + EPI_BYTES + 1024 + 256;
}

struct PairParams {
  float *C;
  const float *bias;
  unsigned *status;
  int M, N, K;
  long long ldc;
  int tiles_m, tiles_n, num_tiles, group_m;  // in 256x256 pair tiles
  int k_blocks;
  // Tail of the persistent schedule: the last `split_tiles` tiles are cut along k into
  // `split` parts each; a part leaves its raw f32 accumulator in `partials` (slot-major,
  // 256x256 per slot) and gemm_splitk_fixup_kernel adds the parts up.  Work items are
  // numbered: whole tiles first (item == tile), then split_tiles * split parts.
  int whole_tiles, split_tiles, split, num_items;
  float *partials;
  int epilogue;
  int accumulate;
  int out_dtype;  // kF32 (TMA tile stores) or kBF16 / kF16 (packed 16-byte stores)
  int fast_epilogue;  // silu through the hardware exp2 / reciprocal units
  uint32_t idesc;
  long long *stats;   // optional per-CTA cycle counters (nullptr = off), 8 per CTA
};

struct WorkItem {
  int mb, nb;    // pair-tile coordinates
  int kb0, kb1;  // k blocks [kb0, kb1)
  int slot;      // partial slot, or -1 for a whole tile (normal epilogue)
};

// Epilogue of the tensor-core path.  The f32 reference chain of silu (expf, IEEE divide)
// costs ~25 instructions per output element; on config 5 that is 13 G instructions per
// step beside a GEMM that runs at the board's power limit.  `fast` evaluates the same
// function with ex2.approx and rcp.approx (relative error ~1e-6 against a 1e-3 budget).
__device__ __forceinline__ float pair_epilogue(float v, int epilogue, int fast) {
  return fast ? apply_epilogue_fast(v, epilogue) : apply_epilogue(v, epilogue);
}

// cycle counter for the optional in-kernel statistics; free when they are off
template <bool STATS> __device__ __forceinline__ long long now() {
  if constexpr (STATS) return clock64();
  return 0;
}

// 16-bit storage formats of C (dt = kBF16 or kF16), round to nearest even
__device__ __forceinline__ uint16_t f32_to_half_bits(float v, int dt) {
  return dt == kBF16 ? __bfloat16_as_ushort(__float2bfloat16_rn(v)) : __half_as_ushort(__float2half_rn(v));
}
__device__ __forceinline__ float half_bits_to_f32(uint16_t b, int dt) {
  return dt == kBF16 ? __uint_as_float(static_cast<uint32_t>(b) << 16) : __half2float(__ushort_as_half(b));
}

__device__ __forceinline__ void pair_tile_coords(int tile, const PairParams &p, int &mb, int &nb) {
  const int band_tiles = p.group_m * p.tiles_n;
  const int band = tile / band_tiles;
  const int first_m = band * p.group_m;
  const int rows_in_band = min(p.group_m, p.tiles_m - first_m);
  const int t = tile - band * band_tiles;
  nb = t / rows_in_band;
  mb = first_m + t % rows_in_band;
}

__device__ __forceinline__ WorkItem item_at(int idx, const PairParams &p) {
  WorkItem w;
  int tile = idx;
  w.kb0 = 0;
  w.kb1 = p.k_blocks;
  w.slot = -1;
  if (idx >= p.whole_tiles) {
    const int s = idx - p.whole_tiles;
    const int part = s % p.split;
    tile = p.whole_tiles + s / p.split;
    w.kb0 = p.k_blocks * part / p.split;
    w.kb1 = p.k_blocks * (part + 1) / p.split;
    w.slot = s;
  }
  pair_tile_coords(tile, p, w.mb, w.nb);
  return w;
}

// TA: A is stored [K,M] (M-major operand: boxes of 64 m x BKT k, like B below);
// TB: B is stored [N,K] (K-major operand: boxes of 64 k x 128 n, like A below).
template <int STAGES, int BKT, bool STATS, bool TA, bool TB>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm_tcgen05_2cta_kernel(const __grid_constant__ CUtensorMap tmap_a,
                         const __grid_constant__ CUtensorMap tmap_b,
                         const __grid_constant__ CUtensorMap tmap_c,
                         const __grid_constant__ CUtensorMap tmap_p, const PairParams p) {
  constexpr int BK = BKT;
  constexpr int STAGE_BYTES = stage_bytes(BKT);
  constexpr int A_STAGE_BYTES = a_stage_bytes(BKT);
  constexpr int B_BOX_BYTES = b_box_bytes(BKT);
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t epi_base = smem_base + STAGES * STAGE_BYTES;  // 1024-byte aligned
  const uint32_t bars = epi_base + EPI_BYTES;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
  auto acc_full_bar = [&](int a) { return bars + 8u * (2 * STAGES + a); };
  auto acc_empty_bar = [&](int a) { return bars + 8u * (2 * STAGES + NUM_ACC + a); };
  const uint32_t tmem_slot = bars + 8u * (2 * STAGES + 2 * NUM_ACC);
  uint8_t *smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
  volatile uint32_t *tmem_slot_ptr = reinterpret_cast<volatile uint32_t *>(
      smem_aligned + STAGES * STAGE_BYTES + EPI_BYTES + 8 * (2 * STAGES + 2 * NUM_ACC));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = cluster_ctarank();
  const bool leader = cta_rank == 0;
  const int cluster_id = blockIdx.x >> 1;
  const int num_clusters = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);   // used in the leader: its own expect-tx arrival
      mbar_init(empty_bar(s), 1);  // one multicast commit per round
    }
    for (int a = 0; a < NUM_ACC; ++a) {
      mbar_init(acc_full_bar(a), 1);
      mbar_init(acc_empty_bar(a), 8);  // used in the leader: 4 epilogue warps x 2 CTAs
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers exist before anything signals them
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_a) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_b) : "memory");
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      long long t_begin = now<STATS>(), w_empty = 0, w_issue = 0;
      for (int item = cluster_id; item < p.num_items && ok; item += num_clusters) {
        const WorkItem w = item_at(item, p);
        const int row0 = w.mb * PAIR_M + static_cast<int>(cta_rank) * BM;
        const int col0 = w.nb * BN + static_cast<int>(cta_rank) * BN_HALF;
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          const long long t0 = now<STATS>();
          if (!mbar_wait(empty_bar(stage), phase ^ 1u)) {
            report(p.status, kStatusTmaWaitTimeout);
            ok = false;
            break;
          }
          w_empty += now<STATS>() - t0;
          const long long t1 = now<STATS>();
          const uint32_t leader_full = map_to_cta(full_bar(stage), 0);
          if (leader) mbar_expect_tx(full_bar(stage), 2 * STAGE_BYTES);
          const uint32_t a_dst = smem_base + stage * STAGE_BYTES;
          const uint32_t b_dst = a_dst + A_STAGE_BYTES;
          if constexpr (!TA) {
#pragma unroll
            for (int j = 0; j < BK / 64; ++j)
              tma_load_2d_pair(a_dst + j * A_BOX_BYTES, &tmap_a, kb * BK + j * 64, row0, leader_full);
          } else {
            tma_load_2d_pair(a_dst, &tmap_a, row0, kb * BK, leader_full);
            tma_load_2d_pair(a_dst + B_BOX_BYTES, &tmap_a, row0 + 64, kb * BK, leader_full);
          }
          if constexpr (!TB) {
            tma_load_2d_pair(b_dst, &tmap_b, col0, kb * BK, leader_full);
            tma_load_2d_pair(b_dst + B_BOX_BYTES, &tmap_b, col0 + 64, kb * BK, leader_full);
          } else {
#pragma unroll
            for (int j = 0; j < BK / 64; ++j)
              tma_load_2d_pair(b_dst + j * A_BOX_BYTES, &tmap_b, kb * BK + j * 64, col0, leader_full);
          }
          w_issue += now<STATS>() - t1;
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (STATS && p.stats) {
        long long *st = p.stats + 8 * blockIdx.x;
        st[3] = now<STATS>() - t_begin;  // producer: total
        st[4] = w_empty;              // ... of which waiting for a free stage
        st[7] = w_issue;              // ... of which issuing the three tile loads
      }
      // Tail: every stage this CTA filled has been consumed (its commit arrived
      // here) before the CTA may exit — nothing is still reading this shared memory
      // or about to signal these barriers.
      for (int s = 0; s < STAGES; ++s) {
        if (!mbar_wait(empty_bar(stage), phase ^ 1u)) break;
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer (leader) -----------------------
    if (leader && lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      long long t_begin = now<STATS>(), w_full = 0, w_acc = 0, w_mma = 0;
      for (int item = cluster_id; item < p.num_items && ok; item += num_clusters) {
        const WorkItem w = item_at(item, p);
        long long t0 = now<STATS>();
        if (!mbar_wait(acc_empty_bar(acc), acc_phase ^ 1u)) {
          report(p.status, kStatusMmaWaitTimeout);
          break;
        }
        w_acc += now<STATS>() - t0;
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          t0 = now<STATS>();
          if (!mbar_wait(full_bar(stage), phase)) {
            report(p.status, kStatusMmaWaitTimeout);
            ok = false;
            break;
          }
          w_full += now<STATS>() - t0;
          tcgen05_fence_after();
          t0 = now<STATS>();
          const uint32_t a_addr = smem_base + stage * STAGE_BYTES;
          const uint32_t b_addr = a_addr + A_STAGE_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // K-major operand: 64-k boxes of 128 rows, 32 bytes per K16 step inside a box;
            // MN-major operand: boxes of 64 rows/columns x BKT k, 16 k-rows (2 KB) per step
            const uint64_t a_desc =
                TA ? make_smem_desc(a_addr + k * (UMMA_K * 128), B_BOX_BYTES, 1024)
                   : make_smem_desc(a_addr + (k >> 2) * A_BOX_BYTES + (k & 3) * (UMMA_K * 2), 16, 1024);
            const uint64_t b_desc =
                TB ? make_smem_desc(b_addr + (k >> 2) * A_BOX_BYTES + (k & 3) * (UMMA_K * 2), 16, 1024)
                   : make_smem_desc(b_addr + k * (UMMA_K * 128), B_BOX_BYTES, 1024);
            tcgen05_mma_f16_pair(d_tmem, a_desc, b_desc, p.idesc, (kb != w.kb0 || k) ? 1u : 0u);
          }
          tcgen05_commit_pair(empty_bar(stage), 3);
          w_mma += now<STATS>() - t0;
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) tcgen05_commit_pair(acc_full_bar(acc), 3);
        if (++acc == NUM_ACC) { acc = 0; acc_phase ^= 1u; }
      }
      if (STATS && p.stats) {
        long long *st = p.stats + 8 * blockIdx.x;
        st[0] = now<STATS>() - t_begin;  // MMA thread: issue loop, total
        st[1] = w_full;               // ... of which waiting for operands
        st[2] = w_acc;                // ... of which waiting for a free accumulator
        p.stats[8 * (blockIdx.x + 1) + 2] = w_mma;  // (peer's unused slot) issuing MMAs + commit
      }
    }
  } else {
    // -------------------------------- epilogue (both CTAs) ---------------------
    const int lane_group = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    long long t_begin = now<STATS>(), w_accfull = 0;
    for (int item = cluster_id; item < p.num_items; item += num_clusters) {
      const WorkItem w = item_at(item, p);
      const int mb = w.mb, nb = w.nb;
      const long long t0 = now<STATS>();
      bool ok = mbar_wait(acc_full_bar(acc), acc_phase);
      w_accfull += now<STATS>() - t0;
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) report(p.status, kStatusEpiWaitTimeout);
        break;
      }
      tcgen05_fence_after();
      const int row0 = mb * PAIR_M + static_cast<int>(cta_rank) * BM + lane_group * 32;
      const int row = row0 + lane;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(lane_group * 32) << 16) + acc * BN;
      float *c_row = p.C + static_cast<size_t>(row) * p.ldc;
      const uint32_t my_bufs = epi_base + (warp - 2) * 2 * EPI_CHUNK_BYTES;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(t_row + c0, r);
        tmem_ld_wait();
        const int col0 = nb * BN + c0;
        if (w.slot >= 0) {
          // part of a k-split tile: the raw accumulator goes to its slot of the scratch
          // buffer (same swizzled staging + tile store as below, no bias, no epilogue)
          const uint32_t buf = my_bufs + ((c0 >> 5) & 1) * EPI_CHUNK_BYTES;
          if (lane == 0) tma_store_wait_read<1>();
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            const float4 v = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                         __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
            st_shared_v4(buf + lane * 128 + ((((j >> 2) ^ (lane & 7))) << 4), v);
          }
          fence_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&tmap_p, buf, c0,
                         w.slot * PAIR_M + static_cast<int>(cta_rank) * BM + lane_group * 32);
            tma_store_commit();
          }
        } else if (p.out_dtype != kF32) {
          // 16-bit C: each lane owns 32 consecutive columns of its row = 64 bytes,
          // written as four 16-byte stores (f32 accumulate / bias / epilogue first,
          // one rounding to bf16 or f16 at the end)
          if (row < p.M && col0 < p.N) {
            uint16_t *c16 = reinterpret_cast<uint16_t *>(p.C) + static_cast<size_t>(row) * p.ldc;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              const int col = col0 + j;
              if (col < p.N) {  // N is a multiple of 8 on this path
                float v[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(r[j + e]);
                if (p.accumulate) {
                  const uint4 c = *reinterpret_cast<const uint4 *>(c16 + col);
                  const uint32_t cw[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
                  for (int e = 0; e < 8; ++e)
                    v[e] += half_bits_to_f32(static_cast<uint16_t>(cw[e >> 1] >> ((e & 1) * 16)),
                                             p.out_dtype);
                }
                if (p.bias) {
                  const float4 b0 = *reinterpret_cast<const float4 *>(p.bias + col);
                  const float4 b1 = *reinterpret_cast<const float4 *>(p.bias + col + 4);
                  v[0] += b0.x; v[1] += b0.y; v[2] += b0.z; v[3] += b0.w;
                  v[4] += b1.x; v[5] += b1.y; v[6] += b1.z; v[7] += b1.w;
                }
                uint32_t o[4];
#pragma unroll
                for (int e = 0; e < 8; e += 2)
                  o[e >> 1] = static_cast<uint32_t>(f32_to_half_bits(pair_epilogue(v[e], p.epilogue, p.fast_epilogue), p.out_dtype)) |
                              (static_cast<uint32_t>(f32_to_half_bits(pair_epilogue(v[e + 1], p.epilogue, p.fast_epilogue), p.out_dtype)) << 16);
                *reinterpret_cast<uint4 *>(c16 + col) = make_uint4(o[0], o[1], o[2], o[3]);
              }
            }
          }
        } else if (p.accumulate) {
          // C is also an input: per-thread row segments, read-modify-write in place
          if (row < p.M && col0 < p.N) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              const int col = col0 + j;
              if (col < p.N) {
                float4 v = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                       __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
                const float4 c = *reinterpret_cast<const float4 *>(c_row + col);
                v.x += c.x; v.y += c.y; v.z += c.z; v.w += c.w;
                if (p.bias) {
                  const float4 b = *reinterpret_cast<const float4 *>(p.bias + col);
                  v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
                }
                v.x = pair_epilogue(v.x, p.epilogue, p.fast_epilogue);
                v.y = pair_epilogue(v.y, p.epilogue, p.fast_epilogue);
                v.z = pair_epilogue(v.z, p.epilogue, p.fast_epilogue);
                v.w = pair_epilogue(v.w, p.epilogue, p.fast_epilogue);
                *reinterpret_cast<float4 *>(c_row + col) = v;
              }
            }
          }
        } else {
          // Stage the 32x32 block in shared memory (128B-swizzled rows, so the 32
          // lanes' 16-byte stores spread over all banks) and let TMA write whole
          // 128-byte lines; rows / columns beyond M / N are clipped by the tensor map.
          const uint32_t buf = my_bufs + ((c0 >> 5) & 1) * EPI_CHUNK_BYTES;
          if (lane == 0) tma_store_wait_read<1>();  // the store that last read this buffer is done
          __syncwarp();
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            float4 v = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                   __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
            if (p.bias) {
              const int col = col0 + j;
              if (col < p.N) {
                const float4 b = *reinterpret_cast<const float4 *>(p.bias + col);
                v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
              }
            }
            v.x = pair_epilogue(v.x, p.epilogue, p.fast_epilogue);
            v.y = pair_epilogue(v.y, p.epilogue, p.fast_epilogue);
            v.z = pair_epilogue(v.z, p.epilogue, p.fast_epilogue);
            v.w = pair_epilogue(v.w, p.epilogue, p.fast_epilogue);
            st_shared_v4(buf + lane * 128 + ((((j >> 2) ^ (lane & 7))) << 4), v);
          }
          fence_async_smem();
          __syncwarp();
          if (lane == 0 && row0 < p.M && col0 < p.N) {
            tma_store_2d(&tmap_c, buf, col0, row0);
            tma_store_commit();
          }
        }
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(acc_empty_bar(acc), 0));
      if (++acc == NUM_ACC) { acc = 0; acc_phase ^= 1u; }
    }
    if (lane == 0) tma_store_wait_all<0>();  // all of this warp's tile stores have landed
    if (STATS && p.stats && warp == 2 && lane == 0) {
      long long *st = p.stats + 8 * blockIdx.x;
      st[5] = now<STATS>() - t_begin;  // epilogue warp: total
      st[6] = w_accfull;            // ... of which waiting for an accumulator
    }
  }

  __syncwarp();
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA leaves while the other may still touch its smem or barriers
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(TMEM_COLS)
                 : "memory");
  }
}

// Second step of a k-split tail: C tile = epilogue(C0 + bias + sum of the tile's parts,
// parts added in order).  One block per 8 rows of a split tile.
__global__ void __launch_bounds__(256)
gemm_splitk_fixup_kernel(const PairParams p) {
  // launched with programmatic stream serialisation: its blocks are set up while the GEMM's last
  // CTAs drain; nothing is read before the GEMM has completed and its writes are visible
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int t = blockIdx.x / (PAIR_M / 8);          // which split tile
  const int strip = blockIdx.x % (PAIR_M / 8);      // which 8 rows of it
  int mb, nb;
  pair_tile_coords(p.whole_tiles + t, p, mb, nb);
  const int col = nb * BN + (threadIdx.x & 63) * 4;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int lr = strip * 8 + (threadIdx.x >> 6) + 4 * h;  // row inside the tile
    const int row = mb * PAIR_M + lr;
    if (row >= p.M || col >= p.N) continue;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int part = 0; part < p.split; ++part) {
      const float4 q = *reinterpret_cast<const float4 *>(
          p.partials + (static_cast<size_t>(t * p.split + part) * PAIR_M + lr) * BN + (threadIdx.x & 63) * 4);
      v.x += q.x; v.y += q.y; v.z += q.z; v.w += q.w;
    }
    if (p.out_dtype != kF32) {
      uint16_t *c = reinterpret_cast<uint16_t *>(p.C) + static_cast<size_t>(row) * p.ldc + col;
      if (p.accumulate) {
        const uint2 c0 = *reinterpret_cast<const uint2 *>(c);
        v.x += half_bits_to_f32(static_cast<uint16_t>(c0.x), p.out_dtype);
        v.y += half_bits_to_f32(static_cast<uint16_t>(c0.x >> 16), p.out_dtype);
        v.z += half_bits_to_f32(static_cast<uint16_t>(c0.y), p.out_dtype);
        v.w += half_bits_to_f32(static_cast<uint16_t>(c0.y >> 16), p.out_dtype);
      }
      if (p.bias) {
        const float4 b = *reinterpret_cast<const float4 *>(p.bias + col);
        v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
      }
      uint2 o;
      o.x = static_cast<uint32_t>(f32_to_half_bits(pair_epilogue(v.x, p.epilogue, p.fast_epilogue), p.out_dtype)) |
            (static_cast<uint32_t>(f32_to_half_bits(pair_epilogue(v.y, p.epilogue, p.fast_epilogue), p.out_dtype)) << 16);
      o.y = static_cast<uint32_t>(f32_to_half_bits(pair_epilogue(v.z, p.epilogue, p.fast_epilogue), p.out_dtype)) |
            (static_cast<uint32_t>(f32_to_half_bits(pair_epilogue(v.w, p.epilogue, p.fast_epilogue), p.out_dtype)) << 16);
      *reinterpret_cast<uint2 *>(c) = o;
      continue;
    }
    float *c = p.C + static_cast<size_t>(row) * p.ldc + col;
    if (p.accumulate) {
      const float4 c0 = *reinterpret_cast<const float4 *>(c);
      v.x += c0.x; v.y += c0.y; v.z += c0.z; v.w += c0.w;
    }
    if (p.bias) {
      const float4 b = *reinterpret_cast<const float4 *>(p.bias + col);
      v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
    }
    v.x = pair_epilogue(v.x, p.epilogue, p.fast_epilogue);
    v.y = pair_epilogue(v.y, p.epilogue, p.fast_epilogue);
    v.z = pair_epilogue(v.z, p.epilogue, p.fast_epilogue);
    v.w = pair_epilogue(v.w, p.epilogue, p.fast_epilogue);
    *reinterpret_cast<float4 *>(c) = v;
  }
}

} // namespace

size_t gemm_tcgen05_workspace_bytes() {
  // one 256x256 f32 slot per CTA pair in flight is the most a k-split tail can use
  return static_cast<size_t>(sm_count() / 2) * PAIR_M * BN * sizeof(float);
}

bool gemm_tcgen05_2cta_supported(const GemmProblem &p) {
  if (p.in_dtype != kBF16 && p.in_dtype != kF16) return false;
  if (p.out_dtype != kF32 && p.out_dtype != kBF16 && p.out_dtype != kF16) return false;
  if (p.M <= 0 || p.N <= 0 || p.K <= 0) return false;
  if (p.M > INT32_MAX || p.N > INT32_MAX || p.K > INT32_MAX) return false;
  // TMA: the contiguous extent and the row pitch of every array are whole 16-byte units
  const int64_t a_inner = p.trans_a ? p.M : p.K, b_inner = p.trans_b ? p.K : p.N;
  const int64_t c_unit = p.out_dtype == kF32 ? 4 : 8;
  if (a_inner % 8 || b_inner % 8 || p.N % c_unit) return false;
  if (p.lda % 8 || p.ldb % 8 || p.ldc % c_unit) return false;
  if ((p.lda && p.lda < a_inner) || (p.ldb && p.ldb < b_inner) || (p.ldc && p.ldc < p.N)) return false;
  auto al = [](const void *q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  return al(p.A) && al(p.B) && al(p.C) && (!p.bias || al(p.bias));
}

bool gemm_tcgen05_2cta_preferred(const GemmProblem &p) {
  // a single row block gains nothing from pairing, but only this kernel takes
  // transposed operands and 16-bit outputs
  if (!gemm_tcgen05_2cta_supported(p)) return false;
  if (p.trans_a || p.trans_b || p.out_dtype != kF32) return true;
  return p.M > 128 && !getenv("IMEX_B200_GEMM_1CTA");
}

cudaError_t launch_gemm_tcgen05_2cta(const GemmProblem &g, unsigned *status, cudaStream_t stream) {
  if (!gemm_tcgen05_2cta_supported(g)) return cudaErrorInvalidValue;
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  static bool with_stats = false;
  std::call_once(once, [] {
    with_stats = getenv("IMEX_GEMM_STATS") != nullptr;
    auto set = [](const void *fn, int bytes) {
      return cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    };
    const cudaError_t e[] = {
        set((const void *)gemm_tcgen05_2cta_kernel<3, 128, false, false, false>, smem_bytes(3, 128)),
        set((const void *)gemm_tcgen05_2cta_kernel<3, 128, true, false, false>, smem_bytes(3, 128)),
        set((const void *)gemm_tcgen05_2cta_kernel<3, 128, false, true, false>, smem_bytes(3, 128)),
        set((const void *)gemm_tcgen05_2cta_kernel<3, 128, false, false, true>, smem_bytes(3, 128)),
        set((const void *)gemm_tcgen05_2cta_kernel<3, 128, false, true, true>, smem_bytes(3, 128))};
    for (cudaError_t x : e)
      if (x != cudaSuccess && attr_err == cudaSuccess) attr_err = x;
  });
  const bool transposed = g.trans_a || g.trans_b;
  const int BK = 128;  // 3 stages of 128 k (see the header of this file)
  if (attr_err != cudaSuccess) return attr_err;

  const int64_t lda = g.lda > 0 ? g.lda : (g.trans_a ? g.M : g.K);
  const int64_t ldb = g.ldb > 0 ? g.ldb : (g.trans_b ? g.K : g.N);
  const int64_t ldc = g.ldc > 0 ? g.ldc : g.N;
  CUtensorMap ta, tb;
  if (!(g.trans_a ? make_map(&ta, g.A, g.in_dtype, g.M, g.K, BK, lda)
                  : make_map(&ta, g.A, g.in_dtype, g.K, g.M, BM, lda)))
    return cudaErrorNotSupported;
  if (!(g.trans_b ? make_map(&tb, g.B, g.in_dtype, g.K, g.N, BN_HALF, ldb)
                  : make_map(&tb, g.B, g.in_dtype, g.N, g.K, BK, ldb)))
    return cudaErrorNotSupported;
  CUtensorMap tc_{};  // the f32 store side; a 16-bit C is written with plain stores
  if (g.out_dtype == kF32 && !make_map_f32_out(&tc_, g.C, g.N, g.M, ldc)) return cudaErrorNotSupported;

  PairParams p;
  p.C = g.C;
  p.bias = g.bias;
  p.status = status;
  p.M = static_cast<int>(g.M);
  p.N = static_cast<int>(g.N);
  p.K = static_cast<int>(g.K);
  p.ldc = ldc;
  p.tiles_m = (p.M + PAIR_M - 1) / PAIR_M;
  p.tiles_n = (p.N + BN - 1) / BN;
  p.num_tiles = p.tiles_m * p.tiles_n;
  p.group_m = 8;
  if (const char *e = getenv("IMEX_GEMM_GROUP_M")) {
    int v = atoi(e);
    if (v > 0) p.group_m = v;
  }
  p.k_blocks = (p.K + BK - 1) / BK;
  p.epilogue = g.epilogue;
  p.accumulate = g.accumulate ? 1 : 0;
  p.out_dtype = g.out_dtype;
  static const bool precise_epilogue = getenv("IMEX_GEMM_PRECISE_EPILOGUE") != nullptr;
  p.fast_epilogue = precise_epilogue ? 0 : 1;
  p.stats = nullptr;
  static long long *stats_buf = nullptr;
  const bool want_stats = with_stats && !transposed;  // development aid (IMEX_GEMM_STATS=1)
  if (want_stats) {
    if (!stats_buf) cudaMallocManaged(&stats_buf, 8 * 148 * sizeof(long long));
    p.stats = stats_buf;
  }
  const uint32_t fmt = g.in_dtype == kBF16 ? 1u : 0u;
  // bit 15 / 16: A / B operand is MN-major (A when stored [K,M]; B when stored [K,N])
  p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((g.trans_a ? 1u : 0u) << 15) |
            ((g.trans_b ? 0u : 1u) << 16) |
            (static_cast<uint32_t>(BN >> 3) << 17) | (static_cast<uint32_t>(PAIR_M >> 4) << 24);

  int usable = sm_count() - (g.sm_margin > 0 ? g.sm_margin : 0);
  if (usable < 2) usable = 2;
  const int max_clusters = usable / 2;
  // k-split tail: when the last wave would leave at least half of the pairs idle, its
  // tiles are cut along k into as many parts as fill the machine (the sums then differ
  // in the last bits from an unsplit run: IMEX_GEMM_NO_SPLITK=1 keeps every tile whole).
  p.whole_tiles = p.num_tiles;
  p.split_tiles = 0;
  p.split = 1;
  p.partials = static_cast<float *>(g.workspace);
  {
    const int rem = p.num_tiles % max_clusters;
    int parts = rem > 0 ? max_clusters / rem : 1;
    if (parts > 8) parts = 8;
    while (parts > 1 && p.k_blocks / parts < 2) --parts;
    const size_t need = static_cast<size_t>(rem) * parts * PAIR_M * BN * sizeof(float);
    if (parts >= 2 && g.workspace && need <= g.workspace_bytes && !getenv("IMEX_GEMM_NO_SPLITK")) {
      p.split_tiles = rem;
      p.split = parts;
      p.whole_tiles = p.num_tiles - rem;
    }
  }
  p.num_items = p.whole_tiles + p.split_tiles * p.split;
  CUtensorMap tp = tc_;  // placeholder when nothing is split (never dereferenced)
  if (p.split_tiles &&
      !make_map_f32_out(&tp, p.partials, BN, static_cast<int64_t>(p.split_tiles) * p.split * PAIR_M, BN))
    return cudaErrorNotSupported;
  const int clusters = p.num_items < max_clusters ? p.num_items : max_clusters;
  const dim3 grid(2 * clusters), block(NUM_THREADS);
  const int sm3 = smem_bytes(3, 128);
  if (g.trans_a && g.trans_b)
    gemm_tcgen05_2cta_kernel<3, 128, false, true, true><<<grid, block, sm3, stream>>>(ta, tb, tc_, tp, p);
  else if (g.trans_a)
    gemm_tcgen05_2cta_kernel<3, 128, false, true, false><<<grid, block, sm3, stream>>>(ta, tb, tc_, tp, p);
  else if (g.trans_b)
    gemm_tcgen05_2cta_kernel<3, 128, false, false, true><<<grid, block, sm3, stream>>>(ta, tb, tc_, tp, p);
  else if (with_stats)
    gemm_tcgen05_2cta_kernel<3, 128, true, false, false><<<grid, block, sm3, stream>>>(ta, tb, tc_, tp, p);
  else
    gemm_tcgen05_2cta_kernel<3, 128, false, false, false><<<grid, block, sm3, stream>>>(ta, tb, tc_, tp, p);
  if (p.split_tiles) {
    cudaError_t le = cudaGetLastError();
    if (le != cudaSuccess) return le;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.split_tiles * (PAIR_M / 8));
    cfg.blockDim = dim3(256);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    le = cudaLaunchKernelEx(&cfg, gemm_splitk_fixup_kernel, p);
    if (le != cudaSuccess) return le;
  }
  if (g.launched) *g.launched = p.split_tiles ? 2 : 1;
  if (want_stats && stats_buf) {
    cudaStreamSynchronize(stream);
    double a[8] = {0};
    for (int c = 0; c < 2 * clusters; ++c)
      for (int i = 0; i < 8; ++i) a[i] += static_cast<double>(stats_buf[8 * c + i]);
    const double nl = clusters, nc = 2.0 * clusters;
    fprintf(stderr,
            "[gemm_2cta stats, mean cycles] mma total %.0f wait_full %.0f wait_acc %.0f | "
            "producer total %.0f wait_empty %.0f issue %.0f | epilogue total %.0f wait_acc_full %.0f\n",
            a[0] / nl, a[1] / nl, a[2] / nl, a[3] / nc, a[4] / nc, a[7] / nc, a[5] / nc, a[6] / nc);
  }
  return cudaGetLastError();
}

} // namespace imex
