// 2-D transpose Y[j,i] = X[i,j] (bit copy) and rank-3 permutations.
// Reference generic: maps (d0,d1)->(d0,d1) in, (d0,d1)->(d1,d0) out
// (benchmarks/transpose/transpose2d_gpu.mlir.in:1-10; 3-D:
// transpose3d_gpu.mlir.in:1-10); its GPU lowering runs one work-item per
// element, uncoalesced on one side (test/SPIRV/OpTest.Transpose_FLOAT32.mlir:55-57).
// Here a 64x64 tile goes through shared memory: 128-bit coalesced loads, a
// padded tile so that the transposed read is bank-conflict free, 128-bit
// coalesced stores.  HBM traffic = read once + write once.
#include "kernels.h"

namespace imex {
namespace {

constexpr int TILE = 64;

// Fast path: 4-byte elements, rows % 4 == 0, cols % 4 == 0, 16-byte aligned.
__global__ void __launch_bounds__(256)
transpose2d_b32_vec_kernel(const uint32_t *__restrict__ x, uint32_t *__restrict__ y,
                           int64_t rows, int64_t cols, int64_t tiles_c) {
  __shared__ uint32_t tile[TILE][TILE + 1];
  const int64_t tr = blockIdx.x / tiles_c, tc = blockIdx.x % tiles_c;
  const int64_t r0 = tr * TILE, c0 = tc * TILE;
  const int tid = threadIdx.x;
  // load: 64 rows x 16 float4.  A warp takes 4 rows x 8 float4 (128 contiguous bytes per
  // row): with the 65-word row pitch its 32 scalar stores of one component fall into 32
  // different banks (bank = row + 4 * vec + k), and so do the transposed reads below.
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    const int slot = tid + 256 * p;
    int r = ((slot >> 3) & 3) + 4 * (slot >> 6), v = (slot & 7) + 8 * ((slot >> 5) & 1);
    int64_t gr = r0 + r, gc = c0 + 4 * v;
    if (gr < rows && gc < cols) {
      uint4 q = *reinterpret_cast<const uint4 *>(x + gr * cols + gc);
      tile[r][4 * v + 0] = q.x;
      tile[r][4 * v + 1] = q.y;
      tile[r][4 * v + 2] = q.z;
      tile[r][4 * v + 3] = q.w;
    }
  }
  __syncthreads();
  // store: output row = c0 + c, output cols r0 .. r0+63 as 16 float4
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    const int slot = tid + 256 * p;
    int c = ((slot >> 3) & 3) + 4 * (slot >> 6), v = (slot & 7) + 8 * ((slot >> 5) & 1);
    int64_t gc = c0 + c, gr = r0 + 4 * v;
    if (gc < cols && gr < rows) {
      uint4 q;
      q.x = tile[4 * v + 0][c];
      q.y = tile[4 * v + 1][c];
      q.z = tile[4 * v + 2][c];
      q.w = tile[4 * v + 3][c];
      *reinterpret_cast<uint4 *>(y + gc * rows + gr) = q;
    }
  }
}

// Any shape / 2- or 4-byte elements: 32x32 tile, scalar accesses.
// `batch` independent matrices (rank-3 permutation (0,2,1)).
template <typename T>
__global__ void __launch_bounds__(256)
transpose2d_generic_kernel(const T *__restrict__ x, T *__restrict__ y, int64_t rows, int64_t cols,
                           int64_t tiles_c, int64_t tiles_per_mat) {
  __shared__ T tile[32][33];
  const int64_t b = blockIdx.x / tiles_per_mat;
  const int64_t t = blockIdx.x % tiles_per_mat;
  const int64_t r0 = (t / tiles_c) * 32, c0 = (t % tiles_c) * 32;
  const T *xb = x + b * rows * cols;
  T *yb = y + b * rows * cols;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    int r = ty + 8 * p;
    if (r0 + r < rows && c0 + tx < cols) tile[r][tx] = xb[(r0 + r) * cols + c0 + tx];
  }
  __syncthreads();
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    int c = ty + 8 * p;
    if (c0 + c < cols && r0 + tx < rows) yb[(c0 + c) * rows + r0 + tx] = tile[tx][c];
  }
}

// Generic rank-3 permutation: one thread per OUTPUT element (coalesced writes).
template <typename T>
__global__ void __launch_bounds__(256)
transpose3d_gather_kernel(const T *__restrict__ x, T *__restrict__ y, int64_t d0,
                          int64_t d1, int64_t d2, int p0, int p1, int p2) {
  const int64_t dims[3] = {d0, d1, d2};
  const int64_t o1 = dims[p1], o2 = dims[p2];
  const int64_t total = d0 * d1 * d2;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t o = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; o < total;
       o += stride) {
    int64_t idx[3];
    idx[p2] = o % o2;
    idx[p1] = (o / o2) % o1;
    idx[p0] = o / (o2 * o1);
    y[o] = x[(idx[0] * d1 + idx[1]) * d2 + idx[2]];
  }
}

} // namespace

cudaError_t launch_transpose2d(const void *x, void *y, int64_t rows, int64_t cols, int elem_bytes,
                               cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return cudaSuccess;
  if (elem_bytes == 4 && rows % 4 == 0 && cols % 4 == 0 &&
      ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0) {
    int64_t tr = (rows + TILE - 1) / TILE, tc = (cols + TILE - 1) / TILE;
    transpose2d_b32_vec_kernel<<<static_cast<unsigned>(tr * tc), 256, 0, stream>>>(
        static_cast<const uint32_t *>(x), static_cast<uint32_t *>(y), rows, cols, tc);
    return cudaGetLastError();
  }
  int64_t tr = (rows + 31) / 32, tc = (cols + 31) / 32;
  if (elem_bytes == 4)
    transpose2d_generic_kernel<uint32_t><<<static_cast<unsigned>(tr * tc), 256, 0, stream>>>(
        static_cast<const uint32_t *>(x), static_cast<uint32_t *>(y), rows, cols, tc, tr * tc);
  else if (elem_bytes == 2)
    transpose2d_generic_kernel<uint16_t><<<static_cast<unsigned>(tr * tc), 256, 0, stream>>>(
        static_cast<const uint16_t *>(x), static_cast<uint16_t *>(y), rows, cols, tc, tr * tc);
  else
    return cudaErrorInvalidValue;
  return cudaGetLastError();
}

namespace {
template <typename T>
cudaError_t transpose3d_typed(const void *x, void *y, const int64_t dims[3], const int perm[3],
                              cudaStream_t stream) {
  const int64_t total = dims[0] * dims[1] * dims[2];
  if (perm[0] == 0 && perm[1] == 2 && perm[2] == 1) {  // batched 2-D transpose
    int64_t tr = (dims[1] + 31) / 32, tc = (dims[2] + 31) / 32;
    transpose2d_generic_kernel<T><<<static_cast<unsigned>(dims[0] * tr * tc), 256, 0, stream>>>(
        static_cast<const T *>(x), static_cast<T *>(y), dims[1], dims[2], tc, tr * tc);
    return cudaGetLastError();
  }
  int64_t blocks = (total + 255) / 256;
  if (blocks > 148 * 64) blocks = 148 * 64;
  transpose3d_gather_kernel<T><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
      static_cast<const T *>(x), static_cast<T *>(y), dims[0], dims[1], dims[2], perm[0], perm[1],
      perm[2]);
  return cudaGetLastError();
}
} // namespace

cudaError_t launch_transpose3d(const void *x, void *y, const int64_t dims[3], const int perm[3],
                               int elem_bytes, cudaStream_t stream) {
  if (dims[0] * dims[1] * dims[2] <= 0) return cudaSuccess;
  if (elem_bytes == 4) return transpose3d_typed<uint32_t>(x, y, dims, perm, stream);
  if (elem_bytes == 2) return transpose3d_typed<uint16_t>(x, y, dims, perm, stream);
  return cudaErrorInvalidValue;
}

} // namespace imex
