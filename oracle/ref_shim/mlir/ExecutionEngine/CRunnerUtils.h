/* Stand-in for the upstream MLIR header of the same name, which the
 * reference's lib/ExecutionEngine/ImexRunnerUtils.cpp includes but which is
 * not part of the reference tree.  TEST INFRASTRUCTURE ONLY: it exists so
 * that oracle/Makefile can compile the reference's own CPU GEMM
 * (_mlir_ciface_gemm*, ImexRunnerUtils.cpp:257-338) from where it lies into
 * oracle/_ref/.  Only the members that source file touches are provided;
 * the descriptor layout is the one include/imex/ExecutionEngine/
 * ImexRunnerUtils.h:36-42 pins (allocated, aligned, offset, sizes[N],
 * strides[N]) behind a {rank, descriptor*} pair. */
#ifndef IMEX_B200_SHIM_CRUNNERUTILS_H
#define IMEX_B200_SHIM_CRUNNERUTILS_H

#include <cstddef>
#include <cstdint>
#include <iterator>
#include <vector>

template <typename T> struct UnrankedMemRefType {
  int64_t rank;
  void *descriptor;
};

template <typename T> class DynamicMemRefIterator;

template <typename T> class DynamicMemRefType {
public:
  int64_t rank;
  T *basePtr;
  T *data;
  int64_t offset;
  const int64_t *sizes;
  const int64_t *strides;

  explicit DynamicMemRefType(const UnrankedMemRefType<T> &u) : rank(u.rank) {
    /* descriptor = { T* allocated; T* aligned; i64 offset; i64 sizes[rank];
     *                i64 strides[rank]; } */
    auto **ptrs = static_cast<T **>(u.descriptor);
    basePtr = ptrs[0];
    data = ptrs[1];
    auto *ints = reinterpret_cast<const int64_t *>(ptrs + 2);
    offset = ints[0];
    sizes = rank ? ints + 1 : nullptr;
    strides = rank ? ints + 1 + rank : nullptr;
  }

  DynamicMemRefIterator<T> begin() { return DynamicMemRefIterator<T>(*this, 0); }
  DynamicMemRefIterator<T> end() { return DynamicMemRefIterator<T>(*this, -1); }
};

/* Row-major walk over a strided memref; `linear == -1` is the end marker. */
template <typename T> class DynamicMemRefIterator {
public:
  using iterator_category = std::forward_iterator_tag;
  using value_type = T;
  using difference_type = std::ptrdiff_t;
  using pointer = T *;
  using reference = T &;

  DynamicMemRefIterator(DynamicMemRefType<T> &m, int64_t start = 0)
      : ref(&m), idx(static_cast<size_t>(m.rank), 0), pos(m.offset), linear(start) {
    total = 1;
    for (int64_t d = 0; d < m.rank; ++d)
      total *= m.sizes[d];
    if (total == 0)
      linear = -1;
  }

  DynamicMemRefIterator &operator++() {
    if (linear < 0)
      return *this;
    if (++linear >= total) {
      linear = -1;
      return *this;
    }
    for (int64_t d = ref->rank - 1; d >= 0; --d) {
      pos += ref->strides[d];
      if (++idx[d] < ref->sizes[d])
        break;
      pos -= idx[d] * ref->strides[d];
      idx[d] = 0;
    }
    return *this;
  }

  reference operator*() { return ref->data[pos]; }
  pointer operator->() { return &ref->data[pos]; }
  bool operator==(const DynamicMemRefIterator &o) const { return linear == o.linear; }
  bool operator!=(const DynamicMemRefIterator &o) const { return linear != o.linear; }

private:
  DynamicMemRefType<T> *ref;
  std::vector<int64_t> idx;
  int64_t pos;
  int64_t linear;
  int64_t total;
};

#endif
