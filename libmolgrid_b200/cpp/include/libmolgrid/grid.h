// Grid<Dtype, N, isCUDA>: non-owning N-dimensional array view, the argument type of every
// libmolgrid operation (reference: include/libmolgrid/grid.h).  Same template signature, member
// layout {pointer, extents[N], strides[N]} (1-D: {pointer, extent}), typedef names and member
// functions, so code written against the reference's header compiles against this one.
#ifndef LMGB200_GRID_H_
#define LMGB200_GRID_H_

#include <algorithm>
#include <cstring>

#include "libmolgrid/common.h"

namespace libmolgrid {

template <typename Dtype, std::size_t NumDims>
class ManagedGrid;

namespace detail {
inline cudaMemcpyKind copy_kind(bool src_gpu, bool dst_gpu) {
  if (src_gpu) return dst_gpu ? cudaMemcpyDeviceToDevice : cudaMemcpyDeviceToHost;
  return dst_gpu ? cudaMemcpyHostToDevice : cudaMemcpyHostToHost;
}
// bytes from one side to the other; host-to-host copies need no CUDA runtime
inline void copy_bytes(void* dst, const void* src, size_t bytes, bool src_gpu, bool dst_gpu) {
  if (!bytes) return;
  if (!src_gpu && !dst_gpu) std::memcpy(dst, src, bytes);
  else LMG_CUDA_CHECK(cudaMemcpy(dst, src, bytes, copy_kind(src_gpu, dst_gpu)));
}
inline void bounds(size_t i, size_t n) {
  if (i >= n) throw std::out_of_range("Invalid range. " + itoa((long long)i) + " >= " + itoa((long long)n));
}
}  // namespace detail

template <typename Dtype, std::size_t NumDims, bool isCUDA = false>
class Grid {
 protected:
  Dtype* buffer;
  size_t dims[NumDims];
  size_t offs[NumDims];

 public:
  using type = Dtype;
  using subgrid_t = Grid<Dtype, NumDims - 1, isCUDA>;
  using managed_t = ManagedGrid<Dtype, NumDims>;
  using cpu_grid_t = Grid<Dtype, NumDims, false>;
  using gpu_grid_t = Grid<Dtype, NumDims, true>;
  static constexpr size_t N = NumDims;
  static constexpr bool GPU = isCUDA;

  Grid() : buffer(nullptr) {
    for (size_t i = 0; i < NumDims; i++) dims[i] = offs[i] = 0;
  }

  // view over `d` with the given extents, densely packed, last index fastest
  template <typename... I>
  Grid(Dtype* const d, I... sizes) : buffer(d), dims{static_cast<size_t>(sizes)...} {
    static_assert(NumDims == sizeof...(sizes), "Incorrect number of grid dimensions");
    size_t stride = 1;
    for (size_t i = NumDims; i-- > 0;) {
      offs[i] = stride;
      stride *= dims[i];
    }
  }

  // slice i of a grid with one more dimension
  explicit Grid(const Grid<Dtype, NumDims + 1, isCUDA>& parent, size_t i)
      : buffer(parent.data() ? parent.data() + i * parent.offset(0) : nullptr) {
    for (size_t k = 0; k < NumDims; k++) {
      dims[k] = parent.dimension(k + 1);
      offs[k] = parent.offset(k + 1);
    }
  }

  const size_t* dimensions() const { return dims; }
  size_t dimension(size_t i) const {
    detail::bounds(i, NumDims);
    return dims[i];
  }
  const size_t* offsets() const { return offs; }
  size_t offset(size_t i) const { return offs[i]; }
  size_t size() const {
    size_t n = 1;
    for (size_t i = 0; i < NumDims; i++) n *= dims[i];
    return n;
  }
  Dtype* data() const { return buffer; }
  void set_buffer(Dtype* p) { buffer = p; }

  subgrid_t operator[](size_t i) const {
    detail::bounds(i, dims[0]);
    return subgrid_t(*this, i);
  }

  // element access; only meaningful on the host for isCUDA == false
  template <typename... I>
  Dtype& operator()(I... idx) {
    return buffer[position(idx...)];
  }
  template <typename... I>
  Dtype operator()(I... idx) const {
    return buffer[position(idx...)];
  }
  template <typename... I>
  Dtype* address(I... idx) const {
    return buffer + position(idx...);
  }

  template <bool destCUDA>
  size_t copyTo(Grid<Dtype, NumDims, destCUDA>& dest) const {
    size_t n = std::min(size(), dest.size());
    detail::copy_bytes(dest.data(), buffer, n * sizeof(Dtype), isCUDA, destCUDA);
    return n;
  }
  template <bool srcCUDA>
  size_t copyFrom(const Grid<Dtype, NumDims, srcCUDA>& src) {
    size_t n = std::min(size(), src.size());
    detail::copy_bytes(buffer, src.data(), n * sizeof(Dtype), srcCUDA, isCUDA);
    return n;
  }
  void fill_zero() {
    if (!size()) return;
    if (isCUDA) LMG_CUDA_CHECK(cudaMemset(buffer, 0, sizeof(Dtype) * size()));
    else std::memset(buffer, 0, sizeof(Dtype) * size());
  }

 private:
  template <typename... I>
  size_t position(I... idx) const {
    static_assert(NumDims == sizeof...(idx), "Incorrect number of grid indices");
    size_t ix[NumDims] = {static_cast<size_t>(idx)...};
    size_t p = 0;
    for (size_t i = 0; i < NumDims; i++) p += ix[i] * offs[i];
    return p;
  }
};

// One-dimensional grids index to scalars and carry no stride array.
template <typename Dtype, bool isCUDA>
class Grid<Dtype, 1, isCUDA> {
 protected:
  Dtype* buffer;
  size_t dims[1];

 public:
  using type = Dtype;
  using subgrid_t = Dtype;
  using managed_t = ManagedGrid<Dtype, 1>;
  using cpu_grid_t = Grid<Dtype, 1, false>;
  using gpu_grid_t = Grid<Dtype, 1, true>;
  static constexpr size_t N = 1;
  static constexpr bool GPU = isCUDA;

  Grid() : buffer(nullptr), dims{0} {}
  Grid(Dtype* const d, size_t n) : buffer(d), dims{n} {}
  explicit Grid(const Grid<Dtype, 2, isCUDA>& parent, size_t i)
      : buffer(parent.data() ? parent.data() + i * parent.offset(0) : nullptr), dims{parent.dimension(1)} {}

  const size_t* dimensions() const { return dims; }
  size_t dimension(size_t i) const {
    detail::bounds(i, 1);
    return dims[0];
  }
  size_t offset(size_t) const { return 1; }
  size_t size() const { return dims[0]; }
  Dtype* data() const { return buffer; }
  void set_buffer(Dtype* p) { buffer = p; }

  Dtype& operator[](size_t i) {
    detail::bounds(i, dims[0]);
    return buffer[i];
  }
  Dtype operator[](size_t i) const {
    detail::bounds(i, dims[0]);
    return buffer[i];
  }
  Dtype& operator()(size_t i) { return buffer[i]; }
  Dtype operator()(size_t i) const { return buffer[i]; }
  Dtype* address(size_t i) const { return buffer + i; }

  template <bool destCUDA>
  size_t copyTo(Grid<Dtype, 1, destCUDA>& dest) const {
    size_t n = std::min(size(), dest.size());
    detail::copy_bytes(dest.data(), buffer, n * sizeof(Dtype), isCUDA, destCUDA);
    return n;
  }
  template <bool srcCUDA>
  size_t copyFrom(const Grid<Dtype, 1, srcCUDA>& src) {
    size_t n = std::min(size(), src.size());
    detail::copy_bytes(buffer, src.data(), n * sizeof(Dtype), srcCUDA, isCUDA);
    return n;
  }
  void fill_zero() {
    if (!size()) return;
    if (isCUDA) LMG_CUDA_CHECK(cudaMemset(buffer, 0, sizeof(Dtype) * size()));
    else std::memset(buffer, 0, sizeof(Dtype) * size());
  }
};

#define LMGB200_GRID_TYPEDEFS(N)                 \
  typedef Grid<float, N, false> Grid##N##f;      \
  typedef Grid<double, N, false> Grid##N##d;     \
  typedef Grid<float, N, true> Grid##N##fCUDA;   \
  typedef Grid<double, N, true> Grid##N##dCUDA;
LMGB200_GRID_TYPEDEFS(1)
LMGB200_GRID_TYPEDEFS(2)
LMGB200_GRID_TYPEDEFS(3)
LMGB200_GRID_TYPEDEFS(4)
LMGB200_GRID_TYPEDEFS(5)
LMGB200_GRID_TYPEDEFS(6)
LMGB200_GRID_TYPEDEFS(7)
LMGB200_GRID_TYPEDEFS(8)
#undef LMGB200_GRID_TYPEDEFS

}  // namespace libmolgrid

#endif
