// ManagedGrid<Dtype, N>: owning array with a host buffer and a lazily created device mirror
// (reference: include/libmolgrid/managed_grid.h).  Copies and sub-grids share one storage block and
// its "where is the valid copy" flag; cpu()/gpu() migrate the whole block on demand and return
// Grid views.  Serialization is not provided.
#ifndef LMGB200_MANAGED_GRID_H_
#define LMGB200_MANAGED_GRID_H_

#include <cstdlib>
#include <memory>

#include "libmolgrid/grid.h"

namespace libmolgrid {

namespace detail {
template <typename Dtype>
struct Storage {
  Dtype* host = nullptr;
  Dtype* dev = nullptr;
  size_t capacity = 0;   // elements
  bool on_gpu = false;   // the device copy is the valid one
  explicit Storage(size_t n) : capacity(n) {
    host = static_cast<Dtype*>(std::calloc(n ? n : 1, sizeof(Dtype)));
    if (!host) throw std::bad_alloc();
  }
  ~Storage() {
    std::free(host);
    if (dev) cudaFree(dev);
  }
  Storage(const Storage&) = delete;
  Storage& operator=(const Storage&) = delete;
  void ensure_dev() {
    if (!dev && capacity) LMG_CUDA_CHECK(cudaMalloc(&dev, capacity * sizeof(Dtype)));
  }
  void to_gpu(bool copy) {
    if (on_gpu) return;
    ensure_dev();
    if (copy && capacity) LMG_CUDA_CHECK(cudaMemcpy(dev, host, capacity * sizeof(Dtype), cudaMemcpyHostToDevice));
    on_gpu = true;
  }
  void to_cpu(bool copy) {
    if (!on_gpu) return;
    if (copy && capacity && dev)
      LMG_CUDA_CHECK(cudaMemcpy(host, dev, capacity * sizeof(Dtype), cudaMemcpyDeviceToHost));
    on_gpu = false;
  }
};
}  // namespace detail

template <typename Dtype, std::size_t NumDims>
class ManagedGrid {
  template <typename D, std::size_t M>
  friend class ManagedGrid;

  std::shared_ptr<detail::Storage<Dtype>> store_;
  size_t first_ = 0;  // element offset of this (sub)grid inside the storage block
  size_t dims_[NumDims];

  size_t stride(size_t i) const {
    size_t s = 1;
    for (size_t k = NumDims - 1; k > i; k--) s *= dims_[k];
    return s;
  }

 public:
  using gpu_grid_t = Grid<Dtype, NumDims, true>;
  using cpu_grid_t = Grid<Dtype, NumDims, false>;
  using type = Dtype;
  static constexpr size_t N = NumDims;

  ManagedGrid() {
    for (size_t i = 0; i < NumDims; i++) dims_[i] = 0;
  }

  template <typename... I>
  explicit ManagedGrid(I... sizes) : dims_{static_cast<size_t>(sizes)...} {
    static_assert(NumDims == sizeof...(sizes), "Incorrect number of grid dimensions");
    store_ = std::make_shared<detail::Storage<Dtype>>(size());
  }

  size_t dimension(size_t i) const {
    detail::bounds(i, NumDims);
    return dims_[i];
  }
  const size_t* dimensions() const { return dims_; }
  size_t size() const {
    size_t n = 1;
    for (size_t i = 0; i < NumDims; i++) n *= dims_[i];
    return n;
  }

  bool ongpu() const { return store_ && store_->on_gpu; }
  bool oncpu() const { return !ongpu(); }
  void togpu(bool copy = true) const {
    if (store_) store_->to_gpu(copy);
  }
  void tocpu(bool copy = true) const {
    if (store_) store_->to_cpu(copy);
  }

  // views; asking for one side makes that side the valid copy
  gpu_grid_t gpu() const {
    if (!store_) return view<true>(nullptr);
    store_->to_gpu(true);
    return view<true>(store_->dev + first_);
  }
  cpu_grid_t cpu() const {
    if (!store_) return view<false>(nullptr);
    store_->to_cpu(true);
    return view<false>(store_->host + first_);
  }
  operator gpu_grid_t() const { return gpu(); }
  operator cpu_grid_t() const { return cpu(); }

  Dtype* data() const {
    if (!store_) return nullptr;
    return ongpu() ? store_->dev + first_ : store_->host + first_;
  }

  // sub-grid sharing this grid's storage
  ManagedGrid<Dtype, NumDims - 1> operator[](size_t i) const {
    detail::bounds(i, dims_[0]);
    ManagedGrid<Dtype, NumDims - 1> sub;
    sub.store_ = store_;
    sub.first_ = first_ + i * stride(0);
    for (size_t k = 1; k < NumDims; k++) sub.dims_[k - 1] = dims_[k];
    return sub;
  }

  // host element access (moves the data to the host if needed)
  template <typename... I>
  Dtype& operator()(I... idx) {
    static_assert(NumDims == sizeof...(idx), "Incorrect number of grid indices");
    tocpu();
    size_t ix[NumDims] = {static_cast<size_t>(idx)...};
    size_t p = 0;
    for (size_t i = 0; i < NumDims; i++) p += ix[i] * stride(i);
    return store_->host[first_ + p];
  }

  void fill_zero() {
    if (ongpu()) gpu().fill_zero();
    else cpu().fill_zero();
  }

  ManagedGrid clone() const {
    ManagedGrid out;
    for (size_t i = 0; i < NumDims; i++) out.dims_[i] = dims_[i];
    out.store_ = std::make_shared<detail::Storage<Dtype>>(size());
    if (size()) {
      if (ongpu()) {
        out.store_->to_gpu(false);
        LMG_CUDA_CHECK(cudaMemcpy(out.store_->dev, store_->dev + first_, size() * sizeof(Dtype), cudaMemcpyDeviceToDevice));
      } else {
        std::memcpy(out.store_->host, store_->host + first_, size() * sizeof(Dtype));
      }
    }
    return out;
  }

  // same data with new extents; grows into a fresh block when the new extents need more room
  template <typename... I>
  ManagedGrid resized(I... sizes) const {
    ManagedGrid out(sizes...);
    size_t n = std::min(size(), out.size());
    if (n) {
      if (ongpu()) {
        out.store_->to_gpu(false);
        LMG_CUDA_CHECK(cudaMemcpy(out.store_->dev, store_->dev + first_, n * sizeof(Dtype), cudaMemcpyDeviceToDevice));
      } else {
        std::memcpy(out.store_->host, store_->host + first_, n * sizeof(Dtype));
      }
    }
    return out;
  }

  template <bool destCUDA>
  size_t copyTo(Grid<Dtype, NumDims, destCUDA>& dest) const {
    return ongpu() ? gpu().copyTo(dest) : cpu().copyTo(dest);
  }
  size_t copyTo(ManagedGrid& dest) const {
    if (dest.ongpu()) { auto g = dest.gpu(); return copyTo(g); }
    auto c = dest.cpu();
    return copyTo(c);
  }
  template <bool srcCUDA>
  size_t copyFrom(const Grid<Dtype, NumDims, srcCUDA>& src) {
    if (ongpu()) { auto g = gpu(); return g.copyFrom(src); }
    auto c = cpu();
    return c.copyFrom(src);
  }
  size_t copyFrom(const ManagedGrid& src) {
    return src.ongpu() ? copyFrom(src.gpu()) : copyFrom(src.cpu());
  }

  bool operator==(const ManagedGrid& o) const { return store_ == o.store_ && first_ == o.first_; }

 private:
  template <bool G>
  Grid<Dtype, NumDims, G> view(Dtype* p) const {
    return make_view<G>(p, std::make_index_sequence<NumDims>());
  }
  template <bool G, size_t... K>
  Grid<Dtype, NumDims, G> make_view(Dtype* p, std::index_sequence<K...>) const {
    return Grid<Dtype, NumDims, G>(p, dims_[K]...);
  }
};

// a 0-dimensional ManagedGrid is never instantiated by users; this stops the recursion of operator[]
template <typename Dtype>
class ManagedGrid<Dtype, 0> {
  template <typename D, std::size_t M>
  friend class ManagedGrid;
  std::shared_ptr<detail::Storage<Dtype>> store_;
  size_t first_ = 0;
  size_t dims_[1] = {0};

 public:
  operator Dtype() const {
    store_->to_cpu(true);
    return store_->host[first_];
  }
  ManagedGrid& operator=(Dtype v) {
    store_->to_cpu(true);
    store_->host[first_] = v;
    return *this;
  }
};

#define LMGB200_MGRID_TYPEDEFS(N)            \
  typedef ManagedGrid<float, N> MGrid##N##f; \
  typedef ManagedGrid<double, N> MGrid##N##d;
LMGB200_MGRID_TYPEDEFS(1)
LMGB200_MGRID_TYPEDEFS(2)
LMGB200_MGRID_TYPEDEFS(3)
LMGB200_MGRID_TYPEDEFS(4)
LMGB200_MGRID_TYPEDEFS(5)
LMGB200_MGRID_TYPEDEFS(6)
LMGB200_MGRID_TYPEDEFS(7)
LMGB200_MGRID_TYPEDEFS(8)
#undef LMGB200_MGRID_TYPEDEFS

}  // namespace libmolgrid

#endif
