// Helpers shared by the translation units of the compiled Python module: the process-wide
// "grids live on the GPU" switch, float3 conversion, and the float32 array argument that views
// torch tensors, numpy arrays and this module's (or the ctypes layer's) Grid / MGrid objects.
#ifndef LMGB200_BINDINGS_COMMON_H_
#define LMGB200_BINDINGS_COMMON_H_
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>

#include <memory>
#include <string>
#include <vector>

#include "libmolgrid/libmolgrid.h"

namespace lmgpy {
namespace py = pybind11;
using namespace libmolgrid;

inline bool& gpu_enabled() {
  static bool on = true;
  return on;
}

inline float3 to_float3(const py::handle& h) {
  if (py::isinstance<float3>(h)) return h.cast<float3>();
  py::sequence s = py::reinterpret_borrow<py::sequence>(h);
  if (py::len(s) != 3) throw py::value_error("a point needs three coordinates");
  return make_float3(s[0].cast<float>(), s[1].cast<float>(), s[2].cast<float>());
}

// What a Python object offers as an array: address, extents, side, element type.  The object is
// one of: a Grid of this module (attributes _lmg_ptr, shape, _lmg_cuda, _lmg_double), an MGrid of
// this module or of the ctypes layer (ongpu / gpu() / cpu(): the side the module-wide switch names is
// taken, as in python/bindings_grids.cpp:146-161), a Grid view of the ctypes layer (attribute t), a
// torch tensor (duck typed, python/bindings_grids.cpp:91-168) or a numpy array (:169-194).
struct ViewInfo {
  void* ptr = nullptr;
  std::vector<size_t> shape;
  bool cuda = false;
  bool is_double = false;
  bool writeable = true;
  py::object keep;
};

// torch's tensor type and dtypes, looked up once (null when torch is not importable)
struct TorchNames {
  PyTypeObject* tensor = nullptr;
  py::object f32, f64, i32;
};
inline const TorchNames& torch_names() {
  static TorchNames* names = [] {
    auto* n = new TorchNames();  // lives as long as the interpreter
    try {
      py::module_ torch = py::module_::import("torch");
      n->f32 = torch.attr("float32");
      n->f64 = torch.attr("float64");
      n->i32 = torch.attr("int32");
      n->tensor = reinterpret_cast<PyTypeObject*>(torch.attr("Tensor").ptr());
    } catch (py::error_already_set&) {
      n->tensor = nullptr;
    }
    return n;
  }();
  return *names;
}

// The common case of a training loop, a plain contiguous torch tensor, read with as few attribute
// look-ups as its checks need.  False: not such a tensor, take the general route.
inline bool tensor_view(const py::object& o, const std::string& name, ViewInfo& v) {
  const TorchNames& tn = torch_names();
  if (tn.tensor == nullptr || Py_TYPE(o.ptr()) != tn.tensor) return false;
  py::object dt = o.attr("dtype");
  if (dt.is(tn.f32)) v.is_double = false;
  else if (dt.is(tn.f64)) v.is_double = true;
  else throw py::value_error(name + ": tensors must be float32 or float64");
  if (!o.attr("is_contiguous")().cast<bool>()) throw py::value_error("Attempt to use non-contiguous tensor as grid");
  int dev = o.attr("get_device")().cast<int>();  // -1 for a host tensor
  v.cuda = dev >= 0;
  if (v.cuda) {
    int cur = 0;
    LMG_CUDA_CHECK(cudaGetDevice(&cur));
    if (dev != cur)
      throw py::value_error("Tensor on different device than current: " + std::to_string(dev) + " vs " +
                            std::to_string(cur));
  }
  v.ptr = reinterpret_cast<void*>(o.attr("data_ptr")().cast<size_t>());
  py::tuple shape = py::reinterpret_borrow<py::tuple>(o.attr("shape"));  // torch.Size is a tuple
  v.shape.reserve(shape.size());
  for (auto d : shape) v.shape.push_back(d.cast<size_t>());
  v.keep = o;
  return true;
}

// A resident int32 tensor with one entry per example (valid atoms of a padded batch), or a
// resident float32 (B,10) tensor of transforms: the device address, after the checks.
inline const int* device_counts(const py::object& o, size_t batch) {
  const TorchNames& tn = torch_names();
  if (tn.tensor == nullptr || !py::isinstance(o, py::reinterpret_borrow<py::object>((PyObject*)tn.tensor)))
    throw py::type_error("n_atoms: expected an int32 CUDA tensor");
  py::object dt = o.attr("dtype");
  if (!dt.is(tn.i32) || o.attr("get_device")().cast<int>() < 0 || !o.attr("is_contiguous")().cast<bool>())
    throw py::type_error("n_atoms: expected a contiguous int32 CUDA tensor");
  if (o.attr("numel")().cast<size_t>() != batch) throw py::value_error("n_atoms must have one entry per example");
  return reinterpret_cast<const int*>(o.attr("data_ptr")().cast<size_t>());
}

inline ViewInfo view_info(const py::handle& h, const std::string& name) {
  ViewInfo v;
  py::object o = py::reinterpret_borrow<py::object>(h);
  if (tensor_view(o, name, v)) return v;
  if (py::hasattr(o, "ongpu") && py::hasattr(o, "gpu")) o = gpu_enabled() ? o.attr("gpu")() : o.attr("cpu")();
  if (py::hasattr(o, "t") && py::hasattr(o, "dimension")) o = o.attr("t");  // Grid view of the ctypes layer
  if (py::hasattr(o, "_lmg_ptr")) {
    v.ptr = reinterpret_cast<void*>(o.attr("_lmg_ptr").cast<size_t>());
    v.cuda = o.attr("_lmg_cuda").cast<bool>();
    v.is_double = o.attr("_lmg_double").cast<bool>();
    for (auto d : o.attr("shape")) v.shape.push_back(d.cast<size_t>());
  } else if (py::hasattr(o, "data_ptr") && py::hasattr(o, "is_cuda")) {
    std::string dt = py::str(o.attr("dtype"));
    if (dt != "torch.float32" && dt != "torch.float64")
      throw py::value_error(name + ": tensors must be float32 or float64");
    v.is_double = dt == "torch.float64";
    if (!o.attr("is_contiguous")().cast<bool>()) throw py::value_error("Attempt to use non-contiguous tensor as grid");
    v.cuda = o.attr("is_cuda").cast<bool>();
    if (v.cuda) {
      int dev = o.attr("device").attr("index").cast<int>(), cur = 0;
      LMG_CUDA_CHECK(cudaGetDevice(&cur));
      if (dev != cur)
        throw py::value_error("Tensor on different device than current: " + std::to_string(dev) + " vs " +
                              std::to_string(cur));
    }
    v.ptr = reinterpret_cast<void*>(o.attr("data_ptr")().cast<size_t>());
    for (auto d : o.attr("shape")) v.shape.push_back(d.cast<size_t>());
  } else if (py::isinstance<py::array>(o)) {
    py::array a = py::reinterpret_borrow<py::array>(o);
    bool f32 = py::isinstance<py::array_t<float>>(a), f64 = py::isinstance<py::array_t<double>>(a);
    if ((!f32 && !f64) || !(a.flags() & py::array::c_style))
      throw py::value_error(name + ": numpy arrays must be C-contiguous float32 or float64");
    v.is_double = f64;
    v.writeable = a.writeable();
    v.ptr = a.writeable() ? a.mutable_data() : const_cast<void*>(a.data());
    for (py::ssize_t i = 0; i < a.ndim(); i++) v.shape.push_back((size_t)a.shape(i));
  } else {
    throw py::type_error(name + ": expected a Grid, MGrid, torch tensor or numpy array");
  }
  v.keep = o;
  return v;
}

// A float32 array argument of a gridding call: where it lives, its shape, and (for host arrays) its
// device copy for the duration of the call.
class Arg {
 public:
  Arg(const py::handle& h, const char* name, int ndim, bool output) : name_(name), output_(output) {
    ViewInfo v = view_info(h, name_);
    if (v.is_double)
      throw py::value_error(name_ + ": arrays must be float32 (double grids are not supported on the GPU path)");
    if (output && !v.writeable) throw py::value_error(name_ + ": array is read-only");
    cuda_ = v.cuda;
    data_ = static_cast<float*>(v.ptr);
    shape_ = v.shape;
    keep_ = v.keep;
    if ((int)shape_.size() != ndim)
      throw py::type_error(name_ + ": expected " + std::to_string(ndim) + " dimensions, got " +
                           std::to_string(shape_.size()));
    if (!cuda_) staged_.reset(new detail::Staged<float>(data_, size(), !output, output));
  }
  size_t size() const {
    size_t n = 1;
    for (size_t d : shape_) n *= d;
    return n;
  }
  size_t dim(int i) const { return shape_[i]; }
  float* dev() const { return cuda_ ? data_ : staged_->get(); }
  bool cuda() const { return cuda_; }
  void finish() {
    if (staged_) staged_->finish();
  }
  Grid<float, 1, true> g1() const { return Grid<float, 1, true>(dev(), shape_[0]); }
  Grid<float, 2, true> g2() const { return Grid<float, 2, true>(dev(), shape_[0], shape_[1]); }
  Grid<float, 3, true> g3() const { return Grid<float, 3, true>(dev(), shape_[0], shape_[1], shape_[2]); }
  Grid<float, 4, true> g4() const { return Grid<float, 4, true>(dev(), shape_[0], shape_[1], shape_[2], shape_[3]); }
  Grid<float, 5, true> g5() const {
    return Grid<float, 5, true>(dev(), shape_[0], shape_[1], shape_[2], shape_[3], shape_[4]);
  }

 private:
  std::string name_;
  bool output_;
  bool cuda_ = false;
  float* data_ = nullptr;
  std::vector<size_t> shape_;
  py::object keep_;
  std::unique_ptr<detail::Staged<float>> staged_;
};

inline int ndim_of(const py::handle& h) {
  py::object o = py::reinterpret_borrow<py::object>(h);
  if (py::hasattr(o, "shape")) return (int)py::len(o.attr("shape"));
  throw py::type_error("expected an array");
}

// Grids, MGrids, CoordinateSet, Example, ExampleVec and the overloads of GridMaker / Transform
// that take them (bindings_objects.cpp).
void bind_objects(py::module_& m, py::class_<GridMaker>& gm, py::class_<Transform>& tr);

}  // namespace lmgpy
#endif
