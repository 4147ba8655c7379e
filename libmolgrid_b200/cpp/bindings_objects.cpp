// Object types of the compiled Python module: Grid{1..8}{f,d}[CUDA], MGrid{1..8}{f,d},
// CoordinateSet, Example, ExampleVec (reference: python/bindings_grids.cpp:218-279,
// python/bindings.in.cpp:436-450,677-735) and the overloads of GridMaker / Transform that take
// them (python/bindings.in.cpp:497-520,829-918), bound from the C++ host layer.
#include <pybind11/numpy.h>
#include <pybind11/operators.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl_bind.h>

#include <cmath>
#include <cstring>
#include <utility>

#include "bindings_common.h"

PYBIND11_MAKE_OPAQUE(std::vector<float>);
PYBIND11_MAKE_OPAQUE(std::vector<libmolgrid::CoordinateSet>);
PYBIND11_MAKE_OPAQUE(std::vector<libmolgrid::Example>);

namespace lmgpy {
namespace {

template <class T>
constexpr bool is_double_v = std::is_same<T, double>::value;

// ---- views ---------------------------------------------------------------------------------

template <class G, size_t... K>
G make_grid(typename G::type* p, const std::vector<size_t>& shape, std::index_sequence<K...>) {
  return G(p, shape[K]...);
}

// A Grid view of a Python object under the reference's conversion rules: same element type, same
// number of dimensions, same side (numpy arrays only make host grids).
template <class G>
G grid_from(const py::handle& h, const char* what = "grid") {
  using T = typename G::type;
  if (py::isinstance<G>(h)) return h.cast<G>();
  ViewInfo v = view_info(h, what);
  if (v.is_double != is_double_v<T>)
    throw py::type_error(std::string(what) + ": element type does not match " + (is_double_v<T> ? "float64" : "float32"));
  if (v.shape.size() != G::N)
    throw py::type_error(std::string(what) + ": expected " + std::to_string(G::N) + " dimensions, got " +
                         std::to_string(v.shape.size()));
  if (v.cuda != G::GPU)
    throw py::type_error(std::string(what) + (G::GPU ? ": a device array is needed" : ": a host array is needed"));
  return make_grid<G>(static_cast<T*>(v.ptr), v.shape, std::make_index_sequence<G::N>());
}

template <class G>
py::tuple shape_of(const G& g) {
  py::tuple t(G::N);
  for (size_t i = 0; i < G::N; i++) t[i] = g.dimension(i);
  return t;
}

template <class G>
size_t offset_of(const G& g, const py::tuple& idx) {
  if (idx.size() != G::N) throw py::index_error("wrong number of indices");
  size_t p = 0;
  for (size_t i = 0; i < G::N; i++) {
    size_t k = idx[i].cast<size_t>();
    if (k >= g.dimension(i)) throw py::index_error("Invalid range. " + std::to_string(k) + " >= " + std::to_string(g.dimension(i)));
    p += k * g.offset(i);
  }
  return p;
}

template <class G>
typename G::type read_element(const G& g, size_t off) {
  typename G::type v;
  detail::copy_bytes(&v, g.data() + off, sizeof v, G::GPU, false);
  return v;
}

template <class G>
void write_element(const G& g, size_t off, typename G::type v) {
  detail::copy_bytes(g.data() + off, &v, sizeof v, false, G::GPU);
}

// copy between a grid and whatever array-like object of the same rank and element type
template <class G>
size_t copy_to(const G& self, const py::object& dest) {
  ViewInfo v = view_info(dest, "dest");
  if (v.is_double != is_double_v<typename G::type>) throw py::type_error("copyTo: element types differ");
  size_t n = 1;
  for (size_t d : v.shape) n *= d;
  n = std::min(n, self.size());
  detail::copy_bytes(v.ptr, self.data(), n * sizeof(typename G::type), G::GPU, v.cuda);
  return n;
}
template <class G>
size_t copy_from(const G& self, const py::object& src) {
  ViewInfo v = view_info(src, "src");
  if (v.is_double != is_double_v<typename G::type>) throw py::type_error("copyFrom: element types differ");
  size_t n = 1;
  for (size_t d : v.shape) n *= d;
  n = std::min(n, self.size());
  detail::copy_bytes(self.data(), v.ptr, n * sizeof(typename G::type), v.cuda, G::GPU);
  return n;
}

template <class G>
py::array to_numpy(const G& g) {
  std::vector<py::ssize_t> shape;
  for (size_t i = 0; i < G::N; i++) shape.push_back((py::ssize_t)g.dimension(i));
  py::array_t<typename G::type> a(shape);
  detail::copy_bytes(a.mutable_data(), g.data(), g.size() * sizeof(typename G::type), G::GPU, false);
  return std::move(a);
}

template <class G>
void define_grid(py::module_& m, const char* name) {
  using T = typename G::type;
  py::class_<G> c(m, name);
  c.def(py::init([](const py::object& o) { return grid_from<G>(o); }), py::keep_alive<1, 2>())
      .def("size", &G::size)
      .def("dimension", [](const G& g, size_t i) { return g.dimension(i); })
      .def("data", [](const G& g) { return (size_t)g.data(); })
      .def_property_readonly("shape", [](const G& g) { return shape_of(g); })
      .def_property_readonly("_lmg_ptr", [](const G& g) { return (size_t)g.data(); })
      .def_property_readonly("_lmg_cuda", [](const G&) { return G::GPU; })
      .def_property_readonly("_lmg_double", [](const G&) { return is_double_v<T>; })
      .def("__len__", [](const G& g) { return g.dimension(0); })
      .def("__getitem__", [](const G& g, const py::tuple& idx) { return read_element(g, offset_of(g, idx)); })
      .def("__setitem__", [](G& g, const py::tuple& idx, T v) { write_element(g, offset_of(g, idx), v); })
      .def("copyTo", [](const G& g, const py::object& d) { return copy_to(g, d); })
      .def("copyFrom", [](G& g, const py::object& s) { return copy_from(g, s); })
      .def("fill_zero", &G::fill_zero)
      .def("type", [](const G&) { return is_double_v<T> ? "float64" : "float32"; })
      .def("tonumpy", [](const G& g) { return to_numpy(g); })
      .def("__array__", [](const G& g, const py::args&, const py::kwargs&) { return to_numpy(g); });
  if constexpr (G::N == 1) {
    c.def("__getitem__", [](const G& g, size_t i) {
      if (i >= g.size()) throw py::index_error("Invalid range. " + std::to_string(i) + " >= " + std::to_string(g.size()));
      return read_element(g, i);
    });
    c.def("__setitem__", [](G& g, size_t i, T v) {
      if (i >= g.size()) throw py::index_error("Invalid range. " + std::to_string(i) + " >= " + std::to_string(g.size()));
      write_element(g, i, v);
    });
  } else {
    c.def("__getitem__", [](const G& g, size_t i) {
      if (i >= g.dimension(0)) throw py::index_error("Invalid range. " + std::to_string(i) + " >= " + std::to_string(g.dimension(0)));
      return g[i];
    }, py::keep_alive<0, 1>());
  }
}

template <class MG, size_t... K>
MG make_mgrid(const std::vector<size_t>& d, std::index_sequence<K...>) {
  return MG(d[K]...);
}

template <class MG>
py::tuple mshape_of(const MG& g) {
  py::tuple t(MG::N);
  for (size_t i = 0; i < MG::N; i++) t[i] = g.dimension(i);
  return t;
}

template <class MG>
size_t moffset(const MG& g, const py::tuple& idx) {
  if (idx.size() != MG::N) throw py::index_error("wrong number of indices");
  size_t p = 0;
  for (size_t i = 0; i < MG::N; i++) {
    size_t k = idx[i].cast<size_t>();
    if (k >= g.dimension(i)) throw py::index_error("Invalid range. " + std::to_string(k) + " >= " + std::to_string(g.dimension(i)));
    p = p * g.dimension(i) + k;
  }
  return p;
}

template <class MG>
void define_mgrid(py::module_& m, const char* name) {
  using T = typename MG::type;
  py::class_<MG> c(m, name);
  c.def(py::init([](const py::args& dims) {
        if (dims.size() != MG::N) throw py::type_error("wrong number of extents");
        std::vector<size_t> d;
        for (auto x : dims) d.push_back(x.cast<size_t>());
        return make_mgrid<MG>(d, std::make_index_sequence<MG::N>());
      }))
      .def("size", &MG::size)
      .def("dimension", [](const MG& g, size_t i) { return g.dimension(i); })
      .def("data", [](const MG& g) { return (size_t)g.data(); })
      .def_property_readonly("shape", [](const MG& g) { return mshape_of(g); })
      .def("__len__", [](const MG& g) { return g.dimension(0); })
      .def("cpu", [](const MG& g) { return g.cpu(); }, py::keep_alive<0, 1>())
      .def("gpu", [](const MG& g) { return g.gpu(); }, py::keep_alive<0, 1>())
      .def("clone", &MG::clone)
      .def("ongpu", &MG::ongpu)
      .def("oncpu", &MG::oncpu)
      .def("togpu", [](const MG& g, bool copy) { g.togpu(copy); }, py::arg("copy") = true)
      .def("tocpu", [](const MG& g, bool copy) { g.tocpu(copy); }, py::arg("copy") = true)
      .def("fill_zero", &MG::fill_zero)
      .def("type", [](const MG&) { return is_double_v<T> ? "float64" : "float32"; })
      .def("__getitem__",
           [](MG& g, const py::tuple& idx) {
             size_t p = moffset(g, idx);
             g.tocpu();
             return g.data()[p];
           })
      .def("__setitem__",
           [](MG& g, const py::tuple& idx, T v) {
             size_t p = moffset(g, idx);
             g.tocpu();
             g.data()[p] = v;
           })
      .def("copyTo",
           [](const MG& g, const py::object& d) {
             ViewInfo v = view_info(d, "dest");
             if (v.is_double != is_double_v<T>) throw py::type_error("copyTo: element types differ");
             size_t n = 1;
             for (size_t x : v.shape) n *= x;
             n = std::min(n, g.size());
             detail::copy_bytes(v.ptr, g.data(), n * sizeof(T), g.ongpu(), v.cuda);
             return n;
           })
      .def("copyFrom",
           [](MG& g, const py::object& s) {
             ViewInfo v = view_info(s, "src");
             if (v.is_double != is_double_v<T>) throw py::type_error("copyFrom: element types differ");
             size_t n = 1;
             for (size_t x : v.shape) n *= x;
             n = std::min(n, g.size());
             detail::copy_bytes(g.data(), v.ptr, n * sizeof(T), v.cuda, g.ongpu());
             return n;
           })
      .def("tonumpy",
           [](const MG& g) {
             std::vector<py::ssize_t> shape;
             for (size_t i = 0; i < MG::N; i++) shape.push_back((py::ssize_t)g.dimension(i));
             py::array_t<T> a(shape);
             detail::copy_bytes(a.mutable_data(), g.data(), g.size() * sizeof(T), g.ongpu(), false);
             return a;
           })
      .def("__array__", [](const py::object& self, const py::args&, const py::kwargs&) { return self.attr("tonumpy")(); });
  if constexpr (MG::N == 1) {
    c.def("__getitem__", [](MG& g, size_t i) {
      if (i >= g.size()) throw py::index_error("Invalid range. " + std::to_string(i) + " >= " + std::to_string(g.size()));
      g.tocpu();
      return g.data()[i];
    });
    c.def("__setitem__", [](MG& g, size_t i, T v) {
      if (i >= g.size()) throw py::index_error("Invalid range. " + std::to_string(i) + " >= " + std::to_string(g.size()));
      g.tocpu();
      g.data()[i] = v;
    });
  } else {
    c.def("__getitem__", [](const MG& g, size_t i) {
      if (i >= g.dimension(0)) throw py::index_error("Invalid range. " + std::to_string(i) + " >= " + std::to_string(g.dimension(0)));
      return g[i];
    });
  }
}

template <size_t N>
void define_rank(py::module_& m) {
  std::string n = std::to_string(N);
  define_grid<Grid<float, N, false>>(m, ("Grid" + n + "f").c_str());
  define_grid<Grid<double, N, false>>(m, ("Grid" + n + "d").c_str());
  define_grid<Grid<float, N, true>>(m, ("Grid" + n + "fCUDA").c_str());
  define_grid<Grid<double, N, true>>(m, ("Grid" + n + "dCUDA").c_str());
  define_mgrid<ManagedGrid<float, N>>(m, ("MGrid" + n + "f").c_str());
  define_mgrid<ManagedGrid<double, N>>(m, ("MGrid" + n + "d").c_str());
}

// ---- CoordinateSet / Example helpers that the C++ containers leave to their callers --------

// float32 contents of an array-like object on the host (copied)
std::vector<float> host_floats(const py::object& o, size_t ndim, std::vector<size_t>* shape, const char* what) {
  ViewInfo v = view_info(o, what);
  if (v.is_double) throw py::type_error(std::string(what) + ": float32 needed");
  if (v.shape.size() != ndim)
    throw py::type_error(std::string(what) + ": expected " + std::to_string(ndim) + " dimensions");
  size_t n = 1;
  for (size_t d : v.shape) n *= d;
  std::vector<float> out(n);
  detail::copy_bytes(out.data(), v.ptr, n * sizeof(float), v.cuda, false);
  if (shape) *shape = v.shape;
  return out;
}

CoordinateSet coordinate_set_from(const py::object& coords, const py::object& types, const py::object& radii,
                                  const py::object& max_type) {
  std::vector<size_t> cs, ts, rs;
  std::vector<float> c = host_floats(coords, 2, &cs, "coords");
  int tnd = ndim_of(types);
  std::vector<float> t = host_floats(types, tnd, &ts, "types");
  std::vector<float> r = host_floats(radii, 1, &rs, "radii");
  if (cs[1] != 3) throw py::value_error("Coordinates have wrong secondary dimension");
  Grid2f cg(c.data(), cs[0], cs[1]);
  Grid1f rg(r.data(), rs[0]);
  if (tnd == 1) {
    if (max_type.is_none()) throw py::type_error("index-typed CoordinateSet needs the number of types");
    Grid1f tg(t.data(), ts[0]);
    return CoordinateSet(cg, tg, rg, max_type.cast<unsigned>());
  }
  Grid2f tg(t.data(), ts[0], ts[1]);
  return CoordinateSet(cg, tg, rg);
}

// CoordinateSet::make_vector_types (src/coordinateset.cpp:187-212)
void make_vector_types(CoordinateSet& s, bool include_dummy_type, const std::vector<float>& type_radii) {
  unsigned n = (unsigned)s.type_index.size();
  if (!type_radii.empty() && type_radii.size() != s.max_type)
    throw std::invalid_argument("Type radii size " + itoa(type_radii.size()) + " does not equal max type " +
                                itoa(s.max_type));
  if (include_dummy_type) s.max_type++;
  s.type_vector = MGrid2f(n, s.max_type);
  for (unsigned i = 0; i < n; i++) {
    unsigned t = (unsigned)s.type_index(i);
    if (t < s.max_type) s.type_vector(i, t) = 1.0f;
  }
  if (!type_radii.empty()) {
    MGrid1f r(s.max_type);
    for (size_t i = 0; i < type_radii.size(); i++) r(i) = type_radii[i];
    s.radii = r;
  }
}

// CoordinateSet::sum_types (src/coordinateset.cpp:352-374) into a host or device array
void sum_types(const CoordinateSet& s, const py::object& sum, bool zerofirst) {
  ViewInfo v = view_info(sum, "sum");
  if (v.is_double || v.shape.size() != 1) throw py::type_error("sum: a one-dimensional float32 array is needed");
  if (v.shape[0] != s.num_types())
    throw std::invalid_argument("Type sum output dimension does not match number of types: " + itoa(v.shape[0]) +
                                " vs " + itoa(s.num_types()));
  bool vec = s.type_vector.size() > 0;
  unsigned n = s.size(), T = s.num_types();
  float* out = static_cast<float*>(v.ptr);
  if (v.cuda) {
    int* dstatus = nullptr;
    LMG_CUDA_CHECK(cudaMalloc(&dstatus, sizeof(int)));
    int rc;
    if (vec) rc = lmg_sum_types(nullptr, s.type_vector.gpu().data(), (int)n, (int)T, out, zerofirst, dstatus, nullptr);
    else rc = lmg_sum_types(s.type_index.gpu().data(), nullptr, (int)n, (int)T, out, zerofirst, dstatus, nullptr);
    int st = 0;
    cudaError_t e = cudaMemcpy(&st, dstatus, sizeof st, cudaMemcpyDeviceToHost);
    cudaFree(dstatus);
    detail::check(rc);
    LMG_CUDA_CHECK(e);
    if (st) throw std::out_of_range("Somehow an index type is too large (internal error).");
    return;
  }
  if (zerofirst) std::memset(out, 0, sizeof(float) * T);
  if (!vec) {
    Grid1f ti = s.type_index.cpu();
    for (unsigned i = 0; i < n; i++) {
      int t = (int)std::round(ti(i));
      if (t < 0) continue;
      if (t >= (int)T) throw std::out_of_range("Somehow an index type is too large (internal error).");
      out[t] += 1.0f;
    }
  } else {
    Grid2f tv = s.type_vector.cpu();
    for (unsigned i = 0; i < n; i++)
      for (unsigned j = 0; j < T; j++) out[j] += tv(i, j);
  }
}

// Example::sum_types (src/example.cpp:355-374)
void example_sum_types(const Example& ex, const py::object& sum, bool unique_types) {
  ViewInfo v = view_info(sum, "sum");
  if (v.is_double || v.shape.size() != 1) throw py::type_error("sum: a one-dimensional float32 array is needed");
  size_t NT = ex.num_types(unique_types);
  if (v.shape[0] != NT)
    throw std::invalid_argument("Size of sum output doesn't match number of types in example: " + itoa(v.shape[0]) +
                                " vs " + itoa(NT));
  size_t offset = 0;
  float* base = static_cast<float*>(v.ptr);
  for (const CoordinateSet& s : ex.sets) {
    if (unique_types) {
      unsigned nt = s.num_types();
      if (nt == 0) continue;
      py::object sub = v.cuda ? py::cast(Grid<float, 1, true>(base + offset, nt)) : py::cast(Grid<float, 1, false>(base + offset, nt));
      offset += nt;
      sum_types(s, sub, true);
    } else {
      sum_types(s, sum, false);
    }
  }
}

bool example_has_vector_types(const Example& ex, unsigned start) {
  bool any = false;
  for (size_t i = start; i < ex.sets.size(); i++)
    if (ex.sets[i].size() > 0) { any = true; if (!ex.sets[i].has_vector_types()) return false; }
  (void)any;
  return true;
}
bool example_has_index_types(const Example& ex, unsigned start) {
  for (size_t i = start; i < ex.sets.size(); i++)
    if (ex.sets[i].size() > 0 && !ex.sets[i].has_indexed_types()) return false;
  return true;
}

// ---- GridMaker / Transform with objects -----------------------------------------------------

py::object arg_or(const py::args& a, size_t i, const py::kwargs& kw, std::initializer_list<const char*> names,
                  const py::object& dflt = py::none()) {
  if (i < a.size()) return py::reinterpret_borrow<py::object>(a[i]);
  for (const char* n : names)
    if (kw.contains(n)) return py::reinterpret_borrow<py::object>(kw[n]);
  return dflt;
}

bool is_example_list(const py::object& o) {
  if (py::isinstance<std::vector<Example>>(o)) return true;
  if (!py::isinstance<py::list>(o) && !py::isinstance<py::tuple>(o)) return false;
  py::sequence s = py::reinterpret_borrow<py::sequence>(o);
  return py::len(s) == 0 || py::isinstance<Example>(s[0]);
}

std::vector<Example> to_examples(const py::object& o) {
  if (py::isinstance<std::vector<Example>>(o)) return o.cast<std::vector<Example>>();
  std::vector<Example> v;
  for (auto e : py::reinterpret_borrow<py::sequence>(o)) v.push_back(e.cast<Example>());
  return v;
}

void gm_forward_objects(GridMaker& gm, const py::args& a, const py::kwargs& kw) {
  py::object a0 = arg_or(a, 0, kw, {"example", "examples", "examplevec", "center"});
  if (a0.is_none()) throw py::type_error("forward: missing arguments");
  if (py::isinstance<Example>(a0)) {
    const Example& ex = a0.cast<const Example&>();
    py::object a1 = arg_or(a, 1, kw, {"transform", "grid"});
    if (py::isinstance<Transform>(a1)) {
      Arg o(arg_or(a, 2, kw, {"grid"}), "grid", 4, true);
      {
        Grid<float, 4, true> og = o.g4();
        gm.forward(ex, a1.cast<const Transform&>(), og);
      }
      o.finish();
      return;
    }
    Arg o(a1, "grid", 4, true);
    float rt = arg_or(a, 2, kw, {"random_translation"}, py::float_(0.0)).cast<float>();
    bool rr = arg_or(a, 3, kw, {"random_rotation"}, py::bool_(false)).cast<bool>();
    {
      Grid<float, 4, true> og = o.g4();
      gm.forward(ex, og, rt, rr);
    }
    o.finish();
    return;
  }
  if (is_example_list(a0)) {
    std::vector<Example> exs = to_examples(a0);
    Arg o(arg_or(a, 1, kw, {"grid"}), "grid", 5, true);
    float rt = arg_or(a, 2, kw, {"random_translation"}, py::float_(0.0)).cast<float>();
    bool rr = arg_or(a, 3, kw, {"random_rotation"}, py::bool_(false)).cast<bool>();
    {
      Grid<float, 5, true> og = o.g5();
      gm.forward(exs, og, rt, rr);
    }
    o.finish();
    return;
  }
  py::object a1 = arg_or(a, 1, kw, {"coordinate_set", "c", "in"});
  if (py::isinstance<CoordinateSet>(a1)) {
    float3 ctr = to_float3(a0);
    Arg o(arg_or(a, 2, kw, {"grid"}), "grid", 4, true);
    {
      Grid<float, 4, true> og = o.g4();
      gm.forward(ctr, a1.cast<const CoordinateSet&>(), og);
    }
    o.finish();
    return;
  }
  throw py::type_error("forward: no overload takes these arguments");
}

void gm_backward_objects(GridMaker& gm, const py::object& center, const CoordinateSet& in, const py::object& diff,
                         const py::object& atomic_gradients, const py::object& type_gradients) {
  float3 ctr = to_float3(center);
  Arg d(diff, "diff", 4, false), ag(atomic_gradients, "atomic_gradients", 2, true);
  if (type_gradients.is_none()) {
    Grid<float, 2, true> g = ag.g2();
    gm.backward(ctr, in, d.g4(), g);
  } else {
    Arg tg(type_gradients, "type_gradients", 2, true);
    Grid<float, 2, true> g = ag.g2(), g2 = tg.g2();
    gm.backward(ctr, in, d.g4(), g, g2);
    tg.finish();
  }
  ag.finish();
}

}  // namespace

void bind_objects(py::module_& m, py::class_<GridMaker>& gm, py::class_<Transform>& tr) {
  define_rank<1>(m);
  define_rank<2>(m);
  define_rank<3>(m);
  define_rank<4>(m);
  define_rank<5>(m);
  define_rank<6>(m);
  define_rank<7>(m);
  define_rank<8>(m);

  py::bind_vector<std::vector<float>>(m, "FloatVec");
  py::implicitly_convertible<py::list, std::vector<float>>();
  py::implicitly_convertible<py::tuple, std::vector<float>>();

  py::class_<CoordinateSet>(m, "CoordinateSet")
      .def(py::init<>())
      .def(py::init([](const CoordinateSet& rec, const CoordinateSet& lig, bool unique_index_types) {
             Example e;
             e.sets = {rec, lig};
             return e.merge_coordinates(0, unique_index_types);
           }),
           py::arg("rec"), py::arg("lig"), py::arg("unique_index_types") = true)
      .def(py::init([](const py::object& coords, const py::object& types, const py::object& radii,
                       const py::object& max_type) { return coordinate_set_from(coords, types, radii, max_type); }),
           py::arg("coords"), py::arg("types"), py::arg("radii"), py::arg("max_type") = py::none())
      .def("has_indexed_types", &CoordinateSet::has_indexed_types)
      .def("has_vector_types", &CoordinateSet::has_vector_types)
      .def("make_vector_types",
           [](CoordinateSet& s, bool dummy, const std::vector<float>& radii) { make_vector_types(s, dummy, radii); },
           py::arg("include_dummy_type") = false, py::arg("type_radii") = std::vector<float>())
      .def("size", &CoordinateSet::size)
      .def("num_types", &CoordinateSet::num_types)
      .def("center", &CoordinateSet::center)
      .def("clone", &CoordinateSet::clone)
      .def("togpu", &CoordinateSet::togpu, py::arg("copy") = true)
      .def("tocpu", &CoordinateSet::tocpu, py::arg("copy") = true)
      .def("copyTo",
           [](const CoordinateSet& s, const py::object& c, const py::object& t, const py::object& r) {
             py::object self = py::cast(s);
             size_t n = self.attr("coords").attr("copyTo")(c).cast<size_t>();
             bool vec = ndim_of(t) == 2;
             self.attr(vec ? "type_vector" : "type_index").attr("copyTo")(t);
             self.attr("radii").attr("copyTo")(r);
             return n / 3;
           })
      .def("sum_types", [](const CoordinateSet& s, const py::object& sum, bool zerofirst) { sum_types(s, sum, zerofirst); },
           py::arg("sum"), py::arg("zerofirst") = true)
      .def_readwrite("coords", &CoordinateSet::coords)
      .def_readwrite("type_index", &CoordinateSet::type_index)
      .def_readwrite("type_vector", &CoordinateSet::type_vector)
      .def_readwrite("radii", &CoordinateSet::radii)
      .def_readwrite("max_type", &CoordinateSet::max_type)
      .def_property_readonly("src", [](const CoordinateSet& s) -> py::object {
        if (s.src == nullptr) return py::none();
        return py::str(s.src);
      });

  py::bind_vector<std::vector<CoordinateSet>>(m, "CoordinateSetVec");

  py::class_<Example>(m, "Example")
      .def(py::init<>())
      .def("num_coordinates", &Example::num_coordinates)
      .def("num_types", &Example::num_types, py::arg("unique_index_type") = true)
      .def("merge_coordinates", &Example::merge_coordinates, py::arg("start") = 0, py::arg("unique_index_types") = true)
      .def("togpu", [](Example& e) { for (auto& s : e.sets) s.togpu(); })
      .def("tocpu", [](Example& e) { for (auto& s : e.sets) s.tocpu(); })
      .def("has_vector_types", &example_has_vector_types, py::arg("start") = 0)
      .def("has_index_types", &example_has_index_types, py::arg("start") = 0)
      .def("sum_types", &example_sum_types, py::arg("sum"), py::arg("unique_types") = true)
      .def_readwrite("coord_sets", &Example::sets)
      .def_readwrite("labels", &Example::labels)
      .def_readwrite("group", &Example::group)
      .def_readwrite("seqcont", &Example::seqcont);

  py::bind_vector<std::vector<Example>>(m, "ExampleVec")
      .def("extract_labels",
           [](const std::vector<Example>& v, const py::object& out) {
             if (v.empty()) return;
             size_t nl = v[0].labels.size();
             std::vector<float> host(v.size() * nl);
             for (size_t i = 0; i < v.size(); i++) {
               if (v[i].labels.size() != nl) throw std::logic_error("Non-uniform number of labels in examples");
               for (size_t j = 0; j < nl; j++) host[i * nl + j] = v[i].labels[j];
             }
             ViewInfo o = view_info(out, "out");
             if (o.is_double || o.shape.size() != 2 || o.shape[0] != v.size() || o.shape[1] != nl)
               throw std::out_of_range("Incorrect output grid shape for labels");
             detail::copy_bytes(o.ptr, host.data(), host.size() * sizeof(float), false, o.cuda);
           })
      .def("extract_label",
           [](const std::vector<Example>& v, int labelpos, const py::object& out) {
             std::vector<float> host(v.size());
             for (size_t i = 0; i < v.size(); i++) {
               if (labelpos < 0 || (size_t)labelpos >= v[i].labels.size())
                 throw std::out_of_range("labelpos invalid: " + itoa(labelpos));
               host[i] = v[i].labels[labelpos];
             }
             ViewInfo o = view_info(out, "out");
             if (o.is_double || o.shape.size() != 1 || o.shape[0] != v.size())
               throw std::out_of_range("Incorrect output grid shape for label");
             detail::copy_bytes(o.ptr, host.data(), host.size() * sizeof(float), false, o.cuda);
           })
      .def("sum_types",
           [](const std::vector<Example>& v, const py::object& sum, bool unique_types) {
             ViewInfo o = view_info(sum, "sum");
             if (o.is_double || o.shape.size() != 2 || o.shape[0] != v.size())
               throw std::invalid_argument("Type sum output has the wrong shape");
             float* base = static_cast<float*>(o.ptr);
             for (size_t i = 0; i < v.size(); i++) {
               py::object row = o.cuda ? py::cast(Grid<float, 1, true>(base + i * o.shape[1], o.shape[1]))
                                       : py::cast(Grid<float, 1, false>(base + i * o.shape[1], o.shape[1]));
               example_sum_types(v[i], row, unique_types);
             }
           },
           py::arg("sum"), py::arg("unique_types") = true);

  gm.def("forward", [](GridMaker& g, const py::args& a, const py::kwargs& kw) { gm_forward_objects(g, a, kw); });
  // the overloads with typed object arguments are tried before the array overloads bound earlier
  // (an array overload accepts any object and fails inside the call instead of passing it on)
  gm.def("backward", &gm_backward_objects, py::arg("center"), py::arg("coordinate_set"), py::arg("diff"),
         py::arg("atomic_gradients"), py::arg("type_gradients") = py::none(), py::prepend());
  gm.def("backward_gradients",
         [](GridMaker& g, const py::object& center, const CoordinateSet& in, const py::object& diff,
            const py::object& atom_gradients, const py::object& type_gradients, const py::object& diffdiff,
            const py::object& atom_diffdiff, const py::object& type_diffdiff) {
           Arg d(diff, "diff", 4, false), ag(atom_gradients, "atom_gradients", 2, false),
               tg(type_gradients, "type_gradients", 2, false), dd(diffdiff, "diffdiff", 4, true),
               add(atom_diffdiff, "atom_diffdiff", 2, true), tdd(type_diffdiff, "type_diffdiff", 2, true);
           float3 ctr = to_float3(center);
           Grid<float, 4, true> g4 = dd.g4();
           Grid<float, 2, true> ga = add.g2(), gt = tdd.g2();
           g.backward_gradients(ctr, in, d.g4(), ag.g2(), tg.g2(), g4, ga, gt);
           dd.finish();
           add.finish();
           tdd.finish();
         }, py::prepend());
  gm.def("backward_relevance",
         [](GridMaker& g, const py::object& center, const CoordinateSet& in, const py::object& density,
            const py::object& diff, const py::object& relevance) {
           Arg de(density, "density", 4, false), d(diff, "diff", 4, false), rel(relevance, "relevance", 1, true);
           float3 ctr = to_float3(center);
           Grid<float, 1, true> r = rel.g1();
           g.backward_relevance(ctr, in, de.g4(), d.g4(), r);
           rel.finish();
         }, py::prepend());

  tr.def("forward", [](const Transform& t, const CoordinateSet& in, CoordinateSet& out, bool dotranslate) {
           t.forward(in, out, dotranslate);
         }, py::arg("in"), py::arg("out"), py::arg("dotranslate") = true, py::prepend());
  tr.def("forward", [](const Transform& t, const Example& in, Example& out, bool dotranslate) {
           t.forward(in, out, dotranslate);
         }, py::arg("in"), py::arg("out"), py::arg("dotranslate") = true, py::prepend());
}

}  // namespace lmgpy
