// Compiled Python module `molgrid_native`: the gridding classes bound from the C++ host layer with
// pybind11, with the names, keywords and overload sets of the reference's module for this path
// (python/bindings.in.cpp:400-408,455-520,816-943) and its argument conversion rules
// (python/bindings_grids.cpp:91-194): torch tensors (duck typed), C-contiguous float32 numpy arrays
// (host side only) and this package's Grid / MGrid objects are viewed in place; a CUDA tensor on
// another device than the current one, or a non-contiguous tensor, is a ValueError.  Host arrays are
// staged through the device around the call.  The GIL is released while the C ABI runs, so one
// Python thread per GPU can drive several GPUs.
#include <pybind11/numpy.h>
#include <pybind11/operators.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <memory>
#include <string>
#include <vector>

#include "bindings_common.h"
#include "libmolgrid/libmolgrid.h"

namespace py = pybind11;
using namespace libmolgrid;

namespace {

using namespace lmgpy;

// forward(center, coords, types, radii, grid): index or vector types, single example or batch
// (plus, for batches, this library's additions: `transforms`, a (B,10) float32 CUDA tensor of
// lmg_transform rows applied inside the kernels, and `n_atoms`, an int32 CUDA tensor of valid atoms)
void gm_forward_arrays(const GridMaker& gm, const py::object& center, const py::object& coords,
                       const py::object& types, const py::object& radii, const py::object& out,
                       const py::object& transforms, const py::object& n_atoms) {
  bool batched = ndim_of(coords) == 3;
  if (!batched) {
    if (!transforms.is_none() || !n_atoms.is_none())
      throw py::type_error("transforms= and n_atoms= belong to the batched overload");
    Arg c(coords, "coords", 2, false), r(radii, "radii", 1, false), o(out, "grid", 4, true);
    bool vec = ndim_of(types) == 2;
    Arg t(types, "types", vec ? 2 : 1, false);
    float3 ctr = to_float3(center);
    {
      py::gil_scoped_release nogil;
      Grid<float, 4, true> og = o.g4();
      if (vec) gm.forward(ctr, c.g2(), t.g2(), r.g1(), og);
      else gm.forward(ctr, c.g2(), t.g1(), r.g1(), og);
    }
    o.finish();
    return;
  }
  Arg ce(center, "centers", 2, false), c(coords, "coords", 3, false), r(radii, "radii", 2, false),
      o(out, "grid", 5, true);
  bool vec = ndim_of(types) == 3;
  Arg t(types, "types", vec ? 3 : 2, false);
  const lmg_transform* trs = nullptr;
  const int* counts = nullptr;
  std::unique_ptr<Arg> trarg;
  if (!transforms.is_none()) {
    trarg.reset(new Arg(transforms, "transforms", 2, false));
    if (trarg->dim(0) != c.dim(0) || trarg->dim(1) != 10) throw py::value_error("transforms must be float32 of shape (batch, 10)");
    trs = reinterpret_cast<const lmg_transform*>(trarg->dev());
  }
  if (!n_atoms.is_none()) counts = device_counts(n_atoms, c.dim(0));
  {
    py::gil_scoped_release nogil;
    Grid<float, 5, true> og = o.g5();
    if (vec) gm.forward<3>(ce.g2(), c.g3(), t.g3(), r.g2(), og, trs, counts);
    else gm.forward<2>(ce.g2(), c.g3(), t.g2(), r.g2(), og, trs, counts);
  }
  o.finish();
}

// backward for a batch (an addition of this library; the reference's overloads take one example)
void gm_backward_batch(const GridMaker& gm, const py::object& center, const py::object& coords,
                       const py::object& types, const py::object& radii, const py::object& diff,
                       const py::object& atom_gradients, const py::object& type_gradients,
                       const py::object& transforms, const py::object& n_atoms) {
  Arg ce(center, "centers", 2, false), c(coords, "coords", 3, false), r(radii, "radii", 2, false),
      d(diff, "diff", 5, false), ag(atom_gradients, "atom_gradients", 3, true);
  bool vec = ndim_of(types) == 3;
  Arg t(types, "types", vec ? 3 : 2, false);
  std::unique_ptr<Arg> tg, trarg;
  float* tgp = nullptr;
  if (!type_gradients.is_none()) {
    tg.reset(new Arg(type_gradients, "type_gradients", 3, true));
    if (tg->dim(0) != c.dim(0) || tg->dim(1) != c.dim(1) || !vec || tg->dim(2) != t.dim(2))
      throw py::value_error("type_gradients must have the shape of the type vectors");
    tgp = tg->dev();
  }
  const lmg_transform* trs = nullptr;
  const int* counts = nullptr;
  if (!transforms.is_none()) {
    trarg.reset(new Arg(transforms, "transforms", 2, false));
    if (trarg->dim(0) != c.dim(0) || trarg->dim(1) != 10) throw py::value_error("transforms must be float32 of shape (batch, 10)");
    trs = reinterpret_cast<const lmg_transform*>(trarg->dev());
  }
  if (!n_atoms.is_none()) counts = device_counts(n_atoms, c.dim(0));
  {
    py::gil_scoped_release nogil;
    Grid<float, 3, true> g = ag.g3();
    if (vec) gm.backward<3>(ce.g2(), c.g3(), t.g3(), r.g2(), d.g5(), g, tgp, trs, counts);
    else gm.backward<2>(ce.g2(), c.g3(), t.g2(), r.g2(), d.g5(), g, tgp, trs, counts);
  }
  if (tg) tg->finish();
  ag.finish();
}

void gm_backward_arrays(const GridMaker& gm, const py::object& center, const py::object& coords,
                        const py::object& types, const py::object& radii, const py::object& diff,
                        const py::object& atom_gradients, const py::object& type_gradients,
                        const py::object& transforms, const py::object& n_atoms) {
  if (ndim_of(coords) == 3) {
    gm_backward_batch(gm, center, coords, types, radii, diff, atom_gradients, type_gradients, transforms, n_atoms);
    return;
  }
  if (!transforms.is_none() || !n_atoms.is_none())
    throw py::type_error("transforms= and n_atoms= belong to the batched overload");
  Arg c(coords, "coords", 2, false), r(radii, "radii", 1, false), d(diff, "diff", 4, false),
      ag(atom_gradients, "atom_gradients", 2, true);
  bool vec = ndim_of(types) == 2;
  Arg t(types, "types", vec ? 2 : 1, false);
  float3 ctr = to_float3(center);
  if (!vec) {
    if (!type_gradients.is_none()) throw py::type_error("type_gradients given with index types");
    py::gil_scoped_release nogil;
    Grid<float, 2, true> g = ag.g2();
    gm.backward(ctr, c.g2(), t.g1(), r.g1(), d.g4(), g);
  } else {
    if (type_gradients.is_none()) throw py::type_error("vector types need type_gradients");
    Arg tg(type_gradients, "type_gradients", 2, true);
    {
      py::gil_scoped_release nogil;
      Grid<float, 2, true> g = ag.g2(), g2 = tg.g2();
      gm.backward(ctr, c.g2(), t.g2(), r.g1(), d.g4(), g, g2);
    }
    tg.finish();
  }
  ag.finish();
}

void transform_apply(const Transform& tr, const py::object& in, const py::object& out, bool dotranslate, bool fwd) {
  Arg i(in, "in", 2, false), o(out, "out", 2, true);
  {
    py::gil_scoped_release nogil;
    Grid<float, 2, true> og = o.g2();
    if (fwd) tr.forward(i.g2(), og, dotranslate);
    else tr.backward(i.g2(), og, dotranslate);
  }
  o.finish();
}

}  // namespace

PYBIND11_MODULE(molgrid_native, m) {
  m.doc() = "GridMaker, GridInterpolater, Transform, Quaternion and float3 of libmolgrid's gridding path on B200";

  m.def("set_random_seed", [](unsigned seed) { set_random_seed(seed); }, py::arg("seed"));
  m.def("set_gpu_enabled", [](bool on) { gpu_enabled() = on; });
  m.def("get_gpu_enabled", []() { return gpu_enabled(); });
  m.def("set_gpu_device", [](int dev) { LMG_CUDA_CHECK(cudaSetDevice(dev)); });
  m.def("get_gpu_device", []() {
    int dev = 0;
    LMG_CUDA_CHECK(cudaGetDevice(&dev));
    return dev;
  });

  py::class_<float3>(m, "float3")
      .def(py::init([](float x, float y, float z) { return make_float3(x, y, z); }), py::arg("x") = 0.f,
           py::arg("y") = 0.f, py::arg("z") = 0.f)
      .def(py::init([](const py::sequence& s) { return to_float3(s); }))
      .def("__getitem__",
           [](const float3& f, int i) {
             if (i < 0 || i > 2) throw py::index_error("float3 index out of range");
             return i == 0 ? f.x : i == 1 ? f.y : f.z;
           })
      .def("__len__", [](const float3&) { return 3; })
      .def("__repr__",
           [](const float3& f) {
             return "float3(" + std::to_string(f.x) + ", " + std::to_string(f.y) + ", " + std::to_string(f.z) + ")";
           })
      .def_readwrite("x", &float3::x)
      .def_readwrite("y", &float3::y)
      .def_readwrite("z", &float3::z);
  py::implicitly_convertible<py::tuple, float3>();
  py::implicitly_convertible<py::list, float3>();

  py::class_<Quaternion>(m, "Quaternion")
      .def(py::init<>())
      .def(py::init<float, float, float, float>())
      .def("R_component_1", &Quaternion::R_component_1)
      .def("R_component_2", &Quaternion::R_component_2)
      .def("R_component_3", &Quaternion::R_component_3)
      .def("R_component_4", &Quaternion::R_component_4)
      .def("real", &Quaternion::real)
      .def("conj", &Quaternion::conj)
      .def("norm", &Quaternion::norm)
      .def("rotate", &Quaternion::rotate, py::arg("x"), py::arg("y"), py::arg("z"))
      .def("transform", [](const Quaternion& q, float x, float y, float z, const py::object& c,
                           const py::object& t) { return q.transform(x, y, z, to_float3(c), to_float3(t)); })
      .def("inverse", &Quaternion::inverse)
      .def(py::self * py::self)
      .def(py::self *= py::self)
      .def(py::self / py::self)
      .def(py::self /= py::self)
      .def(py::self == py::self);

  py::class_<Transform> tr_class(m, "Transform");
  tr_class
      .def(py::init<>())
      .def(py::init([](const Quaternion& q) { return Transform(q); }))
      .def(py::init([](const Quaternion& q, const py::object& c) { return Transform(q, to_float3(c)); }))
      .def(py::init([](const Quaternion& q, const py::object& c, const py::object& t) {
        return Transform(q, to_float3(c), to_float3(t));
      }))
      .def(py::init([](const py::object& center, float random_translate, bool random_rotation) {
             return Transform(to_float3(center), random_translate, random_rotation);
           }),
           py::arg("center"), py::arg("random_translate") = 0.0f, py::arg("random_rotation") = false)
      .def("get_quaternion", &Transform::get_quaternion)
      .def("get_rotation_center", &Transform::get_rotation_center)
      .def("get_translation", &Transform::get_translation)
      .def("set_quaternion", &Transform::set_quaternion)
      .def("set_rotation_center", [](Transform& t, const py::object& c) { t.set_rotation_center(to_float3(c)); })
      .def("set_translation", [](Transform& t, const py::object& c) { t.set_translation(to_float3(c)); })
      .def("forward", [](const Transform& t, const py::object& in, const py::object& out,
                         bool dotranslate) { transform_apply(t, in, out, dotranslate, true); },
           py::arg("in"), py::arg("out"), py::arg("dotranslate") = true)
      .def("backward", [](const Transform& t, const py::object& in, const py::object& out,
                          bool dotranslate) { transform_apply(t, in, out, dotranslate, false); },
           py::arg("in"), py::arg("out"), py::arg("dotranslate") = true);

  py::class_<GridMaker> gm_class(m, "GridMaker");
  gm_class
      .def(py::init<float, float, bool, bool, float, float>(), py::arg("resolution") = 0.5f,
           py::arg("dimension") = 23.5f, py::arg("binary") = false, py::arg("radius_type_indexed") = false,
           py::arg("radius_scale") = 1.0f, py::arg("gaussian_radius_multiple") = 1.0f)
      .def("spatial_grid_dimensions",
           [](const GridMaker& g) {
             int d = (int)g.get_first_dim();
             return py::make_tuple(d, d, d);
           })
      .def("grid_dimensions",
           [](const GridMaker& g, int ntypes) {
             int d = (int)g.get_first_dim();
             return py::make_tuple(ntypes, d, d, d);
           })
      .def("get_resolution", &GridMaker::get_resolution)
      .def("set_resolution", &GridMaker::set_resolution)
      .def("get_dimension", &GridMaker::get_dimension)
      .def("set_dimension", &GridMaker::set_dimension)
      .def("get_binary", &GridMaker::get_binary)
      .def("set_binary", &GridMaker::set_binary)
      .def("get_radii_type_indexed", &GridMaker::get_radii_type_indexed)
      .def("set_radii_type_indexed", &GridMaker::set_radii_type_indexed)
      .def("forward", &gm_forward_arrays, py::arg("center"), py::arg("coords"), py::arg("types"), py::arg("radii"),
           py::arg("grid"), py::arg("transforms") = py::none(), py::arg("n_atoms") = py::none())
      .def("backward", &gm_backward_arrays, py::arg("center"), py::arg("coords"), py::arg("types"),
           py::arg("radii"), py::arg("diff"), py::arg("atom_gradients"), py::arg("type_gradients") = py::none(),
           py::arg("transforms") = py::none(), py::arg("n_atoms") = py::none())
      .def("backward_gradients",
           [](GridMaker& gm, const py::object& center, const py::object& coords, const py::object& types,
              const py::object& radii, const py::object& diff, const py::object& atom_gradients,
              const py::object& type_gradients, const py::object& diffdiff, const py::object& atom_diffdiff,
              const py::object& type_diffdiff) {
             Arg c(coords, "coords", 2, false), t(types, "type_vectors", 2, false), r(radii, "radii", 1, false),
                 d(diff, "diff", 4, false), ag(atom_gradients, "atom_gradients", 2, false),
                 tg(type_gradients, "type_gradients", 2, false), dd(diffdiff, "diffdiff", 4, true),
                 add(atom_diffdiff, "atom_diffdiff", 2, true), tdd(type_diffdiff, "type_diffdiff", 2, true);
             float3 ctr = to_float3(center);
             {
               py::gil_scoped_release nogil;
               Grid<float, 4, true> g4 = dd.g4();
               Grid<float, 2, true> ga = add.g2(), gt = tdd.g2();
               gm.backward_gradients(ctr, c.g2(), t.g2(), r.g1(), d.g4(), ag.g2(), tg.g2(), g4, ga, gt);
             }
             dd.finish();
             add.finish();
             tdd.finish();
           })
      .def("backward_relevance",
           [](const GridMaker& gm, const py::object& center, const py::object& coords, const py::object& types,
              const py::object& radii, const py::object& density, const py::object& diff,
              const py::object& relevance) {
             Arg c(coords, "coords", 2, false), t(types, "type_index", 1, false), r(radii, "radii", 1, false),
                 de(density, "density", 4, false), d(diff, "diff", 4, false), rel(relevance, "relevance", 1, true);
             float3 ctr = to_float3(center);
             {
               py::gil_scoped_release nogil;
               Grid<float, 1, true> g = rel.g1();
               gm.backward_relevance(ctr, c.g2(), t.g1(), r.g1(), de.g4(), d.g4(), g);
             }
             rel.finish();
           })
      .def("check_types", &GridMaker::check_types);

  py::class_<GridInterpolater>(m, "GridInterpolater")
      .def(py::init<float, float, float, float>(), py::arg("in_resolution") = 0.5f, py::arg("in_dimension") = 23.5f,
           py::arg("out_resolution") = 0.5f, py::arg("out_dimension") = 23.5f)
      .def("get_in_resolution", &GridInterpolater::get_in_resolution)
      .def("get_out_resolution", &GridInterpolater::get_out_resolution)
      .def("get_in_dimension", &GridInterpolater::get_in_dimension)
      .def("get_out_dimension", &GridInterpolater::get_out_dimension)
      .def("set_in_resolution", &GridInterpolater::set_in_resolution)
      .def("set_out_resolution", &GridInterpolater::set_out_resolution)
      .def("set_in_dimension", &GridInterpolater::set_in_dimension)
      .def("set_out_dimension", &GridInterpolater::set_out_dimension)
      .def("forward",
           [](const GridInterpolater& gi, const py::object& in, const Transform& tr, const py::object& out) {
             Arg i(in, "in", 4, false), o(out, "out", 4, true);
             {
               py::gil_scoped_release nogil;
               Grid<float, 4, true> og = o.g4();
               gi.forward(i.g4(), tr, og);
             }
             o.finish();
           })
      .def("forward",
           [](const GridInterpolater& gi, const py::object& in_center, const py::object& in, const Transform& tr,
              const py::object& out_center, const py::object& out) {
             Arg i(in, "in", 4, false), o(out, "out", 4, true);
             float3 ic = to_float3(in_center), oc = to_float3(out_center);
             {
               py::gil_scoped_release nogil;
               Grid<float, 4, true> og = o.g4();
               gi.forward(ic, i.g4(), tr, oc, og);
             }
             o.finish();
           })
      .def("backward",
           [](const GridInterpolater& gi, const py::object& grad_out, const Transform& tr, const py::object& grad_in) {
             Arg i(grad_out, "grad_out", 4, false), o(grad_in, "grad_in", 4, true);
             {
               py::gil_scoped_release nogil;
               Grid<float, 4, true> og = o.g4();
               gi.backward(i.g4(), tr, og);
             }
             o.finish();
           });

  bind_objects(m, gm_class, tr_class);
}
