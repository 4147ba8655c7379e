// GridMaker: atoms -> density grids and the matching backward passes (reference:
// include/libmolgrid/grid_maker.h, src/grid_maker.cpp, src/grid_maker.cu).  Same constructor,
// accessors and overload families for float grids; every overload ends in one call of the C ABI,
// which runs hand-written sm_100a kernels.  Host-grid (isCUDA = false) overloads stage their
// arguments through device memory: this library has no CPU implementation of the path.
// double grids are not supported on this path (the reference's CUDA vector backward is float-only too).
#ifndef LMGB200_GRID_MAKER_H_
#define LMGB200_GRID_MAKER_H_

#include <cmath>
#include <limits>
#include <vector>

#include "libmolgrid/coordinateset.h"
#include "libmolgrid/transform.h"

namespace libmolgrid {

class GridMaker {
 protected:
  lmg_gridmaker s_;  // resolution, dimension, scale factors, A..E, dim, binary, radii_type_indexed

 public:
  GridMaker(float res = 0, float d = 0, bool bin = false, bool rti = false, float rscale = 1.0, float grm = 1.0) {
    s_.radii_type_indexed = rti;
    initialize(res, d, bin, rscale, grm);
  }
  virtual ~GridMaker() {}

  void initialize(float res, float d, bool bin = false, float rscale = 1.0, float grm = 1.0) {
    int rti = s_.radii_type_indexed;
    detail::check(lmg_gridmaker_init(&s_, res, d, bin, rti, rscale, grm));
  }

  float3 get_grid_dims() const { return make_float3(s_.dim, s_.dim, s_.dim); }
  float get_resolution() const { return s_.resolution; }
  // as in the reference, the setters recompute the number of grid points and nothing else
  void set_resolution(float res) { s_.resolution = res; s_.dim = (unsigned)(std::round(s_.dimension / s_.resolution) + 1); }
  float get_dimension() const { return s_.dimension; }
  void set_dimension(float d) { s_.dimension = d; s_.dim = (unsigned)(std::round(s_.dimension / s_.resolution) + 1); }
  unsigned get_first_dim() const { return s_.dim; }
  bool get_binary() const { return s_.binary; }
  void set_binary(bool b) { s_.binary = b; }
  bool get_radii_type_indexed() const { return s_.radii_type_indexed; }
  void set_radii_type_indexed(bool b) { s_.radii_type_indexed = b; }
  float get_radiusmultiple() const { return s_.radius_scale * s_.final_radius_multiple; }
  float3 get_grid_origin(const float3& c) const {
    float half = s_.dimension / 2.0;
    return make_float3(c.x - half, c.y - half, c.z - half);
  }
  const lmg_gridmaker& settings() const { return s_; }

  // double grids: the signatures of the reference exist so that code written for them compiles, but
  // the path computes in fp32 only (the reference's own CUDA vector backward and second-order
  // kernels are float-only too, src/grid_maker.cu:645-649,805-809)
  template <size_t N, bool G>
  void forward(float3, const Grid<float, 2, G>&, const Grid<float, N, G>&, const Grid<float, 1, G>&,
               Grid<double, 4, G>&) const {
    throw std::invalid_argument("double grids are not supported on the GPU path: use float grids");
  }
  template <size_t N, bool G>
  void backward(float3, const Grid<float, 2, G>&, const Grid<float, N, G>&, const Grid<float, 1, G>&,
                const Grid<double, 4, G>&, Grid<double, 2, G>&) const {
    throw std::invalid_argument("double grids are not supported on the GPU path: use float grids");
  }
  template <bool G>
  void backward(float3, const Grid<float, 2, G>&, const Grid<float, 2, G>&, const Grid<float, 1, G>&,
                const Grid<double, 4, G>&, Grid<double, 2, G>&, Grid<double, 2, G>&) const {
    throw std::invalid_argument("double grids are not supported on the GPU path: use float grids");
  }

  // ------------------------------------------------------------------ forward, device grids
  void forward(float3 grid_center, const Grid<float, 2, true>& coords, const Grid<float, 1, true>& type_index,
               const Grid<float, 1, true>& radii, Grid<float, 4, true>& out, const Transform* transform = nullptr) const {
    check_out(out);
    size_t n = coords.dimension(0);
    if (type_index.size() != n) throw std::out_of_range("type_index does not match number of atoms: " + itoa(type_index.size()) + " vs " + itoa(n));
    if (radii.size() != n) throw std::out_of_range("radii does not match number of atoms: " + itoa(radii.size()) + " vs " + itoa(n));
    lmg_atoms a = single(grid_center, n, out.dimension(0), coords.data(), radii.data(), transform);
    a.type_index = type_index.data();
    run_forward(a, out.data(), 0);
  }

  void forward(float3 grid_center, const Grid<float, 2, true>& coords, const Grid<float, 2, true>& type_vector,
               const Grid<float, 1, true>& radii, Grid<float, 4, true>& out, const Transform* transform = nullptr) const {
    check_out(out);
    size_t n = coords.dimension(0), T = type_vector.dimension(1);
    if (type_vector.dimension(0) != n) throw std::out_of_range("type_vector does not match number of atoms: " + itoa(type_vector.dimension(0)) + " vs " + itoa(n));
    if (T != out.dimension(0)) throw std::out_of_range("number of types in type_vector does not match number of output channels: " + itoa(T) + " vs " + itoa(out.dimension(0)));
    check_vector_radii(radii.size(), n, T, true);
    lmg_atoms a = single(grid_center, n, T, coords.data(), radii.data(), transform);
    a.type_vector = type_vector.data();
    run_forward(a, out.data(), 1);
  }

  // batched raw arrays: one launch sequence for the whole batch (the reference loops on the host)
  // `transforms` (device, one lmg_transform per example, applied to the coordinates inside the
  // kernels) and `n_atoms` (device, valid atoms per example of a padded batch) are this library's
  // additions; both may be null.
  template <int N>
  void forward(const Grid<float, 2, true>& centers, const Grid<float, 3, true>& coords, const Grid<float, N, true>& types,
               const Grid<float, 2, true>& radii, Grid<float, 5, true>& out, const lmg_transform* transforms = nullptr,
               const int* n_atoms = nullptr) const {
    static_assert(N == 2 || N == 3, "Unsupported types dimension");
    size_t B = centers.dimension(0);
    batch_check(coords.dimension(0), B); batch_check(types.dimension(0), B);
    batch_check(radii.dimension(0), B); batch_check(out.dimension(0), B);
    for (int i = 2; i <= 4; i++)
      if (out.dimension(i) != s_.dim) throw std::out_of_range("Output grid dimension incorrect: " + itoa(s_.dim) + " vs " + itoa(out.dimension(i)));
    lmg_atoms a = {};
    a.batch = (int)B; a.max_atoms = (int)coords.dimension(1); a.ntypes = (int)out.dimension(1);
    a.coords = coords.data(); a.radii = radii.data(); a.centers = centers.data();
    a.transforms = transforms; a.n_atoms = n_atoms;
    if (N == 2) a.type_index = types.data(); else a.type_vector = types.data();
    if (N == 3) check_vector_radii(radii.dimension(1), coords.dimension(1), types.dimension(N - 1), true);
    run_forward(a, out.data(), N == 3);
  }

  // batched backward (an addition: the reference loops over the examples on the host):
  // atom_gradients[B][N][3], and type_gradients[B][N][T] with vector types (null: not wanted)
  template <int N>
  void backward(const Grid<float, 2, true>& centers, const Grid<float, 3, true>& coords, const Grid<float, N, true>& types,
                const Grid<float, 2, true>& radii, const Grid<float, 5, true>& diff, Grid<float, 3, true>& atom_gradients,
                float* type_gradients = nullptr, const lmg_transform* transforms = nullptr, const int* n_atoms = nullptr) const {
    static_assert(N == 2 || N == 3, "Unsupported types dimension");
    size_t B = centers.dimension(0), n = coords.dimension(1);
    batch_check(coords.dimension(0), B); batch_check(types.dimension(0), B); batch_check(radii.dimension(0), B);
    batch_check(diff.dimension(0), B); batch_check(atom_gradients.dimension(0), B);
    if (N == 2 && s_.radii_type_indexed) throw std::invalid_argument("Type indexed radii not supported with index types.");
    if (types.dimension(1) != n) throw std::invalid_argument("Type dimension doesn't equal number of coordinates.");
    if (atom_gradients.dimension(1) != n) throw std::invalid_argument("Gradient dimension doesn't equal number of coordinates");
    if (coords.dimension(2) != 3 || atom_gradients.dimension(2) != 3) throw std::invalid_argument("Need x,y,z,r for coord_radius");
    for (int i = 2; i <= 4; i++)
      if (diff.dimension(i) != s_.dim) throw std::invalid_argument("Incorrect grid dimension for diff");
    size_t T = diff.dimension(1);
    if (N == 3) {
      if (types.dimension(2) != T) throw std::invalid_argument("Channels in diff doesn't equal number of types");
      check_vector_radii(radii.dimension(1), n, T, false);
    } else {
      if (radii.dimension(1) != n) throw std::invalid_argument("Radii dimension doesn't equal number of coordinates");
      if (type_gradients != nullptr) throw std::invalid_argument("type_gradients given with index types");
    }
    lmg_atoms a = {};
    a.batch = (int)B; a.max_atoms = (int)n; a.ntypes = (int)T;
    a.coords = coords.data(); a.radii = radii.data(); a.centers = centers.data();
    a.transforms = transforms; a.n_atoms = n_atoms;
    if (N == 2) a.type_index = types.data(); else a.type_vector = types.data();
    size_t bytes = lmg_workspace_bytes(&s_, LMG_OP_BACKWARD, (int)B, (int)n, (int)T, N == 3);
    detail::check(lmg_backward(&s_, &a, diff.data(), atom_gradients.data(), type_gradients, detail::workspace(bytes), bytes, nullptr));
  }

  void forward(float3 grid_center, const CoordinateSet& in, Grid<float, 4, true>& out, const Transform* transform = nullptr) const {
    // vector types win when the set has both (include/libmolgrid/grid_maker.h:132-153 of the reference)
    if (in.has_vector_types() && in.size() > 0) forward(grid_center, in.coords.gpu(), in.type_vector.gpu(), in.radii.gpu(), out, transform);
    else forward(grid_center, in.coords.gpu(), in.type_index.gpu(), in.radii.gpu(), out, transform);
  }

  // The Transform is applied inside the gridding kernels; the grid stays centred on the
  // transform's rotation centre (src/grid_maker.cpp:109-116).
  void forward(const Example& in, const Transform& transform, Grid<float, 4, true>& out) const {
    CoordinateSet c = in.merge_coordinates();
    if (c.max_type != out.dimension(0))
      throw std::out_of_range("Incorrect number of channels in output grid: " + itoa(c.max_type) + " vs " + itoa(out.dimension(0)));
    forward(transform.get_rotation_center(), c, out, &transform);
  }

  // default centre: centre of the last coordinate set, when any later set is non-empty
  // (the reference's loop, src/grid_maker.cpp:125-136, looks at sets.back() whichever set is non-empty)
  void forward(const Example& in, Grid<float, 4, true>& out, float random_translation = 0.0, bool random_rotation = false,
               const float3& center = make_float3(std::numeric_limits<float>::infinity(), std::numeric_limits<float>::infinity(), std::numeric_limits<float>::infinity())) const {
    Transform t(default_center(in, center), random_translation, random_rotation);
    forward(in, t, out);
  }

  // whole batch of examples in one pass: merged atoms are padded to the longest example on the
  // host, copied once, and gridded with one Transform per example
  void forward(const std::vector<Example>& in, Grid<float, 5, true>& out, float random_translation = 0.0,
               bool random_rotation = false) const {
    if (in.size() != out.dimension(0)) throw std::out_of_range("output grid dimension does not match size of example vector");
    size_t B = in.size(), T = out.dimension(1), nmax = 0;
    std::vector<CoordinateSet> merged(B);
    for (size_t b = 0; b < B; b++) {
      merged[b] = in[b].merge_coordinates();
      if (merged[b].max_type != T)
        throw std::out_of_range("Incorrect number of channels in output grid: " + itoa(merged[b].max_type) + " vs " + itoa(T));
      nmax = std::max<size_t>(nmax, merged[b].size());
    }
    if (nmax == 0) nmax = 1;
    std::vector<float> hc(B * nmax * 3, 0.f), ht(B * nmax, -1.f), hr(B * nmax, 0.f), hcen(B * 3);
    std::vector<lmg_transform> htr(B);
    std::vector<int> hn(B);
    const float3 inf3 = make_float3(std::numeric_limits<float>::infinity(), 0, 0);
    for (size_t b = 0; b < B; b++) {
      Transform t(default_center(in[b], inf3), random_translation, random_rotation);
      htr[b] = t.c_struct();
      float3 c = t.get_rotation_center();
      hcen[3 * b] = c.x; hcen[3 * b + 1] = c.y; hcen[3 * b + 2] = c.z;
      unsigned n = merged[b].size();
      hn[b] = (int)n;
      if (n) {
        Grid2f cc = merged[b].coords.cpu();
        Grid1f tt = merged[b].type_index.cpu(), rr = merged[b].radii.cpu();
        std::memcpy(&hc[b * nmax * 3], cc.data(), n * 3 * sizeof(float));
        std::memcpy(&ht[b * nmax], tt.data(), n * sizeof(float));
        std::memcpy(&hr[b * nmax], rr.data(), n * sizeof(float));
      }
    }
    detail::Staged<float> dc(hc.data(), hc.size(), true, false), dt(ht.data(), ht.size(), true, false),
        dr(hr.data(), hr.size(), true, false), dcen(hcen.data(), hcen.size(), true, false);
    detail::Staged<lmg_transform> dtr(htr.data(), B, true, false);
    detail::Staged<int> dn(hn.data(), B, true, false);
    lmg_atoms a = {};
    a.batch = (int)B; a.max_atoms = (int)nmax; a.ntypes = (int)T;
    a.coords = dc.get(); a.type_index = dt.get(); a.radii = dr.get(); a.centers = dcen.get();
    a.transforms = dtr.get(); a.n_atoms = dn.get();
    for (int i = 2; i <= 4; i++)
      if (out.dimension(i) != s_.dim) throw std::out_of_range("Output grid dimension incorrect: " + itoa(s_.dim) + " vs " + itoa(out.dimension(i)));
    run_forward(a, out.data(), 0);
    LMG_CUDA_CHECK(cudaStreamSynchronize(nullptr));  // staged inputs are released on return
  }

  // ------------------------------------------------------------------ forward, host grids
  void forward(float3 grid_center, const Grid<float, 2, false>& coords, const Grid<float, 1, false>& type_index,
               const Grid<float, 1, false>& radii, Grid<float, 4, false>& out) const {
    detail::Staged<float> c(coords.data(), coords.size(), true, false), t(type_index.data(), type_index.size(), true, false),
        r(radii.data(), radii.size(), true, false), o(out.data(), out.size(), false, true);
    Grid4fCUDA og(o.get(), out.dimension(0), out.dimension(1), out.dimension(2), out.dimension(3));
    forward(grid_center, Grid2fCUDA(c.get(), coords.dimension(0), coords.dimension(1)), Grid1fCUDA(t.get(), type_index.size()),
            Grid1fCUDA(r.get(), radii.size()), og);
    o.finish();
  }
  void forward(float3 grid_center, const Grid<float, 2, false>& coords, const Grid<float, 2, false>& type_vector,
               const Grid<float, 1, false>& radii, Grid<float, 4, false>& out) const {
    detail::Staged<float> c(coords.data(), coords.size(), true, false), t(type_vector.data(), type_vector.size(), true, false),
        r(radii.data(), radii.size(), true, false), o(out.data(), out.size(), false, true);
    Grid4fCUDA og(o.get(), out.dimension(0), out.dimension(1), out.dimension(2), out.dimension(3));
    forward(grid_center, Grid2fCUDA(c.get(), coords.dimension(0), coords.dimension(1)),
            Grid2fCUDA(t.get(), type_vector.dimension(0), type_vector.dimension(1)), Grid1fCUDA(r.get(), radii.size()), og);
    o.finish();
  }

  // ------------------------------------------------------------------ backward
  void backward(float3 grid_center, const Grid<float, 2, true>& coords, const Grid<float, 1, true>& type_index,
                const Grid<float, 1, true>& radii, const Grid<float, 4, true>& diff, Grid<float, 2, true>& atom_gradients,
                const Transform* transform = nullptr) const {
    size_t n = coords.dimension(0);
    if (s_.radii_type_indexed) throw std::invalid_argument("Type indexed radii not supported with index types.");
    if (n != type_index.size()) throw std::invalid_argument("Type dimension doesn't equal number of coordinates.");
    if (n != atom_gradients.dimension(0)) throw std::invalid_argument("Gradient dimension doesn't equal number of coordinates");
    if (n != radii.size()) throw std::invalid_argument("Radii dimension doesn't equal number of coordinates");
    if (coords.dimension(1) != 3) throw std::invalid_argument("Need x,y,z,r for coord_radius");
    check_diff(diff);
    lmg_atoms a = single(grid_center, n, diff.dimension(0), coords.data(), radii.data(), transform);
    a.type_index = type_index.data();
    size_t bytes = lmg_workspace_bytes(&s_, LMG_OP_BACKWARD, 1, (int)n, a.ntypes, 0);
    detail::check(lmg_backward(&s_, &a, diff.data(), atom_gradients.data(), nullptr, detail::workspace(bytes), bytes, nullptr));
  }

  void backward(float3 grid_center, const Grid<float, 2, true>& coords, const Grid<float, 2, true>& type_vector,
                const Grid<float, 1, true>& radii, const Grid<float, 4, true>& diff, Grid<float, 2, true>& atom_gradients,
                Grid<float, 2, true>& type_gradients, const Transform* transform = nullptr) const {
    size_t n = coords.dimension(0), T = type_vector.dimension(1);
    if (n != type_vector.dimension(0)) throw std::invalid_argument("Type dimension doesn't equal number of coordinates.");
    if (T != diff.dimension(0)) throw std::invalid_argument("Channels in diff doesn't equal number of types");
    if (n != atom_gradients.dimension(0)) throw std::invalid_argument("Atom gradient dimension doesn't equal number of coordinates");
    if (n != type_gradients.dimension(0)) throw std::invalid_argument("Type gradient dimension doesn't equal number of coordinates");
    if (type_gradients.dimension(1) != T) throw std::invalid_argument("Type gradient dimension has wrong number of types");
    if (coords.dimension(1) != 3) throw std::invalid_argument("Need x,y,z,r for coord_radius");
    check_vector_radii(radii.size(), n, T, false);
    check_diff(diff);
    lmg_atoms a = single(grid_center, n, T, coords.data(), radii.data(), transform);
    a.type_vector = type_vector.data();
    size_t bytes = lmg_workspace_bytes(&s_, LMG_OP_BACKWARD, 1, (int)n, (int)T, 1);
    detail::check(lmg_backward(&s_, &a, diff.data(), atom_gradients.data(), type_gradients.data(), detail::workspace(bytes), bytes, nullptr));
  }

  void backward(float3 grid_center, const CoordinateSet& in, const Grid<float, 4, true>& diff, Grid<float, 2, true>& atomic_gradients) const {
    if (!in.has_indexed_types()) throw std::invalid_argument("Index types missing from coordinate set");
    backward(grid_center, in.coords.gpu(), in.type_index.gpu(), in.radii.gpu(), diff, atomic_gradients);
  }
  void backward(float3 grid_center, const CoordinateSet& in, const Grid<float, 4, true>& diff, Grid<float, 2, true>& atomic_gradients,
                Grid<float, 2, true>& type_gradients) const {
    if (!in.has_vector_types()) throw std::invalid_argument("Vector types missing from coordinate set");
    backward(grid_center, in.coords.gpu(), in.type_vector.gpu(), in.radii.gpu(), diff, atomic_gradients, type_gradients);
  }

  // second-order pass, vector types only; not const in the reference either
  void backward_gradients(float3 grid_center, const Grid<float, 2, true>& coords, const Grid<float, 2, true>& type_vector,
                          const Grid<float, 1, true>& radii, const Grid<float, 4, true>& diff,
                          const Grid<float, 2, true>& atom_gradients, const Grid<float, 2, true>& type_gradients,
                          Grid<float, 4, true>& diffdiff, Grid<float, 2, true>& atom_diffdiff, Grid<float, 2, true>& type_diffdiff) {
    size_t n = coords.dimension(0), T = type_vector.dimension(1);
    check_out(diff);
    if (type_vector.dimension(0) != n) throw std::out_of_range("type_vector does not match number of atoms: " + itoa(type_vector.dimension(0)) + " vs " + itoa(n));
    if (T != diff.dimension(0)) throw std::out_of_range("number of types in type_vector does not match number of output channels: " + itoa(T) + " vs " + itoa(diff.dimension(0)));
    check_vector_radii(radii.size(), n, T, true);
    if (n != atom_gradients.dimension(0)) throw std::invalid_argument("Atom gradient dimension doesn't equal number of coordinates");
    if (n != type_gradients.dimension(0)) throw std::invalid_argument("Type gradient dimension doesn't equal number of coordinates");
    if (n != atom_diffdiff.dimension(0)) throw std::invalid_argument("Atom gradient gradients dimension doesn't equal number of coordinates");
    if (n != type_diffdiff.dimension(0)) throw std::invalid_argument("Type gradient gradients dimension doesn't equal number of coordinates");
    if (type_gradients.dimension(1) != T || type_diffdiff.dimension(1) != T) throw std::invalid_argument("Type gradient dimension has wrong number of types");
    if (s_.binary) throw std::invalid_argument("Binary densities not supported");
    lmg_atoms a = single(grid_center, n, T, coords.data(), radii.data(), nullptr);
    a.type_vector = type_vector.data();
    size_t bytes = lmg_workspace_bytes(&s_, LMG_OP_BACKWARD_GRADIENTS, 1, (int)n, (int)T, 1);
    detail::check(lmg_backward_gradients(&s_, &a, diff.data(), atom_gradients.data(), type_gradients.data(), diffdiff.data(),
                                         atom_diffdiff.data(), type_diffdiff.data(), detail::workspace(bytes), bytes, nullptr));
  }

  void backward_relevance(float3 grid_center, const Grid<float, 2, true>& coords, const Grid<float, 1, true>& type_index,
                          const Grid<float, 1, true>& radii, const Grid<float, 4, true>& density, const Grid<float, 4, true>& diff,
                          Grid<float, 1, true>& relevance) const {
    size_t n = coords.dimension(0);
    if (n != type_index.size()) throw std::invalid_argument("Type dimension doesn't equal number of coordinates.");
    if (n != relevance.size()) throw std::invalid_argument("Relevance dimension doesn't equal number of coordinates");
    if (n != radii.size()) throw std::invalid_argument("Radii dimension doesn't equal number of coordinates");
    if (coords.dimension(1) != 3) throw std::invalid_argument("Coordinates and radius wrong secondary dimension");
    lmg_atoms a = single(grid_center, n, diff.dimension(0), coords.data(), radii.data(), nullptr);
    a.type_index = type_index.data();
    size_t bytes = lmg_workspace_bytes(&s_, LMG_OP_BACKWARD_RELEVANCE, 1, (int)n, a.ntypes, 0);
    detail::check(lmg_backward_relevance(&s_, &a, density.data(), diff.data(), relevance.data(), detail::workspace(bytes), bytes, nullptr));
  }

  // ------------------------------------------------------------------ host grids and coordinate sets
  // The reference's host-grid overloads (include/libmolgrid/grid_maker.h:392-445,463-485,598-612)
  // run its CPU code; here the arrays are staged through device memory and the GPU path computes.
  void backward(float3 grid_center, const Grid<float, 2, false>& coords, const Grid<float, 1, false>& type_index,
                const Grid<float, 1, false>& radii, const Grid<float, 4, false>& diff, Grid<float, 2, false>& atom_gradients) const {
    detail::Staged<float> c(coords.data(), coords.size(), true, false), t(type_index.data(), type_index.size(), true, false),
        r(radii.data(), radii.size(), true, false), d(diff.data(), diff.size(), true, false),
        g(atom_gradients.data(), atom_gradients.size(), false, true);
    Grid2fCUDA gg(g.get(), atom_gradients.dimension(0), atom_gradients.dimension(1));
    backward(grid_center, Grid2fCUDA(c.get(), coords.dimension(0), coords.dimension(1)), Grid1fCUDA(t.get(), type_index.size()),
             Grid1fCUDA(r.get(), radii.size()), dev4(d, diff), gg);
    g.finish();
  }
  void backward(float3 grid_center, const Grid<float, 2, false>& coords, const Grid<float, 2, false>& type_vector,
                const Grid<float, 1, false>& radii, const Grid<float, 4, false>& diff, Grid<float, 2, false>& atom_gradients,
                Grid<float, 2, false>& type_gradients) const {
    detail::Staged<float> c(coords.data(), coords.size(), true, false), t(type_vector.data(), type_vector.size(), true, false),
        r(radii.data(), radii.size(), true, false), d(diff.data(), diff.size(), true, false),
        g(atom_gradients.data(), atom_gradients.size(), false, true), tg(type_gradients.data(), type_gradients.size(), false, true);
    Grid2fCUDA gg(g.get(), atom_gradients.dimension(0), atom_gradients.dimension(1));
    Grid2fCUDA tgg(tg.get(), type_gradients.dimension(0), type_gradients.dimension(1));
    backward(grid_center, Grid2fCUDA(c.get(), coords.dimension(0), coords.dimension(1)),
             Grid2fCUDA(t.get(), type_vector.dimension(0), type_vector.dimension(1)), Grid1fCUDA(r.get(), radii.size()),
             dev4(d, diff), gg, tgg);
    g.finish();
    tg.finish();
  }
  void backward_gradients(float3 grid_center, const Grid<float, 2, false>& coords, const Grid<float, 2, false>& type_vector,
                          const Grid<float, 1, false>& radii, const Grid<float, 4, false>& diff,
                          const Grid<float, 2, false>& atom_gradients, const Grid<float, 2, false>& type_gradients,
                          Grid<float, 4, false>& diffdiff, Grid<float, 2, false>& atom_diffdiff, Grid<float, 2, false>& type_diffdiff) {
    detail::Staged<float> c(coords.data(), coords.size(), true, false), t(type_vector.data(), type_vector.size(), true, false),
        r(radii.data(), radii.size(), true, false), d(diff.data(), diff.size(), true, false),
        ag(atom_gradients.data(), atom_gradients.size(), true, false), tg(type_gradients.data(), type_gradients.size(), true, false),
        dd(diffdiff.data(), diffdiff.size(), false, true), add(atom_diffdiff.data(), atom_diffdiff.size(), false, true),
        tdd(type_diffdiff.data(), type_diffdiff.size(), false, true);
    Grid4fCUDA ddg = dev4(dd, diffdiff);
    Grid2fCUDA addg(add.get(), atom_diffdiff.dimension(0), atom_diffdiff.dimension(1));
    Grid2fCUDA tddg(tdd.get(), type_diffdiff.dimension(0), type_diffdiff.dimension(1));
    backward_gradients(grid_center, Grid2fCUDA(c.get(), coords.dimension(0), coords.dimension(1)),
                       Grid2fCUDA(t.get(), type_vector.dimension(0), type_vector.dimension(1)), Grid1fCUDA(r.get(), radii.size()),
                       dev4(d, diff), Grid2fCUDA(ag.get(), atom_gradients.dimension(0), atom_gradients.dimension(1)),
                       Grid2fCUDA(tg.get(), type_gradients.dimension(0), type_gradients.dimension(1)), ddg, addg, tddg);
    dd.finish();
    add.finish();
    tdd.finish();
  }
  void backward_relevance(float3 grid_center, const Grid<float, 2, false>& coords, const Grid<float, 1, false>& type_index,
                          const Grid<float, 1, false>& radii, const Grid<float, 4, false>& density,
                          const Grid<float, 4, false>& diff, Grid<float, 1, false>& relevance) const {
    detail::Staged<float> c(coords.data(), coords.size(), true, false), t(type_index.data(), type_index.size(), true, false),
        r(radii.data(), radii.size(), true, false), de(density.data(), density.size(), true, false),
        d(diff.data(), diff.size(), true, false), rel(relevance.data(), relevance.size(), false, true);
    Grid1fCUDA relg(rel.get(), relevance.size());
    backward_relevance(grid_center, Grid2fCUDA(c.get(), coords.dimension(0), coords.dimension(1)), Grid1fCUDA(t.get(), type_index.size()),
                       Grid1fCUDA(r.get(), radii.size()), dev4(de, density), dev4(d, diff), relg);
    rel.finish();
  }

  // Coordinate sets with host grids (include/libmolgrid/grid_maker.h:131-143,314-350): the set's own
  // arrays are used on whichever side the result lives
  void forward(float3 grid_center, const CoordinateSet& in, Grid<float, 4, false>& out) const {
    if (in.has_vector_types() && in.size() > 0) forward(grid_center, in.coords.cpu(), in.type_vector.cpu(), in.radii.cpu(), out);
    else if (in.has_indexed_types()) forward(grid_center, in.coords.cpu(), in.type_index.cpu(), in.radii.cpu(), out);
    else throw std::invalid_argument("Type information missing from coordinate set");
  }
  void backward(float3 grid_center, const CoordinateSet& in, const Grid<float, 4, false>& diff, Grid<float, 2, false>& atomic_gradients) const {
    if (!in.has_indexed_types()) throw std::invalid_argument("Index types missing from coordinate set");
    backward(grid_center, in.coords.cpu(), in.type_index.cpu(), in.radii.cpu(), diff, atomic_gradients);
  }
  void backward(float3 grid_center, const CoordinateSet& in, const Grid<float, 4, false>& diff, Grid<float, 2, false>& atomic_gradients,
                Grid<float, 2, false>& type_gradients) const {
    if (!in.has_vector_types()) throw std::invalid_argument("Vector types missing from coordinate set");
    backward(grid_center, in.coords.cpu(), in.type_vector.cpu(), in.radii.cpu(), diff, atomic_gradients, type_gradients);
  }
  // include/libmolgrid/grid_maker.h:508-547
  template <bool G>
  void backward_gradients(float3 grid_center, const CoordinateSet& in, const Grid<float, 4, G>& diff,
                          const Grid<float, 2, G>& atom_gradients, const Grid<float, 2, G>& type_gradients,
                          Grid<float, 4, G>& diffdiff, Grid<float, 2, G>& atom_diffdiff, Grid<float, 2, G>& type_diffdiff) {
    if (!in.has_vector_types()) throw std::invalid_argument("Vector types missing from coordinate set");
    backward_gradients(grid_center, side<G>(in.coords), side<G>(in.type_vector), side<G>(in.radii), diff, atom_gradients,
                       type_gradients, diffdiff, atom_diffdiff, type_diffdiff);
  }
  // include/libmolgrid/grid_maker.h:558-596
  template <bool G>
  void backward_relevance(float3 grid_center, const CoordinateSet& in, const Grid<float, 4, G>& density,
                          const Grid<float, 4, G>& diff, Grid<float, 1, G>& relevance) const {
    if (!in.has_indexed_types()) throw std::invalid_argument("Index types missing from coordinate set");
    backward_relevance(grid_center, side<G>(in.coords), side<G>(in.type_index), side<G>(in.radii), density, diff, relevance);
  }

  // Synchronises and throws std::out_of_range / std::invalid_argument if the last call on this
  // thread met a type index >= the number of channels (the reference checks this while looping
  // over atoms on the host, src/grid_maker.cpp:172,458-460).
  void check_types() const {
    detail::check(lmg_check_status(detail::workspace(256), nullptr));
  }

 private:
  static Grid4fCUDA dev4(const detail::Staged<float>& st, const Grid<float, 4, false>& g) {
    return Grid4fCUDA(st.get(), g.dimension(0), g.dimension(1), g.dimension(2), g.dimension(3));
  }
  // the view of a managed grid on the side (device or host) that G names
  template <bool G, size_t N>
  static Grid<float, N, G> side(const ManagedGrid<float, N>& m) {
    return m;  // ManagedGrid converts to either view, migrating its block
  }
  static void batch_check(size_t got, size_t B) {
    if (got != B) throw std::invalid_argument("Mismatched batch sizes: " + itoa(got) + " vs " + itoa(B));
  }
  template <bool G>
  void check_out(const Grid<float, 4, G>& out) const {
    for (int i = 1; i <= 3; i++)
      if (out.dimension(i) != s_.dim) throw std::out_of_range("Output grid dimension incorrect: " + itoa(s_.dim) + " vs " + itoa(out.dimension(i)));
  }
  void check_diff(const Grid<float, 4, true>& diff) const {
    for (unsigned i = 1; i <= 3; i++)
      if (diff.dimension(i) != s_.dim)
        throw std::invalid_argument("diff does not have correct dimension " + itoa(i) + ": " + itoa(diff.dimension(i)) + " vs " + itoa(s_.dim));
  }
  void check_vector_radii(size_t nr, size_t n, size_t T, bool forward_pass) const {
    bool bad = s_.radii_type_indexed ? nr != T : nr != n;
    if (!bad) return;
    std::string msg = s_.radii_type_indexed ? "radii does not match number of types: " + itoa(nr) + " vs " + itoa(T)
                                            : "radii does not match number of atoms: " + itoa(nr) + " vs " + itoa(n);
    if (forward_pass) throw std::out_of_range(msg);
    throw std::invalid_argument(msg);
  }
  static float3 default_center(const Example& in, const float3& center) {
    float3 c = center;
    if (std::isinf(c.x)) {
      c = make_float3(0, 0, 0);
      for (int i = (int)in.sets.size() - 1; i >= 0; i--) {
        if (in.sets[i].size()) { c = in.sets.back().center(); break; }
      }
    }
    return c;
  }
  lmg_atoms single(float3 center, size_t n, size_t T, const float* coords, const float* radii, const Transform* tr) const {
    lmg_atoms a = {};
    a.batch = 1; a.max_atoms = (int)n; a.ntypes = (int)T;
    a.coords = coords; a.radii = radii;
    a.center_host[0] = center.x; a.center_host[1] = center.y; a.center_host[2] = center.z;
    if (tr) { tr_ = tr->c_struct(); a.transform_host = &tr_; }
    return a;
  }
  void run_forward(const lmg_atoms& a, float* out, int vec) const {
    size_t bytes = lmg_workspace_bytes(&s_, LMG_OP_FORWARD, a.batch, a.max_atoms, a.ntypes, vec);
    detail::check(lmg_forward(&s_, &a, out, detail::workspace(bytes), bytes, nullptr));
  }
  mutable lmg_transform tr_;  // keeps the by-value transform alive for the duration of a call
};

}  // namespace libmolgrid
#endif
