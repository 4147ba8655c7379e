/* TEST INFRASTRUCTURE ONLY - never linked into or called from the product library.
 *
 * C entry points over the UNMODIFIED reference CPU implementation (libmolgrid's
 * src/grid_maker.cpp + the host bodies in src/grid_maker.cu, src/transform.cpp,
 * src/grid_interpolater.{cpp,cu}), compiled from the reference tree by
 * oracle/Makefile into oracle/_ref/liblmg_ref.so.  The harness only wraps raw
 * pointers in the reference's non-owning Grid views and calls the CPU
 * (isCUDA=false) overloads; no arithmetic of the path lives here.
 *
 * Every function returns 0, or 1 (std::out_of_range), 2 (std::invalid_argument),
 * 3 (anything else); lmgref_last_error() gives the message.
 */
#include <cstring>
#include <iostream>
#include <stdexcept>
#include <string>

#include "libmolgrid/grid_interpolater.h"
#include "libmolgrid/grid_maker.h"
#include "libmolgrid/transform.h"

using namespace libmolgrid;

namespace {
thread_local std::string g_err;

// exposes the protected precomputed coefficients of the reference class
struct GridMakerPeek : public GridMaker {
  using GridMaker::GridMaker;
  void consts(float* out) const {
    out[0] = A; out[1] = B; out[2] = C; out[3] = D; out[4] = E;
    out[5] = final_radius_multiple; out[6] = (float)dim; out[7] = gaussian_radius_multiple;
  }
};

template <class F>
int guarded(F&& f) {
  try {
    f();
    return 0;
  } catch (const std::out_of_range& e) {
    g_err = e.what();
    return 1;
  } catch (const std::invalid_argument& e) {
    g_err = e.what();
    return 2;
  } catch (const std::exception& e) {
    g_err = e.what();
    return 3;
  }
}

struct GM {
  float res, dimension; int binary, rti; float rscale, grm;
};

GridMaker make(const float* p) {
  return GridMaker(p[0], p[1], p[2] != 0, p[3] != 0, p[4], p[5]);
}
}  // namespace

extern "C" {

const char* lmgref_last_error() { return g_err.c_str(); }

/* gm = {resolution, dimension, binary, radii_type_indexed, radius_scale, gaussian_radius_multiple} */
int lmgref_consts(const float* gm, float* out8) {
  return guarded([&] {
    GridMakerPeek g(gm[0], gm[1], gm[2] != 0, gm[3] != 0, gm[4], gm[5]);
    g.consts(out8);
  });
}

int lmgref_forward_index(const float* gm, const float* center, unsigned n, float* coords,
                         float* types, float* radii, unsigned ntypes, float* out) {
  return guarded([&] {
    GridMaker g = make(gm);
    unsigned d = g.get_first_dim();
    Grid2f C(coords, n, 3);
    Grid1f T(types, n);
    Grid1f R(radii, n);
    Grid4f O(out, ntypes, d, d, d);
    g.forward(float3{center[0], center[1], center[2]}, C, T, R, O);
  });
}

int lmgref_forward_vector(const float* gm, const float* center, unsigned n, unsigned ntypes,
                          float* coords, float* type_vector, float* radii, unsigned nradii,
                          float* out) {
  return guarded([&] {
    GridMaker g = make(gm);
    unsigned d = g.get_first_dim();
    Grid2f C(coords, n, 3);
    Grid2f T(type_vector, n, ntypes);
    Grid1f R(radii, nradii);
    Grid4f O(out, ntypes, d, d, d);
    g.forward(float3{center[0], center[1], center[2]}, C, T, R, O);
  });
}

int lmgref_backward_index(const float* gm, const float* center, unsigned n, float* coords,
                          float* types, float* radii, unsigned ntypes, float* diff,
                          float* atom_gradients) {
  return guarded([&] {
    GridMaker g = make(gm);
    unsigned d = g.get_first_dim();
    Grid2f C(coords, n, 3);
    Grid1f T(types, n);
    Grid1f R(radii, n);
    Grid4f D(diff, ntypes, d, d, d);
    Grid2f AG(atom_gradients, n, 3);
    g.backward(float3{center[0], center[1], center[2]}, C, T, R, D, AG);
  });
}

int lmgref_backward_vector(const float* gm, const float* center, unsigned n, unsigned ntypes,
                           float* coords, float* type_vector, float* radii, unsigned nradii,
                           float* diff, float* atom_gradients, float* type_gradients) {
  return guarded([&] {
    GridMaker g = make(gm);
    unsigned d = g.get_first_dim();
    Grid2f C(coords, n, 3);
    Grid2f T(type_vector, n, ntypes);
    Grid1f R(radii, nradii);
    Grid4f D(diff, ntypes, d, d, d);
    Grid2f AG(atom_gradients, n, 3);
    Grid2f TG(type_gradients, n, ntypes);
    g.backward(float3{center[0], center[1], center[2]}, C, T, R, D, AG, TG);
  });
}

int lmgref_backward_gradients(const float* gm, const float* center, unsigned n, unsigned ntypes,
                              float* coords, float* type_vector, float* radii, unsigned nradii,
                              float* diff, float* atom_gradients, float* type_gradients,
                              float* diffdiff, float* atom_diffdiff, float* type_diffdiff) {
  return guarded([&] {
    GridMaker g = make(gm);
    unsigned d = g.get_first_dim();
    Grid2f C(coords, n, 3);
    Grid2f T(type_vector, n, ntypes);
    Grid1f R(radii, nradii);
    Grid4f D(diff, ntypes, d, d, d);
    Grid2f AG(atom_gradients, n, 3);
    Grid2f TG(type_gradients, n, ntypes);
    Grid4f DD(diffdiff, ntypes, d, d, d);
    Grid2f ADD(atom_diffdiff, n, 3);
    Grid2f TDD(type_diffdiff, n, ntypes);
    // the reference CPU routine prints debugging text to std::cerr for every touched voxel
    std::ios_base::iostate old = std::cerr.rdstate();
    std::cerr.setstate(std::ios_base::failbit);
    try {
      g.backward_gradients(float3{center[0], center[1], center[2]}, C, T, R, D, AG, TG, DD, ADD, TDD);
    } catch (...) {
      std::cerr.clear(old);
      throw;
    }
    std::cerr.clear(old);
  });
}

int lmgref_backward_relevance(const float* gm, const float* center, unsigned n, float* coords,
                              float* types, float* radii, unsigned ntypes, float* density,
                              float* diff, float* relevance) {
  return guarded([&] {
    GridMaker g = make(gm);
    unsigned d = g.get_first_dim();
    Grid2f C(coords, n, 3);
    Grid1f T(types, n);
    Grid1f R(radii, n);
    Grid4f DE(density, ntypes, d, d, d);
    Grid4f D(diff, ntypes, d, d, d);
    Grid1f REL(relevance, n);
    g.backward_relevance(float3{center[0], center[1], center[2]}, C, T, R, DE, D, REL);
  });
}

/* tr = {qa,qb,qc,qd, cx,cy,cz, tx,ty,tz} */
static Transform make_tr(const float* tr) {
  return Transform(Quaternion(tr[0], tr[1], tr[2], tr[3]), float3{tr[4], tr[5], tr[6]},
                   float3{tr[7], tr[8], tr[9]});
}

int lmgref_transform_forward(const float* tr, unsigned n, float* in, float* out, int dotranslate) {
  return guarded([&] {
    Transform t = make_tr(tr);
    Grid2f I(in, n, 3);
    Grid2f O(out, n, 3);
    t.forward(I, O, dotranslate != 0);
  });
}

int lmgref_transform_backward(const float* tr, unsigned n, float* in, float* out, int dotranslate) {
  return guarded([&] {
    Transform t = make_tr(tr);
    Grid2f I(in, n, 3);
    Grid2f O(out, n, 3);
    t.backward(I, O, dotranslate != 0);
  });
}

/* Random Transform exactly as the reference draws it, after seeding the library's global engine. */
int lmgref_random_transform(unsigned seed, const float* center, float random_translate,
                            int random_rotate, unsigned ndraws, float* out10) {
  return guarded([&] {
    random_engine.seed(seed);
    for (unsigned i = 0; i < ndraws; i++) {
      Transform t(float3{center[0], center[1], center[2]}, random_translate, random_rotate != 0);
      const Quaternion& q = t.get_quaternion();
      float* o = out10 + 10 * i;
      o[0] = q.R_component_1(); o[1] = q.R_component_2();
      o[2] = q.R_component_3(); o[3] = q.R_component_4();
      float3 c = t.get_rotation_center(), tl = t.get_translation();
      o[4] = c.x; o[5] = c.y; o[6] = c.z;
      o[7] = tl.x; o[8] = tl.y; o[9] = tl.z;
    }
  });
}

/* Quaternion product, quotient, inverse and rotate exactly as the reference class computes them. */
int lmgref_quaternion_ops(const float* qa, const float* qb, const float* pt, float* out15) {
  return guarded([&] {
    Quaternion a(qa[0], qa[1], qa[2], qa[3]), b(qb[0], qb[1], qb[2], qb[3]);
    Quaternion p = a * b, d = a / b, inv = a.inverse();
    float3 r = a.rotate(pt[0], pt[1], pt[2]);
    const Quaternion* qs[3] = {&p, &d, &inv};
    for (int i = 0; i < 3; i++) {
      out15[4 * i + 0] = qs[i]->R_component_1(); out15[4 * i + 1] = qs[i]->R_component_2();
      out15[4 * i + 2] = qs[i]->R_component_3(); out15[4 * i + 3] = qs[i]->R_component_4();
    }
    out15[12] = r.x; out15[13] = r.y; out15[14] = r.z;
  });
}

/* gi = {in_resolution, in_dimension, out_resolution, out_dimension} */
int lmgref_interpolate(const float* gi, const float* in_center, unsigned nchannels, float* in,
                       const float* tr, const float* out_center, float* out) {
  return guarded([&] {
    GridInterpolater g(gi[0], gi[1], gi[2], gi[3]);
    unsigned din = (unsigned)(std::round(gi[1] / gi[0]) + 1);
    unsigned dout = (unsigned)(std::round(gi[3] / gi[2]) + 1);
    Grid4f I(in, nchannels, din, din, din);
    Grid4f O(out, nchannels, dout, dout, dout);
    Transform t = make_tr(tr);
    g.forward(float3{in_center[0], in_center[1], in_center[2]}, I, t,
              float3{out_center[0], out_center[1], out_center[2]}, O);
  });
}

}  // extern "C"
