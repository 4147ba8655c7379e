// Transform: rotation about a centre followed by a translation (reference:
// include/libmolgrid/transform.h, src/transform.cpp, src/transform.cu).  Coordinates are
// transformed on the GPU through the C ABI; host grids are staged through device memory.
#ifndef LMGB200_TRANSFORM_H_
#define LMGB200_TRANSFORM_H_

#include "libmolgrid/coordinateset.h"
#include "libmolgrid/quaternion.h"

namespace libmolgrid {

// reseeds the engine behind random Transforms (the reference's set_random_seed)
inline void set_random_seed(unsigned seed) { lmg_set_random_seed(seed); }

class Transform {
  Quaternion Q;
  float3 center;
  float3 translate;

 public:
  Transform() : center(make_float3(0, 0, 0)), translate(make_float3(0, 0, 0)) {}
  Transform(const Quaternion& q, float3 c = make_float3(0, 0, 0), float3 t = make_float3(0, 0, 0))
      : Q(q), center(c), translate(t) {}
  // random translation in [-random_translate, random_translate]^3 and, if asked, a uniform random
  // rotation; draws from the library's seeded engine in the reference's order
  Transform(float3 c, float random_translate = 0.0f, bool random_rotate = false) : center(c) {
    lmg_transform t;
    float cc[3] = {c.x, c.y, c.z};
    detail::check(lmg_transform_random(&t, cc, random_translate, random_rotate));
    Q = Quaternion(t.q[0], t.q[1], t.q[2], t.q[3]);
    translate = make_float3(t.translate[0], t.translate[1], t.translate[2]);
  }

  const Quaternion& get_quaternion() const { return Q; }
  float3 get_rotation_center() const { return center; }
  float3 get_translation() const { return translate; }
  void set_quaternion(const Quaternion& q) { Q = q; }
  void set_rotation_center(float3 c) { center = c; }
  void set_translation(float3 t) { translate = t; }
  bool is_identity() const { return Q == Quaternion() && translate.x == 0 && translate.y == 0 && translate.z == 0; }

  lmg_transform c_struct() const {
    lmg_transform t;
    t.q[0] = Q.R_component_1(); t.q[1] = Q.R_component_2(); t.q[2] = Q.R_component_3(); t.q[3] = Q.R_component_4();
    t.center[0] = center.x; t.center[1] = center.y; t.center[2] = center.z;
    t.translate[0] = translate.x; t.translate[1] = translate.y; t.translate[2] = translate.z;
    return t;
  }

  void forward(const Grid<float, 2, true>& in, Grid<float, 2, true>& out, bool dotranslate = true) const {
    check_grids(in, out);
    lmg_transform t = c_struct();
    detail::check(lmg_transform_forward(&t, (int)in.dimension(0), in.data(), out.data(), dotranslate, nullptr));
  }
  void backward(const Grid<float, 2, true>& in, Grid<float, 2, true>& out, bool dotranslate = true) const {
    check_grids(in, out);
    lmg_transform t = c_struct();
    detail::check(lmg_transform_backward(&t, (int)in.dimension(0), in.data(), out.data(), dotranslate, nullptr));
  }
  void forward(const Grid<float, 2, false>& in, Grid<float, 2, false>& out, bool dotranslate = true) const {
    host_apply(in, out, dotranslate, true);
  }
  void backward(const Grid<float, 2, false>& in, Grid<float, 2, false>& out, bool dotranslate = true) const {
    host_apply(in, out, dotranslate, false);
  }
  void forward(const CoordinateSet& in, CoordinateSet& out, bool dotranslate = true) const {
    if (in.coords.dimension(0) != out.coords.dimension(0)) throw std::invalid_argument("Incompatible coordinateset sizes");
    Grid2fCUDA i = in.coords.gpu(), o = out.coords.gpu();
    if (in.coords.dimension(0)) forward(i, o, dotranslate);
  }
  void forward(const Example& in, Example& out, bool dotranslate = true) const {
    if (in.sets.size() != out.sets.size()) throw std::invalid_argument("Incompatible example sizes");
    for (size_t i = 0; i < in.sets.size(); i++) forward(in.sets[i], out.sets[i], dotranslate);
  }

 private:
  template <bool G>
  static void check_grids(const Grid<float, 2, G>& in, const Grid<float, 2, G>& out) {
    if (in.dimension(0) != out.dimension(0))
      throw std::invalid_argument("Different dimensions and input and output coordinates grids.");
    if (in.dimension(1) != 3) throw std::invalid_argument("Input coordinates wrong dimension.");
    if (out.dimension(1) != 3) throw std::invalid_argument("Output coordinates are wrong dimension.");
    if (in.data() == nullptr) throw std::invalid_argument("Input coordinates missing memory");
    if (out.data() == nullptr) throw std::invalid_argument("Output coordinates missing memory");
  }
  void host_apply(const Grid<float, 2, false>& in, Grid<float, 2, false>& out, bool dotranslate, bool fwd) const {
    check_grids(in, out);
    size_t n = in.size();
    detail::Staged<float> d(out.data(), n, false, true);
    LMG_CUDA_CHECK(cudaMemcpy(d.get(), in.data(), n * sizeof(float), cudaMemcpyHostToDevice));
    Grid2fCUDA g(d.get(), in.dimension(0), 3);
    if (fwd) forward(g, g, dotranslate);
    else backward(g, g, dotranslate);
    d.finish();
  }
};

}  // namespace libmolgrid
#endif
