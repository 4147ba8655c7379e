// GridInterpolater: trilinear resample of a grid under a Transform (reference:
// include/libmolgrid/grid_interpolater.h, src/grid_interpolater.{cpp,cu}).
#ifndef LMGB200_GRID_INTERPOLATER_H_
#define LMGB200_GRID_INTERPOLATER_H_

#include <cmath>

#include "libmolgrid/transform.h"

namespace libmolgrid {

class GridInterpolater {
  lmg_interpolater s_;

 public:
  GridInterpolater(float inres, float indim, float outres, float outdim) {
    detail::check(lmg_interpolater_init(&s_, inres, indim, outres, outdim));
  }
  virtual ~GridInterpolater() {}

  float get_in_resolution() const { return s_.in_resolution; }
  float get_out_resolution() const { return s_.out_resolution; }
  float get_in_dimension() const { return s_.in_dimension; }
  float get_out_dimension() const { return s_.out_dimension; }
  // The reference's input setters recompute the point count from the values held BEFORE the
  // assignment, and its output setters never recompute it; existing code relies on constructing a
  // new object instead, so the behaviour is kept.
  void set_in_resolution(float res) { s_.in_dim = (unsigned)(std::round(s_.in_dimension / s_.in_resolution) + 1); s_.in_resolution = res; }
  void set_in_dimension(float d) { s_.in_dim = (unsigned)(std::round(s_.in_dimension / s_.in_resolution) + 1); s_.in_dimension = d; }
  void set_out_resolution(float res) { s_.out_resolution = res; }
  void set_out_dimension(float d) { s_.out_dimension = d; }

  void forward(float3 in_center, const Grid<float, 4, true>& in, const Transform& transform, float3 out_center,
               Grid<float, 4, true>& out) const {
    check_grids(in, out);
    lmg_transform t = transform.c_struct();
    float ic[3] = {in_center.x, in_center.y, in_center.z}, oc[3] = {out_center.x, out_center.y, out_center.z};
    detail::check(lmg_interpolate(&s_, 1, (int)in.dimension(0), in.data(), &t, ic, oc, out.data(), nullptr));
  }
  void forward(const Grid<float, 4, true>& in, const Transform& transform, Grid<float, 4, true>& out) const {
    float3 c = transform.get_rotation_center();
    forward(c, in, transform, c, out);
  }
  void forward(const Grid<float, 4, true>& in, Grid<float, 4, true>& out, float random_translation = 0, bool random_rotation = false) const {
    Transform t(make_float3(0, 0, 0), random_translation, random_rotation);
    forward(in, t, out);
  }
  // host grids are staged through the device
  void forward(float3 in_center, const Grid<float, 4, false>& in, const Transform& transform, float3 out_center,
               Grid<float, 4, false>& out) const {
    if (in.data() == out.data()) throw std::invalid_argument("Input and output grid can not be the same in GridInterpolator.");
    detail::Staged<float> i(in.data(), in.size(), true, false), o(out.data(), out.size(), false, true);
    Grid4fCUDA ig(i.get(), in.dimension(0), in.dimension(1), in.dimension(2), in.dimension(3));
    Grid4fCUDA og(o.get(), out.dimension(0), out.dimension(1), out.dimension(2), out.dimension(3));
    forward(in_center, ig, transform, out_center, og);
    o.finish();
  }
  void forward(const Grid<float, 4, false>& in, const Transform& transform, Grid<float, 4, false>& out) const {
    float3 c = transform.get_rotation_center();
    forward(c, in, transform, c, out);
  }
  void forward(const Grid<float, 4, false>& in, Grid<float, 4, false>& out, float random_translation = 0, bool random_rotation = false) const {
    Transform t(make_float3(0, 0, 0), random_translation, random_rotation);
    forward(in, t, out);
  }

  // Gradient with respect to forward's input from the gradient with respect to its output, for the
  // same transform and centres (the reference leaves the backward pass open).
  void backward(float3 in_center, const Grid<float, 4, true>& grad_out, const Transform& transform,
                float3 out_center, Grid<float, 4, true>& grad_in) const {
    check_grids(grad_in, grad_out);
    lmg_transform t = transform.c_struct();
    float ic[3] = {in_center.x, in_center.y, in_center.z}, oc[3] = {out_center.x, out_center.y, out_center.z};
    detail::check(lmg_interpolate_backward(&s_, 1, (int)grad_out.dimension(0), grad_out.data(), &t, ic, oc,
                                           grad_in.data(), nullptr));
  }
  void backward(const Grid<float, 4, true>& grad_out, const Transform& transform, Grid<float, 4, true>& grad_in) const {
    float3 c = transform.get_rotation_center();
    backward(c, grad_out, transform, c, grad_in);
  }

 private:
  void check_grids(const Grid<float, 4, true>& in, const Grid<float, 4, true>& out) const {
    if (in.data() == out.data()) throw std::invalid_argument("Input and output grid can not be the same in GridInterpolator.");
    if (in.dimension(0) != out.dimension(0)) throw std::invalid_argument("Different channel dimensions for input and output  grids.");
    for (int i = 1; i <= 3; i++) {
      if (in.dimension(i) != s_.in_dim) throw std::invalid_argument("Input grid wrong dimension. Should be " + itoa(s_.in_dim) + " along all axes");
      if (out.dimension(i) != s_.out_dim) throw std::invalid_argument("Output grid wrong dimension. Should be " + itoa(s_.out_dim) + " along all axes");
    }
    if (in.data() == nullptr) throw std::invalid_argument("Input grid not allocated");
    if (out.data() == nullptr) throw std::invalid_argument("Output grid not allocated");
  }
};

}  // namespace libmolgrid
#endif
