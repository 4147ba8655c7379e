// Shared device-side definitions of the sm_100a gridding kernels.
//
// Exactness rules used throughout (they make binary grids, footprints and channel assignment
// bit-identical to libmolgrid's CPU path, which is built without fused multiply-add):
//   * every product/sum whose result feeds a comparison is written with __fmul_rn/__fadd_rn/
//     __fsub_rn/__fdiv_rn, which nvcc never contracts into an FMA;
//   * voxel coordinate  = origin + float(i) * resolution          (src/grid_maker.cpp:191-193)
//   * squared distance  = ((gx-ax)^2 + (gy-ay)^2) + (gz-az)^2     (src/grid_maker.cu:82-92)
//   * "dist > cut" on dist = sqrtf(rsq) is evaluated as rsq > T with T the largest float whose
//     correctly rounded square root is <= cut (sqrt is monotone, so the two tests agree exactly);
//   * the per-atom integer footprint [lo,hi) of get_bounds_1d (src/grid_maker.cu:66-79) is
//     honoured in addition to the radial test.
#pragma once
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

namespace lmg {

struct GMParams {
  float res, half, rscale, G, finalm;
  float A, B, C, D, E;
  // The tail polynomial A dr^2 + B dr + C has a double root at dr = final_radius_multiple, so it
  // equals (ta*dr - tb)^2 with ta = 2G e^{-G^2}, tb = (1+2G^2) e^{-G^2}; min(ta*dr - tb, 0)^2 is
  // then also zero beyond the cut-off.  Both are 0 for a truncated Gaussian (no tail).
  float ta, tb;
  unsigned dim;
  int binary, rti;
};

struct Xform {
  float q[4];
  float c[3];
  float t[3];
};

// One atom prepared for gridding (64 bytes).
//   a = {x, y, z, Tcull}     position after the transform; Tcull = largest squared distance that
//                            can still contribute (footprint culling)
//   b = {w, inv_ar2, Tg, inv_ar}   weight, 1/ar^2, Gaussian/quadratic switch threshold, 1/ar
//   c = {lo.x|lo.y<<16, hi.x|hi.y<<16, lo.z|hi.z<<16, chan|flags<<16}
//   d = {Tcut, Tbin, ar, densityrad}
// with ar = radius*radius_scale, Tcut from ar*final_radius_multiple, Tbin = ar*ar.
struct __align__(16) Rec {
  float4 a;
  float4 b;
  uint4 c;
  float4 d;
};

constexpr unsigned REC_VALID = 1u;     // contributes to some voxel

// Per (example, channel) radius constants for type-indexed radii.
struct __align__(16) ChanParam {
  float4 p;  // {inv_ar2, Tg, inv_ar, Tcut}
  float4 q;  // {Tbin, ar, densityrad, Tcull}
};

__device__ __forceinline__ float next_up(float x) { return __int_as_float(__float_as_int(x) + 1); }
__device__ __forceinline__ float next_down(float x) { return __int_as_float(__float_as_int(x) - 1); }

// Largest t >= 0 with sqrtf(t) <= cut (IEEE round-to-nearest sqrt); -1 if cut is negative or NaN.
__device__ __forceinline__ float sqrt_threshold(float cut) {
  if (!(cut >= 0.f)) return -1.f;
  if (isinf(cut)) return cut;
  float t = __fmul_rn(cut, cut);
  if (isinf(t)) t = 3.402823466e38f;
  for (int i = 0; i < 8 && t > 0.f && __fsqrt_rn(t) > cut; i++) t = next_down(t);
  for (int i = 0; i < 8; i++) {
    float n = next_up(t);
    if (isinf(n) || __fsqrt_rn(n) > cut) break;
    t = n;
  }
  return t;
}

// Quaternion product with libmolgrid's term order (include/libmolgrid/quaternion.h:82-91).
__device__ __forceinline__ void quat_mul(const float* l, const float* r, float* o) {
  float la = l[0], lb = l[1], lc = l[2], ld = l[3];
  float ra = r[0], rb = r[1], rc = r[2], rd = r[3];
  o[0] = __fsub_rn(__fsub_rn(__fsub_rn(__fmul_rn(la, ra), __fmul_rn(lb, rb)), __fmul_rn(lc, rc)), __fmul_rn(ld, rd));
  o[1] = __fsub_rn(__fadd_rn(__fadd_rn(__fmul_rn(la, rb), __fmul_rn(lb, ra)), __fmul_rn(lc, rd)), __fmul_rn(ld, rc));
  o[2] = __fadd_rn(__fadd_rn(__fsub_rn(__fmul_rn(la, rc), __fmul_rn(lb, rd)), __fmul_rn(lc, ra)), __fmul_rn(ld, rb));
  o[3] = __fadd_rn(__fsub_rn(__fadd_rn(__fmul_rn(la, rd), __fmul_rn(lb, rc)), __fmul_rn(lc, rb)), __fmul_rn(ld, ra));
}

__device__ __forceinline__ float quat_norm(const float* q) {
  return __fadd_rn(__fadd_rn(__fadd_rn(__fmul_rn(q[0], q[0]), __fmul_rn(q[1], q[1])), __fmul_rn(q[2], q[2])),
                   __fmul_rn(q[3], q[3]));
}

// conj(q)/norm(q), the right factor of Quaternion::rotate (quaternion.h:145-149)
__device__ __forceinline__ void quat_conj_over_norm(const float* q, float* o) {
  float n = quat_norm(q);
  o[0] = __fdiv_rn(q[0], n);
  o[1] = __fdiv_rn(-q[1], n);
  o[2] = __fdiv_rn(-q[2], n);
  o[3] = __fdiv_rn(-q[3], n);
}

// Quaternion::inverse (quaternion.h:163-166)
__device__ __forceinline__ void quat_inverse(const float* q, float* o) {
  float n = quat_norm(q);
  o[0] = __fdiv_rn(q[0], n);
  o[1] = __fdiv_rn(-q[1], n);
  o[2] = __fdiv_rn(-q[2], n);
  o[3] = __fdiv_rn(-q[3], n);
}

// q * (0,x,y,z) * cn  with cn = conj(q)/norm(q) precomputed
__device__ __forceinline__ void quat_rotate(const float* q, const float* cn, float x, float y, float z,
                                            float* out) {
  float p[4] = {0.f, x, y, z};
  float t[4], r[4];
  quat_mul(q, p, t);
  quat_mul(t, cn, r);
  out[0] = r[1];
  out[1] = r[2];
  out[2] = r[3];
}

// Quaternion::transform (quaternion.h:152-159)
__device__ __forceinline__ void xform_apply(const Xform& X, const float* cn, float& x, float& y, float& z,
                                            bool dotranslate) {
  float r[3];
  quat_rotate(X.q, cn, __fsub_rn(x, X.c[0]), __fsub_rn(y, X.c[1]), __fsub_rn(z, X.c[2]), r);
  float tx = dotranslate ? X.t[0] : 0.f, ty = dotranslate ? X.t[1] : 0.f, tz = dotranslate ? X.t[2] : 0.f;
  x = __fadd_rn(__fadd_rn(r[0], X.c[0]), tx);
  y = __fadd_rn(__fadd_rn(r[1], X.c[1]), ty);
  z = __fadd_rn(__fadd_rn(r[2], X.c[2]), tz);
}

// GridMaker::get_bounds_1d (src/grid_maker.cu:66-79); results clamped so that they fit 16 bits
__device__ __forceinline__ void bounds_1d(float origin, float coord, float densityrad, float res,
                                          unsigned dim, unsigned& lo, unsigned& hi) {
  lo = 0;
  hi = 0;
  float low = __fsub_rn(__fsub_rn(coord, densityrad), origin);
  if (low > 0.f) {
    float f = floorf(__fdiv_rn(low, res));
    lo = f >= (float)dim ? dim : (unsigned)f;
  }
  float high = __fsub_rn(__fadd_rn(coord, densityrad), origin);
  if (high > 0.f) {
    float c = ceilf(__fdiv_rn(high, res));
    hi = c >= (float)dim ? dim : (unsigned)c;
  }
}

__device__ __forceinline__ float voxel_coord(float origin, unsigned i, float res) {
  return __fadd_rn(origin, __fmul_rn((float)i, res));
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float sqrt_approx(float x) {
  float y;
  asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float rsqrt_approx(float x) {
  float y;
  asm("rsqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

constexpr float NEG2_LOG2E = -2.8853900817779268f;  // -2*log2(e)

// calc_point<false> (src/grid_maker.cu:95-118) on a precomputed squared distance.
// Fast form: one ex2, one sqrt, fused arithmetic; within ~1e-6 relative of the reference.
__device__ __forceinline__ float density_fast(float rsq, float inv_ar2, float Tg, float Tcut,
                                              float A, float B, float C) {
  float u = rsq * inv_ar2;
  float g = ex2_approx(u * NEG2_LOG2E);
  float s = sqrt_approx(u);
  float q = fmaxf(fmaf(fmaf(A, s, B), s, C), 0.f);
  float v = rsq <= Tg ? g : q;
  return rsq <= Tcut ? v : 0.f;
}

// Same function with the reference's own operation order and double intermediate.
__device__ __forceinline__ float density_precise(float rsq, float ar, float Tg, float Tcut,
                                                 float A, float B, float C) {
  if (!(rsq <= Tcut)) return 0.f;
  float dist = __fsqrt_rn(rsq);
  if (rsq <= Tg) {
    float ar2 = __fmul_rn(ar, ar);
    float ex = (float)(-2.0 * (double)dist * (double)dist / (double)ar2);
    return expf(ex);
  }
  float dr = __fdiv_rn(dist, ar);
  float q = __fadd_rn(__fmul_rn(__fadd_rn(__fmul_rn(A, dr), B), dr), C);
  return q > 0.f ? q : 0.f;
}

__device__ __forceinline__ unsigned lo16(unsigned v) { return v & 0xffffu; }
__device__ __forceinline__ unsigned hi16(unsigned v) { return v >> 16; }

}  // namespace lmg
