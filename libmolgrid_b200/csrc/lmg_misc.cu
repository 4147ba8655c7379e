// sm_100a kernels for Transform forward/backward on coordinate arrays and for the
// GridInterpolater trilinear resample.
#include "lmg_device.cuh"
#include "lmg_misc.h"

namespace lmg {

// Transform::forward (src/transform.cpp:57-79): Q.transform(x, y, z, center, translate)
__global__ void __launch_bounds__(256) k_transform_forward(Xform X, int n, const float* in, float* out,
                                                           int dotranslate) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float cn[4];
  quat_conj_over_norm(X.q, cn);
  float x = in[3 * i], y = in[3 * i + 1], z = in[3 * i + 2];
  xform_apply(X, cn, x, y, z, dotranslate != 0);
  out[3 * i] = x;
  out[3 * i + 1] = y;
  out[3 * i + 2] = z;
}

// Transform::backward (src/transform.cpp:85-108): untranslate, rotate by the inverse, re-centre
__global__ void __launch_bounds__(256) k_transform_backward(Xform X, int n, const float* in, float* out,
                                                            int dotranslate) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float inv[4], cn[4];
  quat_inverse(X.q, inv);
  quat_conj_over_norm(inv, cn);
  float ux, uy, uz;
  if (dotranslate) {
    ux = __fsub_rn(-X.t[0], X.c[0]); uy = __fsub_rn(-X.t[1], X.c[1]); uz = __fsub_rn(-X.t[2], X.c[2]);
  } else {
    ux = -X.c[0]; uy = -X.c[1]; uz = -X.c[2];
  }
  float r[3];
  quat_rotate(inv, cn, __fadd_rn(in[3 * i], ux), __fadd_rn(in[3 * i + 1], uy), __fadd_rn(in[3 * i + 2], uz), r);
  out[3 * i] = __fadd_rn(r[0], X.c[0]);
  out[3 * i + 1] = __fadd_rn(r[1], X.c[1]);
  out[3 * i + 2] = __fadd_rn(r[2], X.c[2]);
}

cudaError_t launch_transform(const Xform& X, int n, const float* in, float* out, int dotranslate,
                             bool forward, cudaStream_t st) {
  if (n <= 0) return cudaSuccess;
  int blocks = (n + 255) / 256;
  if (forward)
    k_transform_forward<<<blocks, 256, 0, st>>>(X, n, in, out, dotranslate);
  else
    k_transform_backward<<<blocks, 256, 0, st>>>(X, n, in, out, dotranslate);
  return cudaGetLastError();
}

// GridInterpolater::get_pt (src/grid_interpolater.cu:16-22)
__device__ __forceinline__ float get_pt(const float* in, int dim, int x, int y, int z) {
  if (x < 0 || x >= dim || y < 0 || y >= dim || z < 0 || z >= dim) return 0.f;
  return __ldg(in + ((size_t)x * dim + y) * dim + z);
}

// One thread per output voxel; the inverse transform is computed once and reused for every
// channel (GridInterpolater::forward, src/grid_interpolater.cpp:31-45; interpolate,
// src/grid_interpolater.cu:26-58).
__global__ void __launch_bounds__(256) k_interpolate(InterpArgs I) {
  int bl = blockIdx.y;
  const InterpExample& E = I.ex[bl];
  unsigned od = I.out_dim;
  unsigned v = blockIdx.x * blockDim.x + threadIdx.x;
  if (v >= od * od * od) return;
  unsigned k = v % od, j = (v / od) % od, i = v / (od * od);

  float in_radius = I.in_half, out_radius = I.out_half;
  float iox = __fsub_rn(E.in_center[0], in_radius), ioy = __fsub_rn(E.in_center[1], in_radius),
        ioz = __fsub_rn(E.in_center[2], in_radius);
  float oox = __fsub_rn(E.out_center[0], out_radius), ooy = __fsub_rn(E.out_center[1], out_radius),
        ooz = __fsub_rn(E.out_center[2], out_radius);
  float inv[4], cn[4];
  quat_inverse(E.X.q, inv);
  quat_conj_over_norm(inv, cn);
  float ux = __fsub_rn(-E.X.t[0], E.X.c[0]), uy = __fsub_rn(-E.X.t[1], E.X.c[1]),
        uz = __fsub_rn(-E.X.t[2], E.X.c[2]);
  float px = voxel_coord(oox, i, I.out_res), py = voxel_coord(ooy, j, I.out_res),
        pz = voxel_coord(ooz, k, I.out_res);
  float r[3];
  quat_rotate(inv, cn, __fadd_rn(px, ux), __fadd_rn(py, uy), __fadd_rn(pz, uz), r);
  float gx = __fdiv_rn(__fsub_rn(__fadd_rn(r[0], E.X.c[0]), iox), I.in_res);
  float gy = __fdiv_rn(__fsub_rn(__fadd_rn(r[1], E.X.c[1]), ioy), I.in_res);
  float gz = __fdiv_rn(__fsub_rn(__fadd_rn(r[2], E.X.c[2]), ioz), I.in_res);

  int xl = (int)floorf(gx), xh = (int)ceilf(gx);
  int yl = (int)floorf(gy), yh = (int)ceilf(gy);
  int zl = (int)floorf(gz), zh = (int)ceilf(gz);
  float xd = xh > xl ? __fdiv_rn(__fsub_rn(gx, (float)xl), (float)(xh - xl)) : 0.f;
  float yd = yh > yl ? __fdiv_rn(__fsub_rn(gy, (float)yl), (float)(yh - yl)) : 0.f;
  float zd = zh > zl ? __fdiv_rn(__fsub_rn(gz, (float)zl), (float)(zh - zl)) : 0.f;
  float xm = __fsub_rn(1.f, xd), ym = __fsub_rn(1.f, yd), zm = __fsub_rn(1.f, zd);

  int id = (int)I.in_dim;
  size_t ichan = (size_t)id * id * id, ochan = (size_t)od * od * od;
  size_t b = (size_t)I.b0 + bl;
  const float* in = I.in + b * I.K * ichan;
  float* out = I.out + b * I.K * ochan + v;
  bool any = !(xh < 0 || xl >= id || yh < 0 || yl >= id || zh < 0 || zl >= id);
  for (int c = 0; c < I.K; c++) {
    float res = 0.f;
    if (any) {
      const float* g = in + c * ichan;
      float p000 = get_pt(g, id, xl, yl, zl), p001 = get_pt(g, id, xl, yl, zh);
      float p010 = get_pt(g, id, xl, yh, zl), p011 = get_pt(g, id, xl, yh, zh);
      float p100 = get_pt(g, id, xh, yl, zl), p101 = get_pt(g, id, xh, yl, zh);
      float p110 = get_pt(g, id, xh, yh, zl), p111 = get_pt(g, id, xh, yh, zh);
      float c00 = __fadd_rn(__fmul_rn(p000, xm), __fmul_rn(p100, xd));
      float c01 = __fadd_rn(__fmul_rn(p001, xm), __fmul_rn(p101, xd));
      float c10 = __fadd_rn(__fmul_rn(p010, xm), __fmul_rn(p110, xd));
      float c11 = __fadd_rn(__fmul_rn(p011, xm), __fmul_rn(p111, xd));
      float c0 = __fadd_rn(__fmul_rn(c00, ym), __fmul_rn(c10, yd));
      float c1 = __fadd_rn(__fmul_rn(c01, ym), __fmul_rn(c11, yd));
      res = __fadd_rn(__fmul_rn(c0, zm), __fmul_rn(c1, zd));
    }
    __stcs(out + c * ochan, res);
  }
}

cudaError_t launch_interpolate(const InterpArgs& I, int nb, cudaStream_t st) {
  unsigned nv = I.out_dim * I.out_dim * I.out_dim;
  if (nv == 0 || nb == 0 || I.K == 0) return cudaSuccess;
  dim3 grid((nv + 255) / 256, nb);
  k_interpolate<<<grid, 256, 0, st>>>(I);
  return cudaGetLastError();
}

}  // namespace lmg
