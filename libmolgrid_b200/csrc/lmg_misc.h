// Launchers of the Transform and GridInterpolater kernels.
#pragma once
#include <cuda_runtime.h>

#include "lmg_device.cuh"

namespace lmg {

struct InterpExample {
  Xform X;
  float in_center[3];
  float out_center[3];
};

// examples per launch whose transforms travel inside the kernel parameter block
constexpr int INTERP_MAX_EX = 48;

struct InterpArgs {
  float in_res, out_res, in_half, out_half;
  unsigned in_dim, out_dim;
  int K;
  int b0;
  const float* in;
  float* out;
  InterpExample ex[INTERP_MAX_EX];
};

cudaError_t launch_transform(const Xform& X, int n, const float* in, float* out, int dotranslate,
                             bool forward, cudaStream_t st);
cudaError_t launch_interpolate(const InterpArgs& I, int nb, cudaStream_t st);

}  // namespace lmg
