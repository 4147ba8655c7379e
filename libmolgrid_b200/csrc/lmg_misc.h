// Launchers of the Transform and GridInterpolater kernels.
#pragma once
#include <cuda.h>
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
// adjoint: I.in = gradient of the output grid (read), I.out = gradient of the input grid (accumulated)
cudaError_t launch_interpolate_backward(const InterpArgs& I, int nb, cudaStream_t st);

// Tiled kernel: output tiles of ITILE^3 voxels read a staged box of the input of at most
// ITILE_BX x ITILE_BY x ITILE_BZ voxels (z is the contiguous axis; the box starts on a multiple of
// four).  Each axis of the box takes the smallest of a few fixed extents that hold the tile, one
// tensor map per combination: a rotated 8^3 tile needs 12.5 x 12.5 x 12.5 input voxels on average
// and 16 x 16 x 16 at worst, so the staged boxes hold 3200 floats on average instead of 5120.
constexpr int ITILE = 8;
constexpr int ITILE_BX = 16, ITILE_BY = 16, ITILE_BZ = 20;
constexpr int ITILE_BOX = ITILE_BX * ITILE_BY * ITILE_BZ;
constexpr int ITILE_NXY = 4, ITILE_NZ = 3;
constexpr int ITILE_XYS[ITILE_NXY] = {10, 12, 14, 16};
constexpr int ITILE_ZS[ITILE_NZ] = {12, 16, 20};
struct alignas(64) InterpMaps {
  // [(ix * ITILE_NXY + iy) * ITILE_NZ + iz]: box {ITILE_ZS[iz], ITILE_XYS[iy], ITILE_XYS[ix], 1}
  CUtensorMap m[ITILE_NXY * ITILE_NXY * ITILE_NZ];
};
// the maps describe the input as a 4-d tensor {z, y, x, example*channels}
cudaError_t launch_interpolate_tiled(const InterpMaps& maps, const InterpArgs& I, int nb, cudaStream_t st);
// how many blocks ever gave up waiting for a staged box (they finish through direct reads)
cudaError_t read_tma_timeouts(unsigned* count);

}  // namespace lmg
