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

// Tiled kernel: output tiles of ITILE^3 voxels read a staged box of the input (z is the contiguous
// axis; the box starts on a multiple of four in z).  A rotated tile needs (ITILE - 1) * (|r1| + |r2| +
// |r3|) + 2 input voxels along an axis (r the row of the rotation): ITILE + 1 unrotated, 1.5 ITILE on
// average, sqrt(3) ITILE at worst.  Each axis of the box takes the smallest of a few fixed extents
// that hold the tile, one tensor map per combination.  Tiles of 12^3 stage 5.8 input voxels per
// output voxel on average (8^3: 6.2 after the rounding of the extents, 16^3: 4.6 but one block per SM).
#ifndef LMG_ITILE
#define LMG_ITILE 12
#endif
#ifndef LMG_ITILE_XYSTEP
#define LMG_ITILE_XYSTEP 2
#endif
constexpr int ITILE = LMG_ITILE;
constexpr int ITILE_XYSTEP = LMG_ITILE_XYSTEP;
constexpr int ITILE_NEED = (int)((ITILE - 1) * 1.7321f + 3.02f);  // largest extent a tile can ask for
constexpr int ITILE_XY0 = ITILE + 2;                              // smallest x / y extent on offer
constexpr int ITILE_NXY = (ITILE_NEED + 1 - ITILE_XY0 + ITILE_XYSTEP - 1) / ITILE_XYSTEP + 1;
constexpr int ITILE_Z0 = (ITILE + 4 + 3) & ~3;                    // z extents: multiples of four
constexpr int ITILE_NZ = (((ITILE_NEED + 3 + 3) & ~3) - ITILE_Z0) / 4 + 1;
__host__ __device__ constexpr int itile_xy(int i) { return ITILE_XY0 + i * ITILE_XYSTEP; }
__host__ __device__ constexpr int itile_z(int i) { return ITILE_Z0 + 4 * i; }
constexpr int ITILE_BX = itile_xy(ITILE_NXY - 1), ITILE_BY = ITILE_BX, ITILE_BZ = itile_z(ITILE_NZ - 1);
constexpr int ITILE_BOX = ITILE_BX * ITILE_BY * ITILE_BZ;
struct alignas(64) InterpMaps {
  // [(ix * ITILE_NXY + iy) * ITILE_NZ + iz]: box {itile_z(iz), itile_xy(iy), itile_xy(ix), 1}
  CUtensorMap m[ITILE_NXY * ITILE_NXY * ITILE_NZ];
};
// the maps describe the input as a 4-d tensor {z, y, x, example*channels}
cudaError_t launch_interpolate_tiled(const InterpMaps& maps, const InterpArgs& I, int nb, cudaStream_t st);
// how many blocks ever gave up waiting for a staged box (they finish through direct reads)
cudaError_t read_tma_timeouts(unsigned* count);

}  // namespace lmg
