// sm_100a kernels for Transform forward/backward on coordinate arrays and for the
// GridInterpolater trilinear resample.
#include <cuda.h>
#include <stdint.h>

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

// What is the same for every output voxel of an example: grid origins and the inverse rotation.
struct InterpFrame {
  float iox, ioy, ioz, oox, ooy, ooz;
  float inv[4], cn[4];
  float ux, uy, uz, cx, cy, cz;
};

__device__ __forceinline__ InterpFrame interp_frame(const InterpArgs& I, const InterpExample& E) {
  InterpFrame F;
  F.iox = __fsub_rn(E.in_center[0], I.in_half);
  F.ioy = __fsub_rn(E.in_center[1], I.in_half);
  F.ioz = __fsub_rn(E.in_center[2], I.in_half);
  F.oox = __fsub_rn(E.out_center[0], I.out_half);
  F.ooy = __fsub_rn(E.out_center[1], I.out_half);
  F.ooz = __fsub_rn(E.out_center[2], I.out_half);
  quat_inverse(E.X.q, F.inv);
  quat_conj_over_norm(F.inv, F.cn);
  F.ux = __fsub_rn(-E.X.t[0], E.X.c[0]);
  F.uy = __fsub_rn(-E.X.t[1], E.X.c[1]);
  F.uz = __fsub_rn(-E.X.t[2], E.X.c[2]);
  F.cx = E.X.c[0]; F.cy = E.X.c[1]; F.cz = E.X.c[2];
  return F;
}

// Position of output voxel (i,j,k) in input-grid index units (src/grid_interpolater.cpp:31-45).
__device__ __forceinline__ void interp_point(const InterpArgs& I, const InterpFrame& F, unsigned i, unsigned j,
                                             unsigned k, float& gx, float& gy, float& gz) {
  float px = voxel_coord(F.oox, i, I.out_res), py = voxel_coord(F.ooy, j, I.out_res),
        pz = voxel_coord(F.ooz, k, I.out_res);
  float r[3];
  quat_rotate(F.inv, F.cn, __fadd_rn(px, F.ux), __fadd_rn(py, F.uy), __fadd_rn(pz, F.uz), r);
  gx = __fdiv_rn(__fsub_rn(__fadd_rn(r[0], F.cx), F.iox), I.in_res);
  gy = __fdiv_rn(__fsub_rn(__fadd_rn(r[1], F.cy), F.ioy), I.in_res);
  gz = __fdiv_rn(__fsub_rn(__fadd_rn(r[2], F.cz), F.ioz), I.in_res);
}

// Corner indices and weights of the trilinear blend (src/grid_interpolater.cu:26-58).
struct InterpCell {
  int xl, xh, yl, yh, zl, zh;
  float xd, yd, zd, xm, ym, zm;
};

__device__ __forceinline__ InterpCell interp_cell(float gx, float gy, float gz) {
  InterpCell C;
  C.xl = (int)floorf(gx); C.xh = (int)ceilf(gx);
  C.yl = (int)floorf(gy); C.yh = (int)ceilf(gy);
  C.zl = (int)floorf(gz); C.zh = (int)ceilf(gz);
  C.xd = C.xh > C.xl ? __fdiv_rn(__fsub_rn(gx, (float)C.xl), (float)(C.xh - C.xl)) : 0.f;
  C.yd = C.yh > C.yl ? __fdiv_rn(__fsub_rn(gy, (float)C.yl), (float)(C.yh - C.yl)) : 0.f;
  C.zd = C.zh > C.zl ? __fdiv_rn(__fsub_rn(gz, (float)C.zl), (float)(C.zh - C.zl)) : 0.f;
  C.xm = __fsub_rn(1.f, C.xd); C.ym = __fsub_rn(1.f, C.yd); C.zm = __fsub_rn(1.f, C.zd);
  return C;
}

__device__ __forceinline__ float interp_blend(const InterpCell& C, float p000, float p001, float p010,
                                              float p011, float p100, float p101, float p110, float p111) {
  float c00 = __fadd_rn(__fmul_rn(p000, C.xm), __fmul_rn(p100, C.xd));
  float c01 = __fadd_rn(__fmul_rn(p001, C.xm), __fmul_rn(p101, C.xd));
  float c10 = __fadd_rn(__fmul_rn(p010, C.xm), __fmul_rn(p110, C.xd));
  float c11 = __fadd_rn(__fmul_rn(p011, C.xm), __fmul_rn(p111, C.xd));
  float c0 = __fadd_rn(__fmul_rn(c00, C.ym), __fmul_rn(c10, C.yd));
  float c1 = __fadd_rn(__fmul_rn(c01, C.ym), __fmul_rn(c11, C.yd));
  return __fadd_rn(__fmul_rn(c0, C.zm), __fmul_rn(c1, C.zd));
}

// One channel of one output voxel read straight from the input grid.
__device__ __forceinline__ float interp_direct(const InterpCell& C, const float* g, int id) {
  if (C.xh < 0 || C.xl >= id || C.yh < 0 || C.yl >= id || C.zh < 0 || C.zl >= id) return 0.f;
  return interp_blend(C, get_pt(g, id, C.xl, C.yl, C.zl), get_pt(g, id, C.xl, C.yl, C.zh),
                      get_pt(g, id, C.xl, C.yh, C.zl), get_pt(g, id, C.xl, C.yh, C.zh),
                      get_pt(g, id, C.xh, C.yl, C.zl), get_pt(g, id, C.xh, C.yl, C.zh),
                      get_pt(g, id, C.xh, C.yh, C.zl), get_pt(g, id, C.xh, C.yh, C.zh));
}

// One thread per output voxel; the inverse transform is computed once and reused for every
// channel (GridInterpolater::forward, src/grid_interpolater.cpp:31-45).  Used when the input grid
// does not meet the alignment rules of the tiled kernel below.
__global__ void __launch_bounds__(256) k_interpolate(InterpArgs I) {
  int bl = blockIdx.y;
  const InterpExample& E = I.ex[bl];
  unsigned od = I.out_dim;
  unsigned v = blockIdx.x * blockDim.x + threadIdx.x;
  if (v >= od * od * od) return;
  unsigned k = v % od, j = (v / od) % od, i = v / (od * od);
  InterpFrame F = interp_frame(I, E);
  float gx, gy, gz;
  interp_point(I, F, i, j, k, gx, gy, gz);
  InterpCell C = interp_cell(gx, gy, gz);
  int id = (int)I.in_dim;
  size_t ichan = (size_t)id * id * id, ochan = (size_t)od * od * od;
  size_t b = (size_t)I.b0 + bl;
  const float* in = I.in + b * I.K * ichan;
  float* out = I.out + b * I.K * ochan + v;
  for (int c = 0; c < I.K; c++) __stcs(out + c * ochan, interp_direct(C, in + c * ichan, id));
}

// ---------------------------------------------------------------------------------------------
// Tiled interpolation: a block owns an ITILE^3 tile of output voxels (12^3).  The input voxels that
// tile can touch form a box (the rotated tile's bounding box, z rounded down to a 16-byte
// boundary).  One elected thread brings that box of channel c into shared memory with a single
// tensor copy (cp.async.bulk.tensor, zero fill outside the grid = the reference's zero padding)
// whose extents are, per axis, the smallest of a few fixed sizes that hold the tile (one tensor map
// per combination).  The staging area of a block is cut into as many slots as boxes of its extents
// fit (two to three on average, one for the few tiles that need the largest box), and each thread
// blends its voxels of the channel from shared memory.  The blend arithmetic is that of the direct
// kernel.  Every wait on a copy is bounded; a wait that runs out makes the block finish its tile
// through the direct reads.
// Measured per 48 examples of 28 x 48^3 with random rotations: tiles of 8^3 with 256 threads 0.683
// ms, 16^3 with 512 threads 0.644 ms, 12^3 with 432 threads and two blocks per SM 0.574 ms.  The
// number of slots (2 to 6) changes nothing: the kernel issues instructions 55 % of the time (about
// 65 per voxel and channel: 8 shared loads, 21 roundings of the blend, addresses) and its shared
// loads see three-way bank conflicts on average, which no row pitch that a tensor copy can write
// (multiples of 16 bytes) avoids for every rotation.  (Staging the box one x plane per copy, which
// needs fewer maps and fewer bytes, is slower: 1.08 against 0.83 ms - the copy engine works row by
// row and per copy.)
// ---------------------------------------------------------------------------------------------
__device__ unsigned g_tma_timeouts = 0;

__device__ __forceinline__ unsigned smem_u32(const void* p) {
  return (unsigned)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// false when the phase did not complete within the limit
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, unsigned parity) {
  for (int it = 0; it < (1 << 20); it++)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
__device__ __forceinline__ void tma_load_box(float* dst, const CUtensorMap* map, uint64_t* bar, int z, int y,
                                             int x, int chan) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(smem_u32(dst)),
      "l"(map), "r"(z), "r"(y), "r"(x), "r"(chan), "r"(smem_u32(bar))
      : "memory");
}

#ifndef LMG_INTERP_THREADS
#define LMG_INTERP_THREADS 432
#endif
#ifndef LMG_INTERP_MINBLOCKS
#define LMG_INTERP_MINBLOCKS 2
#endif
#ifndef LMG_INTERP_MAXSTAGES
#define LMG_INTERP_MAXSTAGES 4
#endif
constexpr int INT = LMG_INTERP_THREADS;                 // threads per block
constexpr int IVPT = ITILE * ITILE * ITILE / INT;       // voxels per thread
static_assert(IVPT * INT == ITILE * ITILE * ITILE, "the threads of a block share the tile evenly");
constexpr int IMAXST = LMG_INTERP_MAXSTAGES;            // most boxes in flight or in use per block
#ifndef LMG_INTERP_RING
#define LMG_INTERP_RING 28160  // 110 KB: two blocks per SM
#endif
constexpr int IRING = LMG_INTERP_RING;                  // floats of staging per block
static_assert(IMAXST >= 1 && IRING >= ITILE_BOX && IRING % 32 == 0, "the staging area holds at least one box");
static_assert(ITILE_BX * ITILE_BY * ITILE_BZ < (1 << 15) && ITILE_BY * ITILE_BZ < (1 << 10) && ITILE_BZ < (1 << 6),
              "a voxel's offsets into the box are packed into one word each");

// What a thread keeps per voxel between the channels: the offset of corner (xl, yl, zl) in the box,
// the steps to the upper corners (zero where floor == ceil) packed as sx | sy << 10 | sz << 16, and
// the three upper weights.
struct InterpVoxel {
  int base;
  unsigned steps;
  float xd, yd, zd;
};

__global__ void __launch_bounds__(INT, LMG_INTERP_MINBLOCKS) k_interpolate_tiled(const __grid_constant__ InterpMaps maps, InterpArgs I) {
  // the staging area is cut into as many slots as boxes of this block's extents fit
  extern __shared__ __align__(128) float ring[];
  __shared__ __align__(8) uint64_t bar[IMAXST];
  const int tid = threadIdx.x, bl = blockIdx.y;
  const InterpExample& E = I.ex[bl];
  const unsigned od = I.out_dim;
  const unsigned nt = (od + ITILE - 1) / ITILE;
  const unsigned tk = blockIdx.x % nt, tj = (blockIdx.x / nt) % nt, ti = blockIdx.x / (nt * nt);
  const InterpFrame F = interp_frame(I, E);

  // bounding box of the tile in input index units, from its eight corner voxels
  float lo[3] = {3e38f, 3e38f, 3e38f}, hi[3] = {-3e38f, -3e38f, -3e38f};
#pragma unroll
  for (int cnr = 0; cnr < 8; cnr++) {
    unsigned ci = min(ti * ITILE + ((cnr & 4) ? ITILE - 1 : 0), od - 1);
    unsigned cj = min(tj * ITILE + ((cnr & 2) ? ITILE - 1 : 0), od - 1);
    unsigned ck = min(tk * ITILE + ((cnr & 1) ? ITILE - 1 : 0), od - 1);
    float g[3];
    interp_point(I, F, ci, cj, ck, g[0], g[1], g[2]);
#pragma unroll
    for (int a = 0; a < 3; a++) {
      lo[a] = fminf(lo[a], g[a]);
      hi[a] = fmaxf(hi[a], g[a]);
    }
  }
  // every voxel of the tile lies in the hull of the corners up to rounding: a margin of 0.01 cells
  bool sane = true;
#pragma unroll
  for (int a = 0; a < 3; a++) sane = sane && lo[a] > -1e6f && hi[a] < 1e6f;  // also false for NaN
  int bx0 = 0, by0 = 0, bz0 = 0;
  int BX = ITILE_BX, BY = ITILE_BY, BZ = ITILE_BZ, mapi = 0;  // extents of the staged box
  bool tiled = sane;
  if (sane) {
    bx0 = (int)floorf(lo[0] - 0.01f);
    by0 = (int)floorf(lo[1] - 0.01f);
    int z0 = (int)floorf(lo[2] - 0.01f);
    bz0 = z0 & ~3;  // rounds down for negative values too (two's complement): 16-byte boundary
    int nx = (int)ceilf(hi[0] + 0.01f) - bx0 + 1, ny = (int)ceilf(hi[1] + 0.01f) - by0 + 1,
        nz = (int)ceilf(hi[2] + 0.01f) - bz0 + 1;
    tiled = nx <= ITILE_BX && ny <= ITILE_BY && nz <= ITILE_BZ;
    int ix = nx <= ITILE_XY0 ? 0 : (nx - ITILE_XY0 + ITILE_XYSTEP - 1) / ITILE_XYSTEP;
    int iy = ny <= ITILE_XY0 ? 0 : (ny - ITILE_XY0 + ITILE_XYSTEP - 1) / ITILE_XYSTEP;
    int iz = nz <= ITILE_Z0 ? 0 : (nz - ITILE_Z0 + 3) / 4;
    BX = itile_xy(ix);
    BY = itile_xy(iy);
    BZ = itile_z(iz);
    mapi = (ix * ITILE_NXY + iy) * ITILE_NZ + iz;
  }

  // this thread's voxels
  const int id = (int)I.in_dim;
  const size_t ichan = (size_t)id * id * id, ochan = (size_t)od * od * od;
  const size_t b = (size_t)I.b0 + bl;
  const float* in = I.in + b * I.K * ichan;
  float* outb = I.out + b * I.K * ochan;
  InterpVoxel V[IVPT];
  unsigned livemask = 0;
  static_assert(INT % (ITILE * ITILE) == 0, "a thread's voxels differ in the slowest index only");
  // voxel u of this thread: (i0 + u * INT / ITILE^2, j0, k0) within the tile
  const unsigned i0 = ti * ITILE + tid / (ITILE * ITILE), j0 = tj * ITILE + (tid / ITILE) % ITILE,
                 k0 = tk * ITILE + tid % ITILE;
  const size_t ov0 = ((size_t)i0 * od + j0) * od + k0;
  const size_t ovstep = (size_t)(INT / (ITILE * ITILE)) * od * od;
#pragma unroll
  for (int u = 0; u < IVPT; u++) {
    unsigned i = i0 + u * (INT / (ITILE * ITILE));
    bool live = i < od && j0 < od && k0 < od;
    float gx, gy, gz;
    interp_point(I, F, min(i, od - 1), min(j0, od - 1), min(k0, od - 1), gx, gy, gz);
    InterpCell C = interp_cell(gx, gy, gz);
    V[u].base = ((C.xl - bx0) * BY + (C.yl - by0)) * BZ + (C.zl - bz0);
    V[u].steps = (unsigned)((C.xh - C.xl) * BY * BZ) | (unsigned)((C.yh - C.yl) * BZ) << 10 |
                 (unsigned)(C.zh - C.zl) << 16;
    V[u].xd = C.xd; V[u].yd = C.yd; V[u].zd = C.zd;
    // belt and braces: a corner outside the staged box sends the whole block down the direct path
    bool inside = C.xl >= bx0 && C.xh < bx0 + BX && C.yl >= by0 && C.yh < by0 + BY &&
                  C.zl >= bz0 && C.zh < bz0 + BZ;
    if (live && !inside) tiled = false;
    if (live) livemask |= 1u << u;
    if (!live) {  // reads the first word of the box, stores nothing
      V[u].base = 0;
      V[u].steps = 0;
    }
  }
  tiled = __syncthreads_and(tiled) != 0;

  int c = 0;
  if (tiled) {
    const int chan0 = (int)(b * I.K);
    const int slot = (BX * BY * BZ + 31) & ~31;  // floats from box to box: 128-byte boundaries
    const int nst = min(IMAXST, IRING / slot);
    if (tid == 0) {
      for (int s = 0; s < IMAXST; s++) mbar_init(&bar[s], 1);
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const CUtensorMap* map = &maps.m[mapi];
    auto stage = [&](int s, int chan) {
      mbar_expect_tx(&bar[s], (unsigned)(BX * BY * BZ) * (unsigned)sizeof(float));
      tma_load_box(ring + s * slot, map, &bar[s], bz0, by0, bx0, chan);
    };
    if (tid == 0) {
      for (int s = 0; s < nst && s < I.K; s++) stage(s, chan0 + s);
    }
    int inflight = min(nst, I.K);
    int s = 0;
    unsigned phase = 0;
    float* oc = outb + ov0;  // this thread's first voxel in channel c
    for (; c < I.K; c++, oc += ochan) {
      bool ok = mbar_wait_bounded(&bar[s], phase);
      if (__syncthreads_or(!ok)) break;  // a copy did not arrive: finish through the direct reads
      inflight--;
      const float* sm = ring + s * slot;
#pragma unroll
      for (int u = 0; u < IVPT; u++) {
        const float* p = sm + V[u].base;
        const int sx = (int)(V[u].steps & 1023u), sy = (int)(V[u].steps >> 10 & 63u), sz = (int)(V[u].steps >> 16);
        InterpCell C;
        C.xd = V[u].xd; C.yd = V[u].yd; C.zd = V[u].zd;
        C.xm = __fsub_rn(1.f, C.xd); C.ym = __fsub_rn(1.f, C.yd); C.zm = __fsub_rn(1.f, C.zd);
        float res = interp_blend(C, p[0], p[sz], p[sy], p[sy + sz], p[sx], p[sx + sz], p[sx + sy], p[sx + sy + sz]);
        if (livemask >> u & 1u) __stcs(oc + u * ovstep, res);
      }
      __syncthreads();  // everyone is done with this slot before it is refilled
      if (tid == 0 && c + nst < I.K) stage(s, chan0 + c + nst);
      if (c + nst < I.K) inflight++;
      if (++s == nst) {
        s = 0;
        phase ^= 1u;
      }
    }
    if (c < I.K) {
      // give the copies still in flight a second, equally bounded chance to land before the shared
      // memory is given up; then fall through to the direct reads
      if (tid == 0) atomicAdd(&g_tma_timeouts, 1u);
      for (int w = 0; w < inflight; w++) {
        mbar_wait_bounded(&bar[s], phase);
        if (++s == nst) {
          s = 0;
          phase ^= 1u;
        }
      }
      __syncthreads();
    }
  }
  if (c < I.K) {
    const InterpFrame F2 = interp_frame(I, E);  // computed again: nothing of it stays live over the channel loop
#pragma unroll 1
    for (int u = 0; u < IVPT; u++) {
      if (!(livemask >> u & 1u)) continue;
      float gx, gy, gz;
      interp_point(I, F2, i0 + u * (INT / (ITILE * ITILE)), j0, k0, gx, gy, gz);
      InterpCell C = interp_cell(gx, gy, gz);
      size_t ov = ov0 + u * ovstep;
      for (int cc = c; cc < I.K; cc++) __stcs(outb + cc * ochan + ov, interp_direct(C, in + cc * ichan, id));
    }
  }
}

unsigned interp_tile_count(unsigned out_dim) {
  unsigned nt = (out_dim + ITILE - 1) / ITILE;
  return nt * nt * nt;
}

cudaError_t launch_interpolate_tiled(const InterpMaps& maps, const InterpArgs& I, int nb, cudaStream_t st) {
  unsigned ntiles = interp_tile_count(I.out_dim);
  if (ntiles == 0 || nb == 0 || I.K == 0) return cudaSuccess;
  dim3 grid(ntiles, nb);
  constexpr size_t smem = (size_t)IRING * sizeof(float);
  if (smem > 48 * 1024) {
    // more than the default dynamic shared memory: opted into once per device
    static bool opted[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64 || !opted[dev]) {
      e = cudaFuncSetAttribute(k_interpolate_tiled, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return e;
      if (dev >= 0 && dev < 64) opted[dev] = true;
    }
  }
  k_interpolate_tiled<<<grid, INT, smem, st>>>(maps, I);
  return cudaGetLastError();
}

cudaError_t read_tma_timeouts(unsigned* count) {
  return cudaMemcpyFromSymbol(count, g_tma_timeouts, sizeof(unsigned));
}

// Adjoint of the interpolation (the reference leaves it as a TODO, include/libmolgrid/
// grid_interpolater.h:179): every output voxel hands its gradient to the eight input voxels it was
// blended from, with the forward pass's weights; contributions outside the input grid are dropped,
// as their values were zeros in the forward pass.  I.in is the gradient with respect to the output
// (read), I.out the gradient with respect to the input (zero-filled by the caller, accumulated here).
__global__ void __launch_bounds__(256) k_interpolate_backward(InterpArgs I) {
  int bl = blockIdx.y;
  const InterpExample& E = I.ex[bl];
  unsigned od = I.out_dim;
  unsigned v = blockIdx.x * blockDim.x + threadIdx.x;
  if (v >= od * od * od) return;
  unsigned k = v % od, j = (v / od) % od, i = v / (od * od);
  InterpFrame F = interp_frame(I, E);
  float gx, gy, gz;
  interp_point(I, F, i, j, k, gx, gy, gz);
  InterpCell C = interp_cell(gx, gy, gz);
  int id = (int)I.in_dim;
  if (C.xh < 0 || C.xl >= id || C.yh < 0 || C.yl >= id || C.zh < 0 || C.zl >= id) return;
  size_t ichan = (size_t)id * id * id, ochan = (size_t)od * od * od;
  size_t b = (size_t)I.b0 + bl;
  const float* gout = I.in + b * I.K * ochan + v;
  float* gin = I.out + b * I.K * ichan;
  // corner (a,b,c) has weight wx[a]*wy[b]*wz[c], the factors of interp_blend
  int xs[2] = {C.xl, C.xh}, ys[2] = {C.yl, C.yh}, zs[2] = {C.zl, C.zh};
  float wx[2] = {C.xm, C.xd}, wy[2] = {C.ym, C.yd}, wz[2] = {C.zm, C.zd};
  for (int c = 0; c < I.K; c++) {
    float g = __ldg(gout + c * ochan);
    if (g == 0.f) continue;
    float* gc = gin + c * ichan;
#pragma unroll
    for (int a = 0; a < 2; a++)
#pragma unroll
      for (int bb = 0; bb < 2; bb++)
#pragma unroll
        for (int cc = 0; cc < 2; cc++) {
          int x = xs[a], y = ys[bb], z = zs[cc];
          float w = wx[a] * wy[bb] * wz[cc];
          if (w != 0.f && x >= 0 && x < id && y >= 0 && y < id && z >= 0 && z < id)
            atomicAdd(gc + ((size_t)x * id + y) * id + z, w * g);
        }
  }
}

cudaError_t launch_interpolate_backward(const InterpArgs& I, int nb, cudaStream_t st) {
  unsigned nv = I.out_dim * I.out_dim * I.out_dim;
  if (nv == 0 || nb == 0 || I.K == 0) return cudaSuccess;
  dim3 grid((nv + 255) / 256, nb);
  k_interpolate_backward<<<grid, 256, 0, st>>>(I);
  return cudaGetLastError();
}

cudaError_t launch_interpolate(const InterpArgs& I, int nb, cudaStream_t st) {
  unsigned nv = I.out_dim * I.out_dim * I.out_dim;
  if (nv == 0 || nb == 0 || I.K == 0) return cudaSuccess;
  dim3 grid((nv + 255) / 256, nb);
  k_interpolate<<<grid, 256, 0, st>>>(I);
  return cudaGetLastError();
}

}  // namespace lmg
