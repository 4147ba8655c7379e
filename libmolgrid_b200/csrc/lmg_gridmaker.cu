// sm_100a kernels for GridMaker forward / backward / backward_gradients / backward_relevance.
//
// Every pass starts with emit: one thread per atom - fused Transform, exact footprint bounds and
// distance thresholds -> 64-byte atom record.
//
// Default forward: the output is zero-filled, then one warp per atom (per (atom, channel) with vector
// types) compacts the columns of the atom's footprint that lie inside the cut-off circle and adds
// the density into the grid with red.global.add (k_forward_quads*, k_forward_scatter).
// Backward passes: one warp per atom reads the grid gradient under the footprint and reduces with
// shuffles, so no global atomics are needed (k_backward_quads*, k_backward_warp).
#include "lmg_device.cuh"
#include "lmg_launch.h"

namespace lmg {

// ---------------------------------------------------------------------------------------------
// emit
// ---------------------------------------------------------------------------------------------

// Type-indexed radii: constants of channel t of example b.
__device__ __forceinline__ void make_chan_param(const GMParams& gm, float radius, ChanParam& cp) {
  float ar = __fmul_rn(radius, gm.rscale);
  float densityrad = __fmul_rn(ar, gm.finalm);
  float Tcut = sqrt_threshold(densityrad);
  float Tg = sqrt_threshold(__fmul_rn(ar, gm.G));
  float Tbin = __fmul_rn(ar, ar);
  bool ok = ar > 0.f;
  float inv_ar = ok ? 1.f / ar : 0.f;
  float inv_ar2 = ok ? 1.f / Tbin : 0.f;
  if (!ok) { Tcut = -1.f; Tg = -1.f; Tbin = -1.f; }
  cp.p = make_float4(inv_ar2, Tg, inv_ar, Tcut);
  cp.q = make_float4(Tbin, ar, densityrad, fmaxf(Tcut, gm.binary ? Tbin : -1.f));
}

__global__ void __launch_bounds__(256) k_chan_params(EmitArgs A) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= A.nb * A.T) return;
  int b = A.b0 + i / A.T, t = i % A.T;
  ChanParam cp;
  make_chan_param(A.gm, A.radii[(size_t)b * A.T + t], cp);
  A.chanp[i] = cp;
}

// One thread per atom slot of the pass.
__global__ void __launch_bounds__(256) k_emit(EmitArgs A) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= A.nb * A.N) return;
  int bl = i / A.N, a = i - bl * A.N;
  int b = A.b0 + bl;
  const GMParams& gm = A.gm;

  Rec r;
  r.a = make_float4(0.f, 0.f, 0.f, -1.f);
  r.b = make_float4(0.f, 0.f, -1.f, 0.f);
  r.c = make_uint4(0u, 0u, 0u, 0u);
  r.d = make_float4(-1.f, -1.f, 0.f, 0.f);

  bool valid = A.n_atoms == nullptr || a < A.n_atoms[b];
  int chan = 0;
  float ox = 0.f, oy = 0.f, oz = 0.f;
  if (valid && !A.vec) {
    float tf = A.type_index[(size_t)b * A.N + a];
    // forward takes floor (src/grid_maker.cpp:171), the backward passes round (:456, :698)
    float tc = A.round_types ? roundf(tf) : floorf(tf);
    if (!(tc >= 0.f)) {
      valid = false;
    } else if (tc >= (float)A.T) {
      valid = false;
      if (A.check_types) atomicMax(A.status, A.round_types ? 2 : 1);
    } else {
      chan = (int)tc;
    }
  }
  if (valid) {
    size_t ci = ((size_t)b * A.N + a) * 3;
    float x = A.coords[ci], y = A.coords[ci + 1], z = A.coords[ci + 2];
    if (A.transforms != nullptr || A.has_xform_host) {
      Xform X = A.transforms != nullptr ? A.transforms[b] : A.xform_host;
      float cn[4];
      quat_conj_over_norm(X.q, cn);
      xform_apply(X, cn, x, y, z, true);
    }
    float cx, cy, cz;
    if (A.centers != nullptr) {
      cx = A.centers[b * 3]; cy = A.centers[b * 3 + 1]; cz = A.centers[b * 3 + 2];
    } else {
      cx = A.center_host[0]; cy = A.center_host[1]; cz = A.center_host[2];
    }
    ox = __fsub_rn(cx, gm.half); oy = __fsub_rn(cy, gm.half); oz = __fsub_rn(cz, gm.half);

    float radius;
    if (gm.rti) {
      // footprint for binning = the largest channel radius of this example
      radius = -CUDART_INF_F;
      for (int t = 0; t < A.T; t++) radius = fmaxf(radius, A.radii[(size_t)b * A.T + t]);
    } else {
      radius = A.radii[(size_t)b * A.N + a];
    }
    ChanParam cp;
    make_chan_param(gm, radius, cp);
    float densityrad = cp.q.z;
    // binary occupancy extends to ar, which exceeds densityrad only when final_radius_multiple < 1;
    // the reference still clips it to the densityrad footprint, and so do the bounds below
    unsigned lox, hix, loy, hiy, loz, hiz;
    bounds_1d(ox, x, densityrad, gm.res, gm.dim, lox, hix);
    bounds_1d(oy, y, densityrad, gm.res, gm.dim, loy, hiy);
    bounds_1d(oz, z, densityrad, gm.res, gm.dim, loz, hiz);
    bool any = cp.q.y > 0.f && hix > lox && hiy > loy && hiz > loz;
    if (any) {
      r.a = make_float4(x, y, z, cp.q.w);
      r.b = make_float4(1.f, cp.p.x, cp.p.y, cp.p.z);
      r.c = make_uint4(lox | (loy << 16), hix | (hiy << 16), loz | (hiz << 16),
                       (unsigned)chan | (REC_VALID << 16));
      r.d = make_float4(cp.p.w, cp.q.x, cp.q.y, cp.q.z);
    }
    valid = any;
  }

  A.recs[i] = r;
}

// ---------------------------------------------------------------------------------------------
// backward
// ---------------------------------------------------------------------------------------------

struct ItemParams {
  float x, y, z;
  float inv_ar2, inv_ar, Tg, Tcut, Tbin, w, ar;
  unsigned lox, hix, loy, hiy, loz, hiz;
  int chan;
  bool valid;
};

// Loads the constants of work item `item` (an atom, or an (atom, channel) pair with VEC).
template <bool VEC>
__device__ __forceinline__ ItemParams load_item(const BwdArgs& G, int bl, int b, int item,
                                                float ox, float oy, float oz) {
  ItemParams P;
  int ai = VEC ? item / G.T : item;
  const Rec* rp = G.recs + (size_t)bl * G.N + ai;
  float4 ra = rp->a, rb = rp->b, rd = rp->d;
  uint4 rc = rp->c;
  P.valid = ((rc.w >> 16) & REC_VALID) != 0;
  P.x = ra.x; P.y = ra.y; P.z = ra.z;
  P.chan = VEC ? item - ai * G.T : (int)(rc.w & 0xffffu);
  P.w = 1.f;
  if (VEC) P.w = G.type_vector[((size_t)b * G.N + ai) * G.T + P.chan];
  if (VEC && G.gm.rti) {
    ChanParam cp = G.chanp[(size_t)bl * G.T + P.chan];
    P.inv_ar2 = cp.p.x; P.Tg = cp.p.y; P.inv_ar = cp.p.z; P.Tcut = cp.p.w; P.Tbin = cp.q.x;
    P.ar = cp.q.y;
    bounds_1d(ox, P.x, cp.q.z, G.gm.res, G.gm.dim, P.lox, P.hix);
    bounds_1d(oy, P.y, cp.q.z, G.gm.res, G.gm.dim, P.loy, P.hiy);
    bounds_1d(oz, P.z, cp.q.z, G.gm.res, G.gm.dim, P.loz, P.hiz);
    P.valid = P.valid && cp.q.y > 0.f;
  } else {
    P.inv_ar2 = rb.y; P.Tg = rb.z; P.inv_ar = rb.w; P.Tcut = rd.x; P.Tbin = rd.y; P.ar = rd.z;
    P.lox = lo16(rc.x); P.loy = hi16(rc.x); P.hix = lo16(rc.y); P.hiy = hi16(rc.y);
    P.loz = lo16(rc.z); P.hiz = hi16(rc.z);
  }
  return P;
}

// Backward and scatter-forward kernels: one warp per work item.  The warp first compacts the
// columns (x,y) of the item's footprint that lie within the cut-off circle, then sweeps eight
// columns at a time with four lanes along z each, and finally reduces with shuffles.  All lanes
// work on the same atom, so footprints of different size do not idle each other.
//
// Everything that depends on z alone (dz, dz^2, the z factor of the Gaussian) is the same for every
// column, so each lane keeps it in registers for its (up to) four z positions of the current chunk
// of 16 voxels; everything that depends on (x,y) alone is computed once per column at compaction
// time and parked in shared memory.  The inner step is then  rsq = dxy2 + dz2[k]  (the reference's
// own association, src/grid_maker.cu:82-92), one compare, and the density arithmetic.  The Gaussian
// is evaluated as exp(-2 dxy2/ar^2) * exp(-2 dz2/ar^2): one ex2 per column instead of one per voxel.
// One warp per block in the backward kernels: the kernel waits on its loads of the grid gradient,
// and a block of several warps keeps its registers until its slowest atom is done.
#ifndef LMG_BWD_WARPS
#define LMG_BWD_WARPS 1
#endif
#ifndef LMG_SCAT_WARPS
#define LMG_SCAT_WARPS 4
#endif
constexpr int BWD2_WARPS = LMG_BWD_WARPS;    // warps (work items) per block, backward kernels
constexpr int SCAT_WARPS = LMG_SCAT_WARPS;   // the same for the scatter kernels
// One warp per block for the quad forward kernels whose work items differ a lot in size (an atom's
// footprint grows with the cube of its radius): a block of several warps keeps its registers and
// its slot until its slowest item is done.  Measured per batch of 50: index-typed forward 0.266 ->
// 0.258 ms, one-hot vector forward 0.322 -> 0.286 ms; the binary and the weighted-channel kernels
// are faster with four and keep SCAT_WARPS.
#ifndef LMG_QS_WARPS
#define LMG_QS_WARPS 1
#endif
constexpr int QS_WARPS = LMG_QS_WARPS;
constexpr int BWD2_COLS = 256;  // compacted columns held per warp at a time
constexpr int ZSTEPS = 4;       // z positions per lane and chunk; a chunk covers 4*ZSTEPS voxels

template <int CAP_>
struct ColBufT {
  static constexpr unsigned CAP = CAP_;
  unsigned row[CAP_];  // x*dim + y
  float dxy2[CAP_];    // (gx-ax)^2 + (gy-ay)^2
};
template <int CAP_>
struct ColBufDT {
  static constexpr unsigned CAP = CAP_;
  unsigned row[CAP_];
  float dxy2[CAP_];
  float dx[CAP_];  // gx-ax
  float dy[CAP_];
};
typedef ColBufT<BWD2_COLS> ColBuf;
typedef ColBufDT<BWD2_COLS> ColBufD;

// Appends the columns of [cbase, ncols) whose squared distance in the xy plane is <= Tcull to the
// buffer until it is (nearly) full; returns how many it holds and advances cbase.
template <class BUF, bool WITH_D>
__device__ __forceinline__ unsigned compact_columns(BUF& buf, const ItemParams& P, unsigned& cbase,
                                                    unsigned ncols, unsigned ny, float inv_ny, float Tcull,
                                                    float ox, float oy, float res, unsigned dim, int lane) {
  unsigned nkept = 0;
  while (cbase < ncols && nkept + 32 <= BUF::CAP) {
    unsigned c = cbase + lane;
    bool keep = false;
    unsigned x = 0, y = 0;
    float dx = 0.f, dy = 0.f, dxy2 = 0.f;
    if (c < ncols) {
      // c / ny through a float reciprocal (exact for the footprint sizes that fit a grid)
      unsigned xi = ncols < (1u << 20) ? (unsigned)(((float)c + 0.5f) * inv_ny) : c / ny;
      unsigned yi = c - xi * ny;
      x = P.lox + xi;
      y = P.loy + yi;
      dx = __fsub_rn(voxel_coord(ox, x, res), P.x);
      dy = __fsub_rn(voxel_coord(oy, y, res), P.y);
      dxy2 = __fadd_rn(__fmul_rn(dx, dx), __fmul_rn(dy, dy));
      keep = dxy2 <= Tcull;
    }
    unsigned m = __ballot_sync(0xffffffffu, keep);
    if (keep) {
      unsigned slot = nkept + __popc(m & ((1u << lane) - 1u));
      buf.row[slot] = x * dim + y;
      buf.dxy2[slot] = dxy2;
      if constexpr (WITH_D) {
        buf.dx[slot] = dx;
        buf.dy[slot] = dy;
      }
    }
    nkept += __popc(m);
    cbase += 32;
  }
  return nkept;
}

// MODE 0: atom gradient (index types)          -> atom_gradients[b][a][3]
// MODE 1: atom + type gradient (vector types)  -> partial[b][a][t][3], type_gradients[b][a][t]
// MODE 2: relevance (index types)              -> relevance[b][a]
// MODE 3: backward_gradients' atom term        -> partial[b][a][t][3]  (src/grid_maker.cpp:636-662)
template <int MODE, bool BINARY>
__global__ void __launch_bounds__(BWD2_WARPS * 32) k_backward_warp(BwdArgs G) {
  constexpr bool VEC = MODE == 1 || MODE == 3;
  __shared__ ColBufD bufs[BWD2_WARPS];
  const GMParams& gm = G.gm;
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  int items_per_ex = VEC ? G.N * G.T : G.N;
  int item = blockIdx.x * BWD2_WARPS + wid;
  int bl = blockIdx.y;
  int b = G.b0 + bl;
  if (item >= items_per_ex) return;
  if (MODE == 3 || (MODE == 1 && G.type_gradients == nullptr)) {
    // an (atom, channel) pair without weight contributes nothing: leave before any other load
    int ea = item / G.T;
    if (G.type_vector[((size_t)b * G.N + ea) * G.T + (item - ea * G.T)] == 0.f) return;
  }
  ColBufD& buf = bufs[wid];

  float cx, cy, cz;
  if (G.centers != nullptr) {
    cx = G.centers[b * 3]; cy = G.centers[b * 3 + 1]; cz = G.centers[b * 3 + 2];
  } else {
    cx = G.center_host[0]; cy = G.center_host[1]; cz = G.center_host[2];
  }
  float ox = __fsub_rn(cx, gm.half), oy = __fsub_rn(cy, gm.half), oz = __fsub_rn(cz, gm.half);
  ItemParams P = load_item<VEC>(G, bl, b, item, ox, oy, oz);

  size_t dim = gm.dim;
  size_t chan_off = ((size_t)b * G.T + P.chan) * dim * dim * dim;
  const float* diff = G.diff + chan_off;
  const float* dens = MODE == 2 ? G.density + chan_off : nullptr;

  float agx = 0.f, agy = 0.f, agz = 0.f, tg = 0.f;
  bool want_ag = MODE == 0 || ((MODE == 1 || MODE == 3) && P.w != 0.f);
  float Tcull = (MODE == 0 || MODE == 3) ? P.Tcut : fmaxf(P.Tcut, BINARY ? P.Tbin : -1.f);
  float inx = 0.f, iny = 0.f, inz = 0.f, intg = 0.f;  // MODE 3: incoming gradients of this item
  if (MODE == 3) {
    size_t gi = (size_t)b * G.N + item / G.T;
    inx = G.ag_in[gi * 3]; iny = G.ag_in[gi * 3 + 1]; inz = G.ag_in[gi * 3 + 2];
    intg = G.tg_in[gi * G.T + P.chan];
    if (!want_ag) P.valid = false;  // zero-weight channels contribute nothing (src/grid_maker.cpp:573)
  }
  const float kexp = P.inv_ar2 * NEG2_LOG2E;
  const float k4 = 4.f * P.inv_ar2, kD = -gm.D * P.inv_ar2, kE = -gm.E * P.inv_ar;  // sign of -(s*dv) folded in

  if (P.valid) {
    unsigned nx = P.hix - P.lox, ny = P.hiy - P.loy;
    unsigned ncols = nx * ny;
    float inv_ny = 1.f / (float)ny;
    int grp = lane >> 2, sub = lane & 3;
    for (unsigned cbase = 0; cbase < ncols;) {
      unsigned nkept = compact_columns<ColBufD, true>(buf, P, cbase, ncols, ny, inv_ny, Tcull, ox, oy,
                                                      gm.res, gm.dim, lane);
      __syncwarp();
      for (unsigned zc = P.loz; zc < P.hiz; zc += 4 * ZSTEPS) {
        // this lane's z positions of the chunk; positions past the footprint get NaN, which fails
        // every comparison below
        unsigned z0 = zc + sub;
        float dzt[ZSTEPS], dz2t[ZSTEPS], ezt[ZSTEPS];
#pragma unroll
        for (int k = 0; k < ZSTEPS; k++) {
          unsigned zz = z0 + 4 * k;
          float dz = __fsub_rn(voxel_coord(oz, zz, gm.res), P.z);
          dzt[k] = dz;
          dz2t[k] = zz < P.hiz ? __fmul_rn(dz, dz) : CUDART_NAN_F;
          ezt[k] = ex2_approx(dz2t[k] * kexp);
        }
        for (unsigned i = grp; i < nkept; i += 8) {
          float dxy2 = buf.dxy2[i], dx = buf.dx[i], dy = buf.dy[i];
          size_t rowoff = (size_t)buf.row[i] * dim + z0;
          const float* row = diff + rowoff;
          float exy = ex2_approx(dxy2 * kexp);
          // the loads of the four z steps are issued together before any is used.  (Fetching one
          // column ahead was measured slower: the extra registers cost more occupancy than the
          // deeper queue of loads gains.)
          float rsqv[ZSTEPS], dvv[ZSTEPS];
          bool okv[ZSTEPS];
#pragma unroll
          for (int k = 0; k < ZSTEPS; k++) {
            rsqv[k] = __fadd_rn(dxy2, dz2t[k]);
            okv[k] = rsqv[k] <= Tcull;
            dvv[k] = okv[k] ? __ldg(row + 4 * k) : 0.f;
          }
          float fsum = 0.f;  // sum over the column of -(d density / d dist) / dist * dv
#pragma unroll
          for (int k = 0; k < ZSTEPS; k++) {
            if (!okv[k]) continue;
            float dz = dzt[k], rsq = rsqv[k], dv = dvv[k];
            float g = exy * ezt[k];  // exp(-2 rsq / ar^2)
            if (MODE == 3) {
              // second derivatives H_ab = alpha*delta_a*delta_b + [a==b]*beta of the density
              // (src/grid_maker.cu:812-878); delta = atom - grid point
              float alpha, beta;
              if (rsq <= P.Tg) {
                alpha = 16.f * g * P.inv_ar2 * P.inv_ar2;
                beta = -4.f * g * P.inv_ar2;
              } else {
                float id = rsqrt_approx(rsq);
                float S = fmaf(gm.D * P.inv_ar, rsq * id, gm.E);
                beta = S * id * P.inv_ar;
                alpha = fmaf(gm.D * P.inv_ar2, id * id, -beta * id * id);
              }
              float dot = fmaf(dx, inx, fmaf(dy, iny, dz * inz));
              float wa = P.w * alpha * dot;
              float wb = P.w * beta;
              float tt = alpha * intg;
              float bt = beta * intg;
              agx = fmaf(dv, fmaf(wa, dx, fmaf(wb, inx, fmaf(tt, dx * dx, bt))), agx);
              agy = fmaf(dv, fmaf(wa, dy, fmaf(wb, iny, fmaf(tt, dy * dy, bt))), agy);
              agz = fmaf(dv, fmaf(wa, dz, fmaf(wb, inz, fmaf(tt, dz * dz, bt))), agz);
            } else if (MODE != 2) {
              if (want_ag && rsq <= P.Tcut) {
                // -(d density / d dist) / dist * dv, src/grid_maker.cu:881-919; rsq == 0 contributes
                // nothing because dx = dy = dz = 0 there
                float s = rsq <= P.Tg ? k4 * g : fmaf(kE, rsqrt_approx(rsq), kD);
                float f = s * dv;
                fsum += f;
                agz = fmaf(f, dz, agz);
              }
            }
            if (MODE == 1 || MODE == 2) {
              float v;
              if (BINARY) {
                v = rsq < P.Tbin ? 1.f : 0.f;
              } else if (MODE == 2) {
                v = density_precise(rsq, P.ar, P.Tg, P.Tcut, gm.A, gm.B, gm.C);
              } else {
                float sq = sqrt_approx(rsq * P.inv_ar2);
                float q = fmaxf(fmaf(fmaf(gm.A, sq, gm.B), sq, gm.C), 0.f);
                v = rsq <= P.Tg ? g : q;
                v = rsq <= P.Tcut ? v : 0.f;
              }
              if (MODE == 1) {
                tg = fmaf(v, dv, tg);
              } else if (v > 0.f) {
                float de = __ldg(dens + rowoff + 4 * k);
                if (de > 0.f) tg += __fdiv_rn(__fmul_rn(dv, v), de);
              }
            }
          }  // k
          if (MODE == 0 || MODE == 1) {
            agx = fmaf(fsum, dx, agx);
            agy = fmaf(fsum, dy, agy);
          }
        }
      }
      __syncwarp();
    }
  }
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) {
    if (MODE != 2) {
      agx += __shfl_xor_sync(0xffffffffu, agx, o);
      agy += __shfl_xor_sync(0xffffffffu, agy, o);
      agz += __shfl_xor_sync(0xffffffffu, agz, o);
    }
    if (MODE == 1 || MODE == 2) tg += __shfl_xor_sync(0xffffffffu, tg, o);
  }
  if (lane == 0) {
    size_t ai = (size_t)b * G.N + (VEC ? item / G.T : item);
    if (MODE == 0) {
      G.atom_gradients[ai * 3] = agx;
      G.atom_gradients[ai * 3 + 1] = agy;
      G.atom_gradients[ai * 3 + 2] = agz;
    } else if (MODE == 1 || MODE == 3) {
      size_t pi = (size_t)bl * G.N * G.T + item;
      G.partial[pi * 3] = agx;
      G.partial[pi * 3 + 1] = agy;
      G.partial[pi * 3 + 2] = agz;
      if (MODE == 1 && G.type_gradients != nullptr) G.type_gradients[ai * G.T + P.chan] = tg;
    } else {
      G.relevance[ai] = tg;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// forward by scatter: the grid is zero-filled first, then one warp per atom (or per (atom, channel)
// pair with vector types) sweeps the atom's footprint exactly as the backward kernel does and adds
// its density into the grid with fire-and-forget reductions (red.global.add.f32), which resolve in
// L2.  No lists, no per-region work: the cost is proportional to the atoms' footprints.  Binary
// occupancy with index types needs no reduction at all (every writer stores the same 1.0).
// ---------------------------------------------------------------------------------------------
template <bool BINARY, bool PRECISE, bool VEC>
__global__ void __launch_bounds__(SCAT_WARPS * 32) k_forward_scatter(BwdArgs G) {
  __shared__ ColBuf bufs[SCAT_WARPS];
  const GMParams& gm = G.gm;
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  int items_per_ex = VEC ? G.N * G.T : G.N;
  int item = blockIdx.x * SCAT_WARPS + wid;
  int bl = blockIdx.y;
  int b = G.b0 + bl;
  if (item >= items_per_ex) return;
  if (VEC) {
    // an (atom, channel) pair without weight contributes nothing: leave before any other load
    int ea = item / G.T;
    if (G.type_vector[((size_t)b * G.N + ea) * G.T + (item - ea * G.T)] == 0.f) return;
  }
  ColBuf& buf = bufs[wid];

  float cx, cy, cz;
  if (G.centers != nullptr) {
    cx = G.centers[b * 3]; cy = G.centers[b * 3 + 1]; cz = G.centers[b * 3 + 2];
  } else {
    cx = G.center_host[0]; cy = G.center_host[1]; cz = G.center_host[2];
  }
  float ox = __fsub_rn(cx, gm.half), oy = __fsub_rn(cy, gm.half), oz = __fsub_rn(cz, gm.half);
  ItemParams P = load_item<VEC>(G, bl, b, item, ox, oy, oz);
  if (!P.valid || (VEC && P.w == 0.f)) return;  // zero weights add nothing (src/grid_maker.cpp:229)

  size_t dim = gm.dim;
  float* out = G.out_grid + ((size_t)b * G.T + P.chan) * dim * dim * dim;
  const float Tcull = BINARY ? P.Tbin : P.Tcut;
  const float kexp = P.inv_ar2 * NEG2_LOG2E;

  unsigned nx = P.hix - P.lox, ny = P.hiy - P.loy;
  unsigned ncols = nx * ny;
  float inv_ny = 1.f / (float)ny;
  int grp = lane >> 2, sub = lane & 3;
  for (unsigned cbase = 0; cbase < ncols;) {
    unsigned nkept = compact_columns<ColBuf, false>(buf, P, cbase, ncols, ny, inv_ny, Tcull, ox, oy,
                                                    gm.res, gm.dim, lane);
    __syncwarp();
    for (unsigned zc = P.loz; zc < P.hiz; zc += 4 * ZSTEPS) {
      unsigned z0 = zc + sub;
      float dz2t[ZSTEPS], ezt[ZSTEPS];
#pragma unroll
      for (int k = 0; k < ZSTEPS; k++) {
        unsigned zz = z0 + 4 * k;
        float dz = __fsub_rn(voxel_coord(oz, zz, gm.res), P.z);
        dz2t[k] = zz < P.hiz ? __fmul_rn(dz, dz) : CUDART_NAN_F;
        ezt[k] = (BINARY || PRECISE) ? 0.f : ex2_approx(dz2t[k] * kexp);
      }
      for (unsigned i = grp; i < nkept; i += 8) {
        float dxy2 = buf.dxy2[i];
        float* row = out + (size_t)buf.row[i] * dim + z0;
        float exy = (BINARY || PRECISE) ? 0.f : ex2_approx(dxy2 * kexp);
#pragma unroll
        for (int k = 0; k < ZSTEPS; k++) {
          float rsq = __fadd_rn(dxy2, dz2t[k]);
          if (BINARY) {
            if (rsq < P.Tbin) {
              if (VEC) atomicAdd(row + 4 * k, P.w);
              else row[4 * k] = 1.f;
            }
          } else {
            if (!(rsq <= P.Tcut)) continue;
            float v;
            if (PRECISE) {
              v = density_precise(rsq, P.ar, P.Tg, P.Tcut, gm.A, gm.B, gm.C);
            } else {
              float sq = sqrt_approx(rsq * P.inv_ar2);
              float q = fmaxf(fmaf(fmaf(gm.A, sq, gm.B), sq, gm.C), 0.f);
              v = rsq <= P.Tg ? exy * ezt[k] : q;
            }
            if (VEC) v *= P.w;
            if (v != 0.f) atomicAdd(row + 4 * k, v);
          }
        }
      }
    }
    __syncwarp();
  }
}

// Grid term of backward_gradients by scatter (src/grid_maker.cpp:618-634): per (atom, channel) with
// non-zero weight, every voxel within the cut-off receives
//   density * type_gradient  -  w * ((d density/d dist)/dist) * (delta . atom_gradient),
// delta = grid point - atom.  The output is zero-filled before the launch.
__global__ void __launch_bounds__(SCAT_WARPS * 32) k_gradgrad_scatter(BwdArgs G) {
  __shared__ ColBufD bufs[SCAT_WARPS];
  const GMParams& gm = G.gm;
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  int item = blockIdx.x * SCAT_WARPS + wid;
  int bl = blockIdx.y;
  int b = G.b0 + bl;
  if (item >= G.N * G.T) return;
  if (true) {
    // an (atom, channel) pair without weight contributes nothing: leave before any other load
    int ea = item / G.T;
    if (G.type_vector[((size_t)b * G.N + ea) * G.T + (item - ea * G.T)] == 0.f) return;
  }
  ColBufD& buf = bufs[wid];

  float cx, cy, cz;
  if (G.centers != nullptr) {
    cx = G.centers[b * 3]; cy = G.centers[b * 3 + 1]; cz = G.centers[b * 3 + 2];
  } else {
    cx = G.center_host[0]; cy = G.center_host[1]; cz = G.center_host[2];
  }
  float ox = __fsub_rn(cx, gm.half), oy = __fsub_rn(cy, gm.half), oz = __fsub_rn(cz, gm.half);
  ItemParams P = load_item<true>(G, bl, b, item, ox, oy, oz);
  if (!P.valid || P.w == 0.f) return;

  size_t dim = gm.dim;
  float* out = G.out_grid + ((size_t)b * G.T + P.chan) * dim * dim * dim;
  size_t gi = (size_t)b * G.N + item / G.T;
  const float inx = G.ag_in[gi * 3], iny = G.ag_in[gi * 3 + 1], inz = G.ag_in[gi * 3 + 2];
  const float intg = G.tg_in[gi * G.T + P.chan];
  const float kexp = P.inv_ar2 * NEG2_LOG2E;
  // -w * (d density/d dist)/dist: Gaussian 4 w g / ar^2; tail -w (D/ar^2 + E/(ar dist))
  const float k4 = 4.f * P.inv_ar2 * P.w, kD = -gm.D * P.inv_ar2 * P.w, kE = -gm.E * P.inv_ar * P.w;

  unsigned nx = P.hix - P.lox, ny = P.hiy - P.loy;
  unsigned ncols = nx * ny;
  float inv_ny = 1.f / (float)ny;
  int grp = lane >> 2, sub = lane & 3;
  for (unsigned cbase = 0; cbase < ncols;) {
    unsigned nkept = compact_columns<ColBufD, true>(buf, P, cbase, ncols, ny, inv_ny, P.Tcut, ox, oy,
                                                    gm.res, gm.dim, lane);
    __syncwarp();
    for (unsigned zc = P.loz; zc < P.hiz; zc += 4 * ZSTEPS) {
      unsigned z0 = zc + sub;
      float dzt[ZSTEPS], dz2t[ZSTEPS], ezt[ZSTEPS];
#pragma unroll
      for (int k = 0; k < ZSTEPS; k++) {
        unsigned zz = z0 + 4 * k;
        float dz = __fsub_rn(voxel_coord(oz, zz, gm.res), P.z);
        dzt[k] = dz * inz;
        dz2t[k] = zz < P.hiz ? __fmul_rn(dz, dz) : CUDART_NAN_F;
        ezt[k] = ex2_approx(dz2t[k] * kexp);
      }
      for (unsigned i = grp; i < nkept; i += 8) {
        float dxy2 = buf.dxy2[i];
        float dotxy = fmaf(buf.dx[i], inx, buf.dy[i] * iny);
        float* row = out + (size_t)buf.row[i] * dim + z0;
        float exy = ex2_approx(dxy2 * kexp);
#pragma unroll
        for (int k = 0; k < ZSTEPS; k++) {
          float rsq = __fadd_rn(dxy2, dz2t[k]);
          if (!(rsq <= P.Tcut)) continue;
          float g = exy * ezt[k];
          float sq = sqrt_approx(rsq * P.inv_ar2);
          float q = fmaxf(fmaf(fmaf(gm.A, sq, gm.B), sq, gm.C), 0.f);
          bool gauss = rsq <= P.Tg;
          float val = gauss ? g : q;
          float s = gauss ? k4 * g : fmaf(kE, rsqrt_approx(rsq), kD);
          float dot = rsq > 0.f ? dotxy + dzt[k] : 0.f;
          float gval = fmaf(val, intg, s * dot);
          if (gval != 0.f) atomicAdd(row + 4 * k, gval);
        }
      }
    }
    __syncwarp();
  }
}

// ---------------------------------------------------------------------------------------------
// Quad kernels: the same work items, for grids whose rows are 16-byte aligned (dim % 4 == 0 and an
// aligned base).  Here a lane owns a whole column (x,y) and walks it in aligned quads of four z
// voxels: the forward adds a quad with one red.global.add.v4.f32, the backward reads it with one
// 16-byte load, so a warp has 32 columns x 4 quads in flight per round trip to memory instead of
// 8 columns x 4 voxels.  What depends on z alone sits in a small shared table per warp (one pass
// covers 32 z positions from the aligned start of the footprint).  This lane-per-column layout
// serves the backward passes and the per-atom vector kernels, which spend their time issuing
// instructions and amortise the per-column terms over the quads of a column; the forward pass of
// index types and of (atom, channel) items is bound by the lines its reductions touch and uses
// the (column, z-quad) layout of qlane_sweep instead.
// ---------------------------------------------------------------------------------------------
constexpr int QPASS = 8;  // quads per pass

struct __align__(16) ZTabs {
  float4 dz2[QPASS];  // (gz-az)^2, NaN outside [loz, hiz)
  float4 ez[QPASS];   // exp(-2 dz2 / ar^2)
  float4 dz[QPASS];   // gz-az
  float lo[QPASS];    // smallest dz2 of the quad (NaN when no z of it lies in the footprint)
};

__device__ __forceinline__ void fill_ztabs(ZTabs& zt, unsigned zc, const ItemParams& P, float oz, float res,
                                           float kexp, int lane) {
  unsigned zz = zc + lane;
  float dz = __fsub_rn(voxel_coord(oz, zz, res), P.z);
  bool in = zz >= P.loz && zz < P.hiz;
  float d2 = in ? __fmul_rn(dz, dz) : CUDART_NAN_F;
  reinterpret_cast<float*>(zt.dz2)[lane] = d2;
  reinterpret_cast<float*>(zt.ez)[lane] = ex2_approx(d2 * kexp);
  reinterpret_cast<float*>(zt.dz)[lane] = dz;
  float lo = fminf(d2, __shfl_xor_sync(0xffffffffu, d2, 1));  // fminf skips the NaN entries
  lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, 2));
  if ((lane & 3) == 0) zt.lo[lane >> 2] = lo;
}

__device__ __forceinline__ void red_add_v4(float* p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}

// Sweep over the compacted columns of a footprint with the lanes laid out as (column, z-quad): ZQ
// lanes along z hold one aligned quad each, 32/ZQ columns per step (ZQ need not divide 32: with 3, 5
// or 6 quads two lanes idle, which costs less than a quad lane without voxels for every column).  A lane's z terms live in
// registers for the whole item, and the lanes of a column touch neighbouring 16-byte pieces of one
// line, so a warp's reduction reaches 32/ZQ rows instead of 32 (the scatter kernels are bound by the
// number of distinct lines their reductions touch).  `quad(i, dxy2, exy, d2v, ev, dzv, off)` is called
// by every lane whose quad can hold a voxel of the item: i = column slot, off = row*dim + z of the quad.
template <int ZQ, bool SCALED, class BUF, class QuadFn>
__device__ __forceinline__ void qlane_sweep(const ItemParams& P, const BUF& buf, unsigned nkept, size_t dim,
                                            float oz, float res, float kexp, float Tcull, float scale, int lane,
                                            QuadFn quad) {
  constexpr int CPI = 32 / ZQ;
  const int zq = lane % ZQ, cl = lane / ZQ;
  for (unsigned zc = P.loz & ~3u; zc < P.hiz; zc += 4 * ZQ) {
    float d2v[4], ev[4], dzv[4];
    float lo = CUDART_INF_F;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      unsigned zz = zc + 4 * zq + j;
      dzv[j] = __fsub_rn(voxel_coord(oz, zz, res), P.z);
      bool in = zz >= P.loz && zz < P.hiz;
      d2v[j] = in ? __fmul_rn(dzv[j], dzv[j]) : CUDART_NAN_F;
      if (SCALED) d2v[j] *= scale;
      ev[j] = ex2_approx(d2v[j] * kexp);
      lo = fminf(lo, d2v[j]);  // fminf skips the NaN entries
    }
    const size_t zoff = zc + 4 * zq;
    for (unsigned c0 = 0; c0 < nkept; c0 += CPI) {
      unsigned i = c0 + cl;
      float dxy2 = (cl < CPI && i < nkept) ? buf.dxy2[i] : CUDART_NAN_F;
      if (SCALED) dxy2 *= scale;
      if (!(__fadd_rn(dxy2, lo) <= Tcull)) continue;  // also false for NaN: no column, or no z in range
      quad(i, dxy2, ex2_approx(dxy2 * kexp), d2v, ev, dzv, (size_t)buf.row[i] * dim + zoff);
    }
  }
}

// The sweep with as many lanes along z as the footprint spans aligned quads.  Measured: dense type
// vectors at 96^3 (spans of 6) 2.16 -> 1.97 ms per 4 examples; the index-typed benchmark (spans of
// 3 to 5) unchanged at 0.259 ms per 50.
// SCALED: squared distances are handed to `quad` (and compared with Tcull) in units of the squared
// atom radius, `scale` = 1 / ar^2 and `kexp` = -2 log2(e): one multiplication per column instead of
// one per voxel for callers that want rsq / ar^2 (density only: the binary test keeps rsq itself).
template <bool SCALED, class BUF, class QuadFn>
__device__ __forceinline__ void qlane_sweep_span_t(unsigned span, const ItemParams& P, const BUF& buf, unsigned nkept,
                                                   size_t dim, float oz, float res, float kexp, float Tcull,
                                                   float scale, int lane, QuadFn quad) {
  if (span <= 2) qlane_sweep<2, SCALED>(P, buf, nkept, dim, oz, res, kexp, Tcull, scale, lane, quad);
  else if (span == 3) qlane_sweep<3, SCALED>(P, buf, nkept, dim, oz, res, kexp, Tcull, scale, lane, quad);
  else if (span == 4) qlane_sweep<4, SCALED>(P, buf, nkept, dim, oz, res, kexp, Tcull, scale, lane, quad);
  else if (span == 5) qlane_sweep<5, SCALED>(P, buf, nkept, dim, oz, res, kexp, Tcull, scale, lane, quad);
  else if (span == 6) qlane_sweep<6, SCALED>(P, buf, nkept, dim, oz, res, kexp, Tcull, scale, lane, quad);
  else qlane_sweep<8, SCALED>(P, buf, nkept, dim, oz, res, kexp, Tcull, scale, lane, quad);
}
template <class BUF, class QuadFn>
__device__ __forceinline__ void qlane_sweep_span(unsigned span, const ItemParams& P, const BUF& buf, unsigned nkept,
                                                 size_t dim, float oz, float res, float kexp, float Tcull, int lane,
                                                 QuadFn quad) {
  qlane_sweep_span_t<false>(span, P, buf, nkept, dim, oz, res, kexp, Tcull, 1.f, lane, quad);
}

// number of aligned quads between the first and the last z of a footprint
__device__ __forceinline__ unsigned quad_span(const ItemParams& P) { return (P.hiz - (P.loz & ~3u) + 3) >> 2; }

// One work item (an atom, or an (atom, channel) pair with VEC) of the forward pass on aligned quads.
template <bool VEC>
__device__ __forceinline__ void forward_quads_item(const BwdArgs& G, int item, int bl, ColBuf& buf, int lane) {
  const GMParams& gm = G.gm;
  int b = G.b0 + bl;
  if (VEC) {
    // an (atom, channel) pair without weight contributes nothing: leave before any other load
    int ea = item / G.T;
    if (G.type_vector[((size_t)b * G.N + ea) * G.T + (item - ea * G.T)] == 0.f) return;
  }

  float cx, cy, cz;
  if (G.centers != nullptr) {
    cx = G.centers[b * 3]; cy = G.centers[b * 3 + 1]; cz = G.centers[b * 3 + 2];
  } else {
    cx = G.center_host[0]; cy = G.center_host[1]; cz = G.center_host[2];
  }
  float ox = __fsub_rn(cx, gm.half), oy = __fsub_rn(cy, gm.half), oz = __fsub_rn(cz, gm.half);
  ItemParams P = load_item<VEC>(G, bl, b, item, ox, oy, oz);
  if (!P.valid || (VEC && P.w == 0.f)) return;  // zero weights add nothing (src/grid_maker.cpp:229)

  size_t dim = gm.dim;
  float* out = G.out_grid + ((size_t)b * G.T + P.chan) * dim * dim * dim;
  const float kexp = P.inv_ar2 * NEG2_LOG2E;
  const float ta = gm.ta, ntb = -gm.tb;

  unsigned nx = P.hix - P.lox, ny = P.hiy - P.loy;
  unsigned ncols = nx * ny;
  float inv_ny = 1.f / (float)ny;
  for (unsigned cbase = 0; cbase < ncols;) {
    unsigned nkept = compact_columns<ColBuf, false>(buf, P, cbase, ncols, ny, inv_ny, P.Tcut, ox, oy,
                                                    gm.res, gm.dim, lane);
    __syncwarp();
    // With a tail the density is continuous in the distance, and the squared distances may be taken
    // in units of ar^2 (s = rsq / ar^2: one multiplication per column and z position instead of one per
    // voxel; the Gaussian part ends at s = G^2, the tail clamps to zero at the cut-off).  Without a
    // tail (negative gaussian_radius_multiple) the density jumps at the cut-off, and the comparison
    // stays the reference's own, rsq against the threshold.
    const bool tail = ta != 0.f || ntb != 0.f;
    if (tail) {
      const float sg = P.Tg * P.inv_ar2, scut = P.Tcut * P.inv_ar2;
      auto quad = [&](unsigned, float dxy2, float exy, const float (&d2v)[4], const float (&ev)[4],
                      const float (&)[4], size_t off) {
        float v[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
          float sq = dxy2 + d2v[j];
          float tq = fminf(fmaf(ta, sqrt_approx(sq), ntb), 0.f);  // a NaN gives zero too
          float val = sq <= sg ? exy * ev[j] : tq * tq;
          v[j] = VEC ? val * P.w : val;
        }
        red_add_v4(out + off, v[0], v[1], v[2], v[3]);
      };
      qlane_sweep_span_t<true>(quad_span(P), P, buf, nkept, dim, oz, gm.res, NEG2_LOG2E, scut, P.inv_ar2, lane, quad);
    } else {
      auto quad = [&](unsigned, float dxy2, float exy, const float (&d2v)[4], const float (&ev)[4],
                      const float (&)[4], size_t off) {
        float v[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
          float rsq = __fadd_rn(dxy2, d2v[j]);
          // tail (ta*dr - tb)^2 clamped to zero beyond the cut-off; a NaN rsq gives zero too
          float tq = fminf(fmaf(ta, sqrt_approx(rsq * P.inv_ar2), ntb), 0.f);
          float val = rsq <= P.Tg ? exy * ev[j] : tq * tq;
          v[j] = VEC ? val * P.w : val;
        }
        red_add_v4(out + off, v[0], v[1], v[2], v[3]);
      };
      qlane_sweep_span(quad_span(P), P, buf, nkept, dim, oz, gm.res, kexp, P.Tcut, lane, quad);
    }
    __syncwarp();
  }
}

template <bool VEC>
__global__ void __launch_bounds__(QS_WARPS * 32) k_forward_quads(BwdArgs G) {
  __shared__ ColBuf bufs[QS_WARPS];
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  int item = blockIdx.x * QS_WARPS + wid;
  if (item >= (VEC ? G.N * G.T : G.N)) return;
  forward_quads_item<VEC>(G, item, blockIdx.y, bufs[wid], lane);
}

// Vector types whose radii differ by channel: one warp takes a group of NZ_GROUP consecutive channels
// of an atom and runs the (atom, channel) item of every channel of the group in which the atom
// carries weight - no work item, and no block, per channel without weight (27 of 28 with one-hot
// types), and still several warps per atom when every channel is weighted.
constexpr int NZ_GROUP = 8;
__host__ __device__ inline int nz_groups(int T) { return (T + NZ_GROUP - 1) / NZ_GROUP; }

#define LMG_FOR_EACH_WEIGHTED_CHANNEL(G, b, unit, lane, atom, t)                                        \
  if (int atom = (unit) % (G).N; true)                                                                  \
    if (int t0_ = ((unit) / (G).N) * NZ_GROUP; true)                                                    \
      for (unsigned m_ = __ballot_sync(                                                                 \
               0xffffffffu, (lane) < NZ_GROUP && t0_ + (lane) < (G).T &&                                \
                                (G).type_vector[((size_t)(b) * (G).N + atom) * (G).T + t0_ + (lane)] != 0.f); \
           m_ != 0u; m_ &= m_ - 1u)                                                                     \
        if (int t = t0_ + __ffs(m_) - 1; true)

__global__ void __launch_bounds__(SCAT_WARPS * 32) k_forward_quads_nz(BwdArgs G) {
  __shared__ ColBuf bufs[SCAT_WARPS];
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  int unit = blockIdx.x * SCAT_WARPS + wid;
  if (unit >= G.N * nz_groups(G.T)) return;
  int b = G.b0 + blockIdx.y;
  LMG_FOR_EACH_WEIGHTED_CHANNEL(G, b, unit, lane, atom, t) {
    forward_quads_item<true>(G, atom * G.T + t, blockIdx.y, bufs[wid], lane);
    __syncwarp();
  }
}

// The backward passes (modes as in k_backward_warp) on aligned quads.
struct BwdSums {
  float agx, agy, agz, tg;  // reduced over the warp: every lane holds the totals
};

// The sweep of one work item whose constants are in P: sums over the item's footprint, reduced
// over the warp.  `item` and `b` only serve MODE 3 (its incoming gradients).
template <int MODE, bool BINARY, class BUF>
__device__ __forceinline__ BwdSums backward_quads_core(const BwdArgs& G, ItemParams& P, int b, int item,
                                                       float ox, float oy, float oz, BUF& buf, ZTabs& zt,
                                                       int lane) {
  const GMParams& gm = G.gm;
  size_t dim = gm.dim;
  size_t chan_off = ((size_t)b * G.T + P.chan) * dim * dim * dim;
  const float* diff = G.diff + chan_off;
  const float* dens = MODE == 2 ? G.density + chan_off : nullptr;
  float agx = 0.f, agy = 0.f, agz = 0.f, tg = 0.f;
  bool want_ag = MODE == 0 || ((MODE == 1 || MODE == 3) && P.w != 0.f);
  const float Tcull = (MODE == 0 || MODE == 3) ? P.Tcut : fmaxf(P.Tcut, BINARY ? P.Tbin : -1.f);
  float inx = 0.f, iny = 0.f, inz = 0.f, intg = 0.f;  // MODE 3: incoming gradients of this item
  if (MODE == 3) {
    size_t gi = (size_t)b * G.N + item / G.T;
    inx = G.ag_in[gi * 3]; iny = G.ag_in[gi * 3 + 1]; inz = G.ag_in[gi * 3 + 2];
    intg = G.tg_in[gi * G.T + P.chan];
    if (!want_ag) P.valid = false;  // zero-weight channels contribute nothing (src/grid_maker.cpp:573)
  }
  const float kexp = P.inv_ar2 * NEG2_LOG2E;
  // The gradient's radial factor beyond the Gaussian part is kE/d + kD: positive inside the cut-off,
  // zero at it (the tail polynomial has a double root there) and negative beyond, so a clamp at zero
  // stands in for the comparison with the cut-off.  Items that want no atom gradient (zero weight)
  // and grid makers without a tail (ta == tb == 0) get zero factors.
  const bool tail = gm.ta != 0.f || gm.tb != 0.f;
  const float k4 = want_ag ? 4.f * P.inv_ar2 : 0.f;
  const float kD = (want_ag && tail) ? -gm.D * P.inv_ar2 : 0.f, kE = (want_ag && tail) ? -gm.E * P.inv_ar : 0.f;
  const float ta = gm.ta, ntb = -gm.tb;
  const float g16 = 16.f * P.inv_ar2 * P.inv_ar2, gm4 = -4.f * P.inv_ar2;  // MODE 3, Gaussian part
  float sb = 0.f;                                                            // MODE 3: sum of diff*beta

  if (P.valid) {
    unsigned nx = P.hix - P.lox, ny = P.hiy - P.loy;
    unsigned ncols = nx * ny;
    float inv_ny = 1.f / (float)ny;
    for (unsigned cbase = 0; cbase < ncols;) {
      unsigned nkept = compact_columns<BUF, true>(buf, P, cbase, ncols, ny, inv_ny, Tcull, ox, oy,
                                                  gm.res, gm.dim, lane);
      for (unsigned zc = P.loz & ~3u; zc < P.hiz; zc += 4 * QPASS) {
        __syncwarp();
        fill_ztabs(zt, zc, P, oz, gm.res, kexp, lane);
        __syncwarp();
        unsigned nq = min((unsigned)QPASS, (P.hiz - zc + 3) >> 2);
        for (unsigned c0 = 0; c0 < nkept; c0 += 32) {
          unsigned i = c0 + lane;
          bool have = i < nkept;
          float dxy2 = have ? buf.dxy2[i] : CUDART_NAN_F;
          float dx = have ? buf.dx[i] : 0.f, dy = have ? buf.dy[i] : 0.f;
          size_t rowoff = (size_t)(have ? buf.row[i] : 0u) * dim + zc;
          const float4* row = reinterpret_cast<const float4*>(diff + rowoff);
          float exy = ex2_approx(dxy2 * kexp);
          float exy4 = k4 * exy;
          float fsum = 0.f;
          float dotxy = MODE == 3 ? fmaf(dx, inx, dy * iny) : 0.f;
          float a0 = 0.f, a1 = 0.f, a2 = 0.f;  // MODE 3: sums over the column of diff*alpha*{1, dz, dz^2}
          for (unsigned q0 = 0; q0 < nq; q0 += 4) {
            // up to four quads of the column are requested together, then used
            float4 dv[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
              dv[u] = make_float4(0.f, 0.f, 0.f, 0.f);
              // no load where no voxel of the quad can lie inside the cut-off (false for a NaN too)
              if (q0 + u < nq && __fadd_rn(dxy2, zt.lo[q0 + u]) <= Tcull) dv[u] = __ldg(row + q0 + u);
            }
#pragma unroll
            for (int u = 0; u < 4; u++) {
              if (q0 + u < nq) {
                float4 d2 = zt.dz2[q0 + u], e = zt.ez[q0 + u], dz = zt.dz[q0 + u];
                float d2v[4] = {d2.x, d2.y, d2.z, d2.w}, ev[4] = {e.x, e.y, e.z, e.w};
                float dzv[4] = {dz.x, dz.y, dz.z, dz.w}, dvv[4] = {dv[u].x, dv[u].y, dv[u].z, dv[u].w};
                float dev[4] = {0.f, 0.f, 0.f, 0.f};
                if (MODE == 2) {
                  // the density is only needed where this quad can hold a voxel of the atom
                  if (__fadd_rn(dxy2, zt.lo[q0 + u]) <= Tcull) {
                    float4 de = __ldg(reinterpret_cast<const float4*>(dens + rowoff) + q0 + u);
                    dev[0] = de.x; dev[1] = de.y; dev[2] = de.z; dev[3] = de.w;
                  }
                }
#pragma unroll
                for (int j = 0; j < 4; j++) {
                  float rsq = __fadd_rn(dxy2, d2v[j]);
                  float g = exy * ev[j];  // exp(-2 rsq / ar^2)
                  if (MODE == 0 || MODE == 1) {
                    // -(d density / d dist) / dist * dv, src/grid_maker.cu:881-919; rsq == 0
                    // contributes nothing because dx = dy = dz = 0 there
                    // a NaN rsq (z outside the footprint) takes the second branch and clamps to zero
                    float sg = rsq <= P.Tg ? exy4 * ev[j] : fmaxf(fmaf(kE, rsqrt_approx(rsq), kD), 0.f);
                    float f = sg * dvv[j];
                    fsum += f;
                    agz = fmaf(f, dzv[j], agz);
                  }
                  if (MODE == 1) {
                    float v;
                    if (BINARY) {
                      v = rsq < P.Tbin ? 1.f : 0.f;
                    } else {
                      float tq = fminf(fmaf(ta, sqrt_approx(rsq * P.inv_ar2), ntb), 0.f);
                      v = rsq <= P.Tg ? g : tq * tq;  // tq is zero beyond the cut-off and for a NaN rsq
                    }
                    tg = fmaf(v, dvv[j], tg);
                  }
                  if (MODE == 2) {
                    float v = BINARY ? (rsq < P.Tbin ? 1.f : 0.f)
                                     : density_precise(rsq, P.ar, P.Tg, P.Tcut, gm.A, gm.B, gm.C);
                    if (v > 0.f && dev[j] > 0.f) tg += __fdiv_rn(__fmul_rn(dvv[j], v), dev[j]);
                  }
                  if (MODE == 3) {
                    // second derivatives H_ab = alpha*delta_a*delta_b + [a==b]*beta of the density
                    // (src/grid_maker.cu:812-878); delta = atom - grid point.  Per voxel only the
                    // moments of diff*alpha in dz and the sum of diff*beta are taken; what is the same
                    // for a whole column (dx, dy, the incoming gradients) is applied after it.
                    float alpha, beta;
                    if (rsq <= P.Tg) {
                      alpha = g16 * g;
                      beta = gm4 * g;
                    } else {
                      float id = rsqrt_approx(rsq);
                      float S = fmaf(gm.D * P.inv_ar, rsq * id, gm.E);
                      beta = S * id * P.inv_ar;
                      alpha = fmaf(gm.D * P.inv_ar2, id * id, -beta * id * id);
                    }
                    // nothing beyond the cut-off, nor for a NaN rsq (z outside the footprint), whose
                    // alpha and beta are NaN as well: the products are selected, not multiplied by zero
                    const bool inside = rsq <= P.Tcut;
                    float t0 = inside ? dvv[j] * alpha : 0.f, tb = inside ? dvv[j] * beta : 0.f;
                    float t1 = t0 * dzv[j];
                    a0 += t0;
                    a1 += t1;
                    a2 = fmaf(t1, dzv[j], a2);
                    sb += tb;
                  }
                }
              }
            }
          }
          if (MODE == 0 || MODE == 1) {
            agx = fmaf(fsum, dx, agx);
            agy = fmaf(fsum, dy, agy);
          }
          if (MODE == 3) {
            // sum over the column of diff * (w*alpha*dot*delta_c + intg*alpha*delta_c^2), dot = dotxy + dz*inz
            float wd = P.w * fmaf(dotxy, a0, inz * a1);
            agx = fmaf(dx, fmaf(intg * dx, a0, wd), agx);
            agy = fmaf(dy, fmaf(intg * dy, a0, wd), agy);
            agz += fmaf(P.w, fmaf(dotxy, a1, inz * a2), intg * a2);
          }
        }
      }
      __syncwarp();
    }
  }
  if (MODE == 3) {
    // the isotropic part: diff*beta*(w*in_c + intg), the same factor for every voxel of the item
    agx = fmaf(sb, fmaf(P.w, inx, intg), agx);
    agy = fmaf(sb, fmaf(P.w, iny, intg), agy);
    agz = fmaf(sb, fmaf(P.w, inz, intg), agz);
  }
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) {
    if (MODE != 2) {
      agx += __shfl_xor_sync(0xffffffffu, agx, o);
      agy += __shfl_xor_sync(0xffffffffu, agy, o);
      agz += __shfl_xor_sync(0xffffffffu, agz, o);
    }
    if (MODE == 1 || MODE == 2) tg += __shfl_xor_sync(0xffffffffu, tg, o);
  }
  BwdSums R;
  R.agx = agx; R.agy = agy; R.agz = agz; R.tg = tg;
  return R;
}

// One work item (an atom, or an (atom, channel) pair for the vector modes) from its record in the
// workspace.
template <int MODE, bool BINARY>
__device__ __forceinline__ void backward_quads_item(const BwdArgs& G, int item, int bl, ColBufD& buf, ZTabs& zt,
                                                    int lane) {
  constexpr bool VEC = MODE == 1 || MODE == 3;
  const GMParams& gm = G.gm;
  int b = G.b0 + bl;
  if (MODE == 3 || (MODE == 1 && G.type_gradients == nullptr)) {
    // an (atom, channel) pair without weight contributes nothing: leave before any other load
    int ea = item / G.T;
    if (G.type_vector[((size_t)b * G.N + ea) * G.T + (item - ea * G.T)] == 0.f) return;
  }

  float cx, cy, cz;
  if (G.centers != nullptr) {
    cx = G.centers[b * 3]; cy = G.centers[b * 3 + 1]; cz = G.centers[b * 3 + 2];
  } else {
    cx = G.center_host[0]; cy = G.center_host[1]; cz = G.center_host[2];
  }
  float ox = __fsub_rn(cx, gm.half), oy = __fsub_rn(cy, gm.half), oz = __fsub_rn(cz, gm.half);
  ItemParams P = load_item<VEC>(G, bl, b, item, ox, oy, oz);
  BwdSums R = backward_quads_core<MODE, BINARY, ColBufD>(G, P, b, item, ox, oy, oz, buf, zt, lane);
  float agx = R.agx, agy = R.agy, agz = R.agz, tg = R.tg;
  if (lane == 0) {
    size_t ai = (size_t)b * G.N + (VEC ? item / G.T : item);
    if (MODE == 0) {
      G.atom_gradients[ai * 3] = agx;
      G.atom_gradients[ai * 3 + 1] = agy;
      G.atom_gradients[ai * 3 + 2] = agz;
    } else if (MODE == 1 || MODE == 3) {
      size_t pi = (size_t)bl * G.N * G.T + item;
      G.partial[pi * 3] = agx;
      G.partial[pi * 3 + 1] = agy;
      G.partial[pi * 3 + 2] = agz;
      if (MODE == 1 && G.type_gradients != nullptr) G.type_gradients[ai * G.T + P.chan] = tg;
    } else {
      G.relevance[ai] = tg;
    }
  }
}

template <int MODE, bool BINARY>
__global__ void __launch_bounds__(BWD2_WARPS * 32) k_backward_quads(BwdArgs G) {
  constexpr bool VEC = MODE == 1 || MODE == 3;
  __shared__ ColBufD bufs[BWD2_WARPS];
  __shared__ ZTabs ztabs[BWD2_WARPS];
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  int item = blockIdx.x * BWD2_WARPS + wid;
  if (item >= (VEC ? G.N * G.T : G.N)) return;
  backward_quads_item<MODE, BINARY>(G, item, blockIdx.y, bufs[wid], ztabs[wid], lane);
}

// The (atom, channel) items of the weighted channels of one atom, by one warp: modes that need
// nothing from channels without weight (MODE 1 when no type gradients are wanted, MODE 3).
template <int MODE, bool BINARY>
__global__ void __launch_bounds__(BWD2_WARPS * 32) k_backward_quads_nz(BwdArgs G) {
  __shared__ ColBufD bufs[BWD2_WARPS];
  __shared__ ZTabs ztabs[BWD2_WARPS];
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  int unit = blockIdx.x * BWD2_WARPS + wid;
  if (unit >= G.N * nz_groups(G.T)) return;
  int b = G.b0 + blockIdx.y;
  LMG_FOR_EACH_WEIGHTED_CHANNEL(G, b, unit, lane, atom, t) {
    backward_quads_item<MODE, BINARY>(G, atom * G.T + t, blockIdx.y, bufs[wid], ztabs[wid], lane);
    __syncwarp();
  }
}

// Grid term of backward_gradients on aligned quads (see k_gradgrad_scatter).
__device__ __forceinline__ void gradgrad_quads_item(const BwdArgs& G, int item, int bl, ColBufD& buf, ZTabs& zt,
                                                    int lane) {
  const GMParams& gm = G.gm;
  int b = G.b0 + bl;
  if (true) {
    // an (atom, channel) pair without weight contributes nothing: leave before any other load
    int ea = item / G.T;
    if (G.type_vector[((size_t)b * G.N + ea) * G.T + (item - ea * G.T)] == 0.f) return;
  }

  float cx, cy, cz;
  if (G.centers != nullptr) {
    cx = G.centers[b * 3]; cy = G.centers[b * 3 + 1]; cz = G.centers[b * 3 + 2];
  } else {
    cx = G.center_host[0]; cy = G.center_host[1]; cz = G.center_host[2];
  }
  float ox = __fsub_rn(cx, gm.half), oy = __fsub_rn(cy, gm.half), oz = __fsub_rn(cz, gm.half);
  ItemParams P = load_item<true>(G, bl, b, item, ox, oy, oz);
  if (!P.valid || P.w == 0.f) return;

  size_t dim = gm.dim;
  float* out = G.out_grid + ((size_t)b * G.T + P.chan) * dim * dim * dim;
  size_t gi = (size_t)b * G.N + item / G.T;
  const float inx = G.ag_in[gi * 3], iny = G.ag_in[gi * 3 + 1], inz = G.ag_in[gi * 3 + 2];
  const float intg = G.tg_in[gi * G.T + P.chan];
  const float kexp = P.inv_ar2 * NEG2_LOG2E;
  const float k4 = 4.f * P.inv_ar2 * P.w, kD = -gm.D * P.inv_ar2 * P.w, kE = -gm.E * P.inv_ar * P.w;
  const float ta = gm.ta, ntb = -gm.tb;

  unsigned nx = P.hix - P.lox, ny = P.hiy - P.loy;
  unsigned ncols = nx * ny;
  float inv_ny = 1.f / (float)ny;
  for (unsigned cbase = 0; cbase < ncols;) {
    unsigned nkept = compact_columns<ColBufD, true>(buf, P, cbase, ncols, ny, inv_ny, P.Tcut, ox, oy,
                                                    gm.res, gm.dim, lane);
    for (unsigned zc = P.loz & ~3u; zc < P.hiz; zc += 4 * QPASS) {
      __syncwarp();
      fill_ztabs(zt, zc, P, oz, gm.res, kexp, lane);
      __syncwarp();
      unsigned nq = min((unsigned)QPASS, (P.hiz - zc + 3) >> 2);
      for (unsigned c0 = 0; c0 < nkept; c0 += 32) {
        unsigned i = c0 + lane;
        bool have = i < nkept;
        float dxy2 = have ? buf.dxy2[i] : CUDART_NAN_F;
        float dotxy = have ? fmaf(buf.dx[i], inx, buf.dy[i] * iny) : 0.f;
        float* row = out + (size_t)(have ? buf.row[i] : 0u) * dim + zc;
        float exy = ex2_approx(dxy2 * kexp);
        for (unsigned q = 0; q < nq; q++) {
          float4 d2 = zt.dz2[q], e = zt.ez[q], dz = zt.dz[q];
          float d2v[4] = {d2.x, d2.y, d2.z, d2.w}, ev[4] = {e.x, e.y, e.z, e.w};
          float dzv[4] = {dz.x, dz.y, dz.z, dz.w}, v[4];
#pragma unroll
          for (int j = 0; j < 4; j++) {
            float rsq = __fadd_rn(dxy2, d2v[j]);
            float g = exy * ev[j];
            float tq = fminf(fmaf(ta, sqrt_approx(rsq * P.inv_ar2), ntb), 0.f);
            bool gauss = rsq <= P.Tg;
            float val = gauss ? g : tq * tq;
            float sg = gauss ? k4 * g : fmaf(kE, rsqrt_approx(rsq), kD);
            float dot = rsq > 0.f ? fmaf(dzv[j], inz, dotxy) : 0.f;
            float gval = fmaf(val, intg, sg * dot);
            v[j] = rsq <= P.Tcut ? gval : 0.f;
          }
          unsigned any = __float_as_uint(v[0]) | __float_as_uint(v[1]) | __float_as_uint(v[2]) |
                         __float_as_uint(v[3]);
          if (any != 0u) red_add_v4(row + 4 * q, v[0], v[1], v[2], v[3]);
        }
      }
    }
    __syncwarp();
  }
}

__global__ void __launch_bounds__(SCAT_WARPS * 32) k_gradgrad_quads_nz(BwdArgs G) {
  __shared__ ColBufD bufs[SCAT_WARPS];
  __shared__ ZTabs ztabs[SCAT_WARPS];
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  int unit = blockIdx.x * SCAT_WARPS + wid;
  if (unit >= G.N * nz_groups(G.T)) return;
  int b = G.b0 + blockIdx.y;
  LMG_FOR_EACH_WEIGHTED_CHANNEL(G, b, unit, lane, atom, t) {
    gradgrad_quads_item(G, atom * G.T + t, blockIdx.y, bufs[wid], ztabs[wid], lane);
    __syncwarp();
  }
}

// ---------------------------------------------------------------------------------------------
// Vector types with per-atom radii (the layout of the autograd bindings): the footprint and the
// density of an atom are the same for every channel, so one warp owns the ATOM, evaluates each voxel
// once and loops over the channels inside - the reuse the reference's kernel makes too
// (src/grid_maker.cu:322-325).  With one-hot type vectors this is the index-typed cost instead of
// one work item per (atom, channel).  Channels are handled in rounds of VA_CH.
// ---------------------------------------------------------------------------------------------
constexpr int VA_CH = 32;  // channels per round
constexpr int VA_SPARSE = 2;  // rounds with at most this many weighted channels sweep once per channel

template <bool BINARY, bool PRECISE>
__global__ void __launch_bounds__(QS_WARPS * 32) k_forward_quads_atom(BwdArgs G) {
  __shared__ ColBuf bufs[QS_WARPS];
  __shared__ ZTabs ztabs[QS_WARPS];
  __shared__ int nz_t[QS_WARPS][VA_CH];
  __shared__ float nz_w[QS_WARPS][VA_CH];
  const GMParams& gm = G.gm;
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  int item = blockIdx.x * QS_WARPS + wid;
  int bl = blockIdx.y;
  int b = G.b0 + bl;
  if (item >= G.N) return;
  ColBuf& buf = bufs[wid];
  ZTabs& zt = ztabs[wid];

  float cx, cy, cz;
  if (G.centers != nullptr) {
    cx = G.centers[b * 3]; cy = G.centers[b * 3 + 1]; cz = G.centers[b * 3 + 2];
  } else {
    cx = G.center_host[0]; cy = G.center_host[1]; cz = G.center_host[2];
  }
  float ox = __fsub_rn(cx, gm.half), oy = __fsub_rn(cy, gm.half), oz = __fsub_rn(cz, gm.half);
  ItemParams P = load_item<false>(G, bl, b, item, ox, oy, oz);
  if (!P.valid) return;

  size_t dim = gm.dim;
  const size_t chan_stride = dim * dim * dim;
  float* outb = G.out_grid + (size_t)b * G.T * chan_stride;
  const float* wrow = G.type_vector + ((size_t)b * G.N + item) * G.T;
  const float Tcull = BINARY ? P.Tbin : P.Tcut;
  const float kexp = P.inv_ar2 * NEG2_LOG2E;
  const float ta = gm.ta, ntb = -gm.tb;

  unsigned nx = P.hix - P.lox, ny = P.hiy - P.loy;
  unsigned ncols = nx * ny;
  float inv_ny = 1.f / (float)ny;
  for (int tb = 0; tb < G.T; tb += VA_CH) {
    // channels of this round that carry weight (zero weights add nothing, src/grid_maker.cpp:229)
    int t = tb + lane;
    float w = t < G.T ? wrow[t] : 0.f;
    unsigned m = __ballot_sync(0xffffffffu, w != 0.f);
    int nnz = __popc(m);
    if (nnz == 0) continue;
    __syncwarp();
    if (w != 0.f) {
      int slot = __popc(m & ((1u << lane) - 1u));
      nz_t[wid][slot] = t;
      nz_w[wid][slot] = w;
    }
    __syncwarp();
    for (unsigned cbase = 0; cbase < ncols;) {
      unsigned nkept = compact_columns<ColBuf, false>(buf, P, cbase, ncols, ny, inv_ny, Tcull, ox, oy,
                                                      gm.res, gm.dim, lane);
      if (!BINARY && !PRECISE && nnz <= VA_SPARSE) {
        // few weighted channels (one-hot types): one sweep per channel in the lane layout of the
        // index-typed forward, whose reductions touch a quarter of the rows
        __syncwarp();
        for (int k = 0; k < nnz; k++) {
          float* out = outb + (size_t)nz_t[wid][k] * chan_stride;
          const float wk = nz_w[wid][k];
          auto quad = [&](unsigned, float dxy2, float exy, const float (&d2v)[4], const float (&ev)[4],
                          const float (&)[4], size_t off) {
            float v[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
              float rsq = __fadd_rn(dxy2, d2v[j]);
              float tq = fminf(fmaf(ta, sqrt_approx(rsq * P.inv_ar2), ntb), 0.f);
              v[j] = (rsq <= P.Tg ? exy * ev[j] : tq * tq) * wk;
            }
            red_add_v4(out + off, v[0], v[1], v[2], v[3]);
          };
          qlane_sweep_span(quad_span(P), P, buf, nkept, dim, oz, gm.res, kexp, Tcull, lane, quad);
        }
        __syncwarp();
        continue;
      }
      for (unsigned zc = P.loz & ~3u; zc < P.hiz; zc += 4 * QPASS) {
        __syncwarp();
        fill_ztabs(zt, zc, P, oz, gm.res, kexp, lane);
        __syncwarp();
        unsigned nq = min((unsigned)QPASS, (P.hiz - zc + 3) >> 2);
        for (unsigned c0 = 0; c0 < nkept; c0 += 32) {
          unsigned i = c0 + lane;
          bool have = i < nkept;
          float dxy2 = have ? buf.dxy2[i] : CUDART_NAN_F;
          float* row = outb + (size_t)(have ? buf.row[i] : 0u) * dim + zc;
          float exy = ex2_approx(dxy2 * kexp);
          for (unsigned q = 0; q < nq; q++) {
            float4 d2 = zt.dz2[q], e = zt.ez[q];
            float d2v[4] = {d2.x, d2.y, d2.z, d2.w}, ev[4] = {e.x, e.y, e.z, e.w}, v[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
              float rsq = __fadd_rn(dxy2, d2v[j]);
              if (BINARY) {
                v[j] = rsq < P.Tbin ? 1.f : 0.f;
              } else if (PRECISE) {
                v[j] = density_precise(rsq, P.ar, P.Tg, P.Tcut, gm.A, gm.B, gm.C);
              } else {
                float tq = fminf(fmaf(ta, sqrt_approx(rsq * P.inv_ar2), ntb), 0.f);
                v[j] = rsq <= P.Tg ? exy * ev[j] : tq * tq;
              }
            }
            unsigned any = __float_as_uint(v[0]) | __float_as_uint(v[1]) | __float_as_uint(v[2]) |
                           __float_as_uint(v[3]);
            if (any != 0u) {
              for (int k = 0; k < nnz; k++) {
                float wk = nz_w[wid][k];
                red_add_v4(row + (size_t)nz_t[wid][k] * chan_stride + 4 * q, v[0] * wk, v[1] * wk, v[2] * wk,
                           v[3] * wk);
              }
            }
          }
        }
      }
      __syncwarp();
    }
  }
}

// Backward for the same layout: atom gradient = sum over voxels of s * delta * (sum_t w_t diff_t),
// type gradient of EVERY channel = sum over voxels of density * diff_t (src/grid_maker.cpp:508-517).
// A lane keeps the type gradients of a round's channels in registers; rounds of VA_BCH channels,
// the quads of VA_LD channels requested together.  The kernel waits on those loads (they come from
// L2: every channel is read under every footprint), so what counts is how many are in flight per SM:
// registers per warp against loads per warp.  Measured per batch of 50 (28 channels, one-hot types):
// rounds of 16 with 4 loads together 2.79 ms, 8 / 8 2.08 ms, 14 / 7 1.82 ms, 14 / 14 1.70 ms,
// 16 / 16 2.17 ms, 28 / 14 2.05 ms; capping the registers below what the compiler picks, blocks of
// several warps, or atoms sorted by cell (for L1 reuse between neighbours) change nothing or lose.
#ifndef LMG_VA_BCH
#define LMG_VA_BCH 14
#endif
constexpr int VA_BCH = LMG_VA_BCH;
#ifndef LMG_VA_LD
#define LMG_VA_LD 14
#endif
constexpr int VA_LD = LMG_VA_LD;  // channels whose quads are requested together
static_assert(VA_BCH % VA_LD == 0, "a round is a whole number of load batches");
static_assert(VA_BCH <= 32, "a lane per channel of a round reads the weights");
#ifndef LMG_VA_WARPS
#define LMG_VA_WARPS BWD2_WARPS
#endif
constexpr int VA_WARPS = LMG_VA_WARPS;
#ifndef LMG_VA_REREAD
#define LMG_VA_REREAD 2
#endif
constexpr int VA_REREAD = LMG_VA_REREAD;  // weighted channels of a round up to which they are re-read from a list

// per-warp shared state of the kernel below
struct VaShared {
  ColBufD buf;
  float w[VA_BCH];   // weights of the round's channels
  int nz_t[VA_BCH];  // the weighted ones: channel (relative to the round) and weight
  float nz_w[VA_BCH];
};

// One round of k_backward_quads_atom: channels [tb, tb + nch) under the whole footprint of the atom.
// Lanes as (column, z-quad): the lanes of a column read neighbouring 16-byte pieces of one line in
// every channel, a quarter of the lines a lane-per-column load touches.  The sum over weighted
// channels that the atom gradient needs is taken inside the channel loop when many channels of the
// round carry weight (DENSE), and from a re-read of the few that do otherwise (one-hot types: one
// extra load per quad in one round, nothing in the others).
template <bool BINARY, bool DENSE>
__device__ __forceinline__ void va_round(const BwdArgs& G, const ItemParams& P, VaShared& sh, const float* diffb,
                                         int tb, int nch, int nnz, float ox, float oy, float oz,
                                         float (&tgacc)[VA_BCH], float& agx, float& agy, float& agz, int lane) {
  const GMParams& gm = G.gm;
  const size_t dim = gm.dim;
  const size_t cs4 = dim * dim * dim / 4;  // channel stride in quads
  const float Tcull = fmaxf(P.Tcut, BINARY ? P.Tbin : -1.f);
  const float kexp = P.inv_ar2 * NEG2_LOG2E;
  const bool tail = gm.ta != 0.f || gm.tb != 0.f;  // without a tail nothing lies beyond the Gaussian part
  const float k4 = 4.f * P.inv_ar2, kD = tail ? -gm.D * P.inv_ar2 : 0.f, kE = tail ? -gm.E * P.inv_ar : 0.f;
  const float ta = gm.ta, ntb = -gm.tb;
  const unsigned span = quad_span(P);
  ColBufD& buf = sh.buf;
  unsigned nx = P.hix - P.lox, ny = P.hiy - P.loy;
  unsigned ncols = nx * ny;
  float inv_ny = 1.f / (float)ny;
  for (unsigned cbase = 0; cbase < ncols;) {
    unsigned nkept = compact_columns<ColBufD, true>(buf, P, cbase, ncols, ny, inv_ny, Tcull, ox, oy, gm.res,
                                                    gm.dim, lane);
    __syncwarp();
    auto quad = [&](unsigned i, float dxy2, float exy, const float (&d2v)[4], const float (&ev)[4],
                    const float (&dzv)[4], size_t off) {
      float v[4], dsum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int j = 0; j < 4; j++) {
        float rsq = __fadd_rn(dxy2, d2v[j]);
        if (BINARY) {
          v[j] = rsq < P.Tbin ? 1.f : 0.f;
        } else {
          float tq = fminf(fmaf(ta, sqrt_approx(rsq * P.inv_ar2), ntb), 0.f);
          v[j] = rsq <= P.Tg ? exy * ev[j] : tq * tq;  // tq is zero beyond the cut-off and for a NaN rsq
        }
      }
      const float4* qp = reinterpret_cast<const float4*>(diffb + off) + (size_t)tb * cs4;
#pragma unroll
      for (int c4 = 0; c4 < VA_BCH; c4 += VA_LD) {
        if (c4 >= nch) break;
        // a batch of channels requested together, then used
        float4 dv[VA_LD];
#pragma unroll
        for (int u = 0; u < VA_LD; u++) {
          dv[u] = (c4 + u < nch) ? __ldg(qp) : make_float4(0.f, 0.f, 0.f, 0.f);
          qp += cs4;
        }
#pragma unroll
        for (int u = 0; u < VA_LD; u++) {
          tgacc[c4 + u] = fmaf(v[0], dv[u].x, fmaf(v[1], dv[u].y, fmaf(v[2], dv[u].z,
                               fmaf(v[3], dv[u].w, tgacc[c4 + u]))));
          if (DENSE) {
            float wk = sh.w[c4 + u];
            dsum[0] = fmaf(wk, dv[u].x, dsum[0]);
            dsum[1] = fmaf(wk, dv[u].y, dsum[1]);
            dsum[2] = fmaf(wk, dv[u].z, dsum[2]);
            dsum[3] = fmaf(wk, dv[u].w, dsum[3]);
          }
        }
      }
      if (!DENSE) {
        if (nnz == 0) return;  // the same for every lane
        const float4* q0 = reinterpret_cast<const float4*>(diffb + off) + (size_t)tb * cs4;
        for (int k = 0; k < nnz; k++) {
          float4 d = __ldg(q0 + (size_t)sh.nz_t[k] * cs4);
          float wk = sh.nz_w[k];
          dsum[0] = fmaf(wk, d.x, dsum[0]);
          dsum[1] = fmaf(wk, d.y, dsum[1]);
          dsum[2] = fmaf(wk, d.z, dsum[2]);
          dsum[3] = fmaf(wk, d.w, dsum[3]);
        }
      }
      float fsum = 0.f;
#pragma unroll
      for (int j = 0; j < 4; j++) {
        float rsq = __fadd_rn(dxy2, d2v[j]);
        // kE/d + kD is zero at the cut-off and negative beyond it: the clamp stands in for the comparison
        float s1 = rsq <= P.Tg ? k4 * (exy * ev[j]) : fmaxf(fmaf(kE, rsqrt_approx(rsq), kD), 0.f);
        float f = s1 * dsum[j];
        fsum += f;
        agz = fmaf(f, dzv[j], agz);
      }
      agx = fmaf(fsum, buf.dx[i], agx);
      agy = fmaf(fsum, buf.dy[i], agy);
    };
    qlane_sweep_span(span, P, buf, nkept, dim, oz, gm.res, kexp, Tcull, lane, quad);
    __syncwarp();
  }
}

template <bool BINARY>
__global__ void __launch_bounds__(VA_WARPS * 32) k_backward_quads_atom(BwdArgs G) {
  __shared__ VaShared shs[VA_WARPS];
  const GMParams& gm = G.gm;
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  int item = blockIdx.x * VA_WARPS + wid;
  int bl = blockIdx.y;
  int b = G.b0 + bl;
  if (item >= G.N) return;
  VaShared& sh = shs[wid];

  float cx, cy, cz;
  if (G.centers != nullptr) {
    cx = G.centers[b * 3]; cy = G.centers[b * 3 + 1]; cz = G.centers[b * 3 + 2];
  } else {
    cx = G.center_host[0]; cy = G.center_host[1]; cz = G.center_host[2];
  }
  float ox = __fsub_rn(cx, gm.half), oy = __fsub_rn(cy, gm.half), oz = __fsub_rn(cz, gm.half);
  ItemParams P = load_item<false>(G, bl, b, item, ox, oy, oz);

  const size_t chan_stride = (size_t)gm.dim * gm.dim * gm.dim;
  const float* diffb = G.diff + (size_t)b * G.T * chan_stride;
  const size_t ai = (size_t)b * G.N + item;
  const float* wrow = G.type_vector + ai * G.T;
  float agx = 0.f, agy = 0.f, agz = 0.f;

  for (int tb = 0; tb < G.T; tb += VA_BCH) {
    const int nch = min(VA_BCH, G.T - tb);
    float tgacc[VA_BCH];
#pragma unroll
    for (int c = 0; c < VA_BCH; c++) tgacc[c] = 0.f;
    if (P.valid) {
      // the round's weights, and the list of the channels that carry one
      __syncwarp();
      float w = lane < nch ? wrow[tb + lane] : 0.f;
      unsigned m = __ballot_sync(0xffffffffu, w != 0.f);
      if (lane < VA_BCH) sh.w[lane] = w;
      if (w != 0.f) {
        int k = __popc(m & ((1u << lane) - 1u));
        sh.nz_t[k] = lane;
        sh.nz_w[k] = w;
      }
      __syncwarp();
      int nnz = __popc(m);
      if (nnz > VA_REREAD) va_round<BINARY, true>(G, P, sh, diffb, tb, nch, nnz, ox, oy, oz, tgacc, agx, agy, agz, lane);
      else va_round<BINARY, false>(G, P, sh, diffb, tb, nch, nnz, ox, oy, oz, tgacc, agx, agy, agz, lane);
    }
    // type gradients of this round
#pragma unroll
    for (int c = 0; c < VA_BCH; c++) {
      float x = tgacc[c];
#pragma unroll
      for (int o = 16; o >= 1; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
      if (lane == 0 && c < nch) G.type_gradients[ai * G.T + tb + c] = x;
    }
  }
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) {
    agx += __shfl_xor_sync(0xffffffffu, agx, o);
    agy += __shfl_xor_sync(0xffffffffu, agy, o);
    agz += __shfl_xor_sync(0xffffffffu, agz, o);
  }
  if (lane == 0) {
    G.atom_gradients[ai * 3] = agx;
    G.atom_gradients[ai * 3 + 1] = agy;
    G.atom_gradients[ai * 3 + 2] = agz;
  }
}

// The same without type gradients (the caller passed none: types that are inputs, not parameters):
// only the channels that carry weight are read.
__global__ void __launch_bounds__(BWD2_WARPS * 32) k_backward_quads_atom_ag(BwdArgs G) {
  __shared__ ColBufD bufs[BWD2_WARPS];
  __shared__ ZTabs ztabs[BWD2_WARPS];
  __shared__ int nz_t[BWD2_WARPS][VA_CH];
  __shared__ float nz_w[BWD2_WARPS][VA_CH];
  const GMParams& gm = G.gm;
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  int item = blockIdx.x * BWD2_WARPS + wid;
  int bl = blockIdx.y;
  int b = G.b0 + bl;
  if (item >= G.N) return;
  ColBufD& buf = bufs[wid];
  ZTabs& zt = ztabs[wid];

  float cx, cy, cz;
  if (G.centers != nullptr) {
    cx = G.centers[b * 3]; cy = G.centers[b * 3 + 1]; cz = G.centers[b * 3 + 2];
  } else {
    cx = G.center_host[0]; cy = G.center_host[1]; cz = G.center_host[2];
  }
  float ox = __fsub_rn(cx, gm.half), oy = __fsub_rn(cy, gm.half), oz = __fsub_rn(cz, gm.half);
  ItemParams P = load_item<false>(G, bl, b, item, ox, oy, oz);

  size_t dim = gm.dim;
  const size_t chan_stride = dim * dim * dim;
  const float* diffb = G.diff + (size_t)b * G.T * chan_stride;
  const size_t ai = (size_t)b * G.N + item;
  const float* wrow = G.type_vector + ai * G.T;
  const float kexp = P.inv_ar2 * NEG2_LOG2E;
  const float k4 = 4.f * P.inv_ar2, kD = -gm.D * P.inv_ar2, kE = -gm.E * P.inv_ar;
  float agx = 0.f, agy = 0.f, agz = 0.f;

  for (int tb = 0; P.valid && tb < G.T; tb += VA_CH) {
    int t = tb + lane;
    float w = t < G.T ? wrow[t] : 0.f;
    unsigned m = __ballot_sync(0xffffffffu, w != 0.f);
    int nnz = __popc(m);
    if (nnz == 0) continue;
    __syncwarp();
    if (w != 0.f) {
      int slot = __popc(m & ((1u << lane) - 1u));
      nz_t[wid][slot] = t;
      nz_w[wid][slot] = w;
    }
    __syncwarp();
    unsigned nx = P.hix - P.lox, ny = P.hiy - P.loy;
    unsigned ncols = nx * ny;
    float inv_ny = 1.f / (float)ny;
    for (unsigned cbase = 0; cbase < ncols;) {
      unsigned nkept = compact_columns<ColBufD, true>(buf, P, cbase, ncols, ny, inv_ny, P.Tcut, ox, oy,
                                                      gm.res, gm.dim, lane);
      for (unsigned zc = P.loz & ~3u; zc < P.hiz; zc += 4 * QPASS) {
        __syncwarp();
        fill_ztabs(zt, zc, P, oz, gm.res, kexp, lane);
        __syncwarp();
        unsigned nq = min((unsigned)QPASS, (P.hiz - zc + 3) >> 2);
        for (unsigned c0 = 0; c0 < nkept; c0 += 32) {
          unsigned i = c0 + lane;
          bool have = i < nkept;
          float dxy2 = have ? buf.dxy2[i] : CUDART_NAN_F;
          float dx = have ? buf.dx[i] : 0.f, dy = have ? buf.dy[i] : 0.f;
          const float4* row = reinterpret_cast<const float4*>(diffb + (size_t)(have ? buf.row[i] : 0u) * dim + zc);
          float exy4 = k4 * ex2_approx(dxy2 * kexp);
          float fsum = 0.f;
          for (unsigned q = 0; q < nq; q++) {
            float4 d2 = zt.dz2[q], e = zt.ez[q], dz = zt.dz[q];
            float lo = zt.lo[q];
            bool live = __fadd_rn(dxy2, lo) <= P.Tcut;
            float4 ds = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int k = 0; k < nnz; k++) {
              if (live) {
                float wk = nz_w[wid][k];
                float4 dv = __ldg(row + q + (size_t)nz_t[wid][k] * (chan_stride / 4));
                ds.x = fmaf(wk, dv.x, ds.x); ds.y = fmaf(wk, dv.y, ds.y);
                ds.z = fmaf(wk, dv.z, ds.z); ds.w = fmaf(wk, dv.w, ds.w);
              }
            }
            float d2v[4] = {d2.x, d2.y, d2.z, d2.w}, ev[4] = {e.x, e.y, e.z, e.w};
            float dzv[4] = {dz.x, dz.y, dz.z, dz.w}, dsv[4] = {ds.x, ds.y, ds.z, ds.w};
#pragma unroll
            for (int j = 0; j < 4; j++) {
              float rsq = __fadd_rn(dxy2, d2v[j]);
              float sg = rsq <= P.Tg ? exy4 * ev[j] : fmaf(kE, rsqrt_approx(rsq), kD);
              float f = rsq <= P.Tcut ? sg * dsv[j] : 0.f;
              fsum += f;
              agz = fmaf(f, dzv[j], agz);
            }
          }
          agx = fmaf(fsum, dx, agx);
          agy = fmaf(fsum, dy, agy);
        }
      }
      __syncwarp();
    }
  }
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) {
    agx += __shfl_xor_sync(0xffffffffu, agx, o);
    agy += __shfl_xor_sync(0xffffffffu, agy, o);
    agz += __shfl_xor_sync(0xffffffffu, agz, o);
  }
  if (lane == 0) {
    G.atom_gradients[ai * 3] = agx;
    G.atom_gradients[ai * 3 + 1] = agy;
    G.atom_gradients[ai * 3 + 2] = agz;
  }
}

// backward_gradients for the same layout (vector types, per-atom radii), one warp per atom.  Only
// channels in which the atom carries weight take part (src/grid_maker.cpp:573).
// Grid term, per voxel and such channel t:  density * tgrad_t  -  w_t * s * (delta . agrad), with
// s = (d density/d dist)/dist: the two voxel-dependent factors are shared by the channels.
__global__ void __launch_bounds__(QS_WARPS * 32) k_gradgrad_quads_atom(BwdArgs G) {
  __shared__ ColBufD bufs[QS_WARPS];
  __shared__ ZTabs ztabs[QS_WARPS];
  __shared__ int nz_t[QS_WARPS][VA_CH];
  __shared__ float nz_w[QS_WARPS][VA_CH], nz_g[QS_WARPS][VA_CH];
  const GMParams& gm = G.gm;
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  int item = blockIdx.x * QS_WARPS + wid;
  int bl = blockIdx.y;
  int b = G.b0 + bl;
  if (item >= G.N) return;
  ColBufD& buf = bufs[wid];
  ZTabs& zt = ztabs[wid];

  float cx, cy, cz;
  if (G.centers != nullptr) {
    cx = G.centers[b * 3]; cy = G.centers[b * 3 + 1]; cz = G.centers[b * 3 + 2];
  } else {
    cx = G.center_host[0]; cy = G.center_host[1]; cz = G.center_host[2];
  }
  float ox = __fsub_rn(cx, gm.half), oy = __fsub_rn(cy, gm.half), oz = __fsub_rn(cz, gm.half);
  ItemParams P = load_item<false>(G, bl, b, item, ox, oy, oz);
  if (!P.valid) return;

  size_t dim = gm.dim;
  const size_t chan_stride = dim * dim * dim;
  float* outb = G.out_grid + (size_t)b * G.T * chan_stride;
  const size_t ai = (size_t)b * G.N + item;
  const float* wrow = G.type_vector + ai * G.T;
  const float* grow = G.tg_in + ai * G.T;
  const float inx = G.ag_in[ai * 3], iny = G.ag_in[ai * 3 + 1], inz = G.ag_in[ai * 3 + 2];
  const float kexp = P.inv_ar2 * NEG2_LOG2E;
  const float k4 = 4.f * P.inv_ar2, kD = -gm.D * P.inv_ar2, kE = -gm.E * P.inv_ar;
  const float ta = gm.ta, ntb = -gm.tb;

  unsigned nx = P.hix - P.lox, ny = P.hiy - P.loy;
  unsigned ncols = nx * ny;
  float inv_ny = 1.f / (float)ny;
  for (int tb = 0; tb < G.T; tb += VA_CH) {
    int t = tb + lane;
    float w = t < G.T ? wrow[t] : 0.f;
    unsigned m = __ballot_sync(0xffffffffu, w != 0.f);
    int nnz = __popc(m);
    if (nnz == 0) continue;
    __syncwarp();
    if (w != 0.f) {
      int slot = __popc(m & ((1u << lane) - 1u));
      nz_t[wid][slot] = t;
      nz_w[wid][slot] = w;
      nz_g[wid][slot] = grow[t];
    }
    __syncwarp();
    for (unsigned cbase = 0; cbase < ncols;) {
      unsigned nkept = compact_columns<ColBufD, true>(buf, P, cbase, ncols, ny, inv_ny, P.Tcut, ox, oy,
                                                      gm.res, gm.dim, lane);
      for (unsigned zc = P.loz & ~3u; zc < P.hiz; zc += 4 * QPASS) {
        __syncwarp();
        fill_ztabs(zt, zc, P, oz, gm.res, kexp, lane);
        __syncwarp();
        unsigned nq = min((unsigned)QPASS, (P.hiz - zc + 3) >> 2);
        for (unsigned c0 = 0; c0 < nkept; c0 += 32) {
          unsigned i = c0 + lane;
          bool have = i < nkept;
          float dxy2 = have ? buf.dxy2[i] : CUDART_NAN_F;
          float dotxy = have ? fmaf(buf.dx[i], inx, buf.dy[i] * iny) : 0.f;
          float* row = outb + (size_t)(have ? buf.row[i] : 0u) * dim + zc;
          float exy = ex2_approx(dxy2 * kexp);
          for (unsigned q = 0; q < nq; q++) {
            float4 d2 = zt.dz2[q], e = zt.ez[q], dz = zt.dz[q];
            float d2v[4] = {d2.x, d2.y, d2.z, d2.w}, ev[4] = {e.x, e.y, e.z, e.w};
            float dzv[4] = {dz.x, dz.y, dz.z, dz.w}, val[4], sd[4];
            bool any = false;
#pragma unroll
            for (int j = 0; j < 4; j++) {
              float rsq = __fadd_rn(dxy2, d2v[j]);
              float g = exy * ev[j];
              float tq = fminf(fmaf(ta, sqrt_approx(rsq * P.inv_ar2), ntb), 0.f);
              bool gauss = rsq <= P.Tg, in = rsq <= P.Tcut;
              float sg = gauss ? k4 * g : fmaf(kE, rsqrt_approx(rsq), kD);
              float dot = rsq > 0.f ? fmaf(dzv[j], inz, dotxy) : 0.f;
              val[j] = in ? (gauss ? g : tq * tq) : 0.f;
              sd[j] = in ? sg * dot : 0.f;
              any = any || in;
            }
            if (any) {
              for (int k = 0; k < nnz; k++) {
                float wk = nz_w[wid][k], gk = nz_g[wid][k];
                red_add_v4(row + (size_t)nz_t[wid][k] * chan_stride + 4 * q, fmaf(val[0], gk, sd[0] * wk),
                           fmaf(val[1], gk, sd[1] * wk), fmaf(val[2], gk, sd[2] * wk),
                           fmaf(val[3], gk, sd[3] * wk));
              }
            }
          }
        }
      }
      __syncwarp();
    }
  }
}

// Atom term (src/grid_maker.cpp:636-662, second derivatives of src/grid_maker.cu:812-878): per voxel
//   sum_t dv_t [ w_t (alpha (delta.agrad) delta_a + beta agrad_a) + tgrad_t (alpha delta_a^2 + beta) ]
// = (alpha (delta.agrad) delta_a + beta agrad_a) S1 + (alpha delta_a^2 + beta) S2
// with S1 = sum_t w_t dv_t and S2 = sum_t tgrad_t dv_t over the weighted channels.
__global__ void __launch_bounds__(BWD2_WARPS * 32) k_backward_quads_atom_gg(BwdArgs G) {
  __shared__ ColBufD bufs[BWD2_WARPS];
  __shared__ ZTabs ztabs[BWD2_WARPS];
  __shared__ int nz_t[BWD2_WARPS][VA_CH];
  __shared__ float nz_w[BWD2_WARPS][VA_CH], nz_g[BWD2_WARPS][VA_CH];
  const GMParams& gm = G.gm;
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  int item = blockIdx.x * BWD2_WARPS + wid;
  int bl = blockIdx.y;
  int b = G.b0 + bl;
  if (item >= G.N) return;
  ColBufD& buf = bufs[wid];
  ZTabs& zt = ztabs[wid];

  float cx, cy, cz;
  if (G.centers != nullptr) {
    cx = G.centers[b * 3]; cy = G.centers[b * 3 + 1]; cz = G.centers[b * 3 + 2];
  } else {
    cx = G.center_host[0]; cy = G.center_host[1]; cz = G.center_host[2];
  }
  float ox = __fsub_rn(cx, gm.half), oy = __fsub_rn(cy, gm.half), oz = __fsub_rn(cz, gm.half);
  ItemParams P = load_item<false>(G, bl, b, item, ox, oy, oz);

  size_t dim = gm.dim;
  const size_t chan_stride = dim * dim * dim;
  const float* diffb = G.diff + (size_t)b * G.T * chan_stride;
  const size_t ai = (size_t)b * G.N + item;
  const float* wrow = G.type_vector + ai * G.T;
  const float* grow = G.tg_in + ai * G.T;
  const float inx = G.ag_in[ai * 3], iny = G.ag_in[ai * 3 + 1], inz = G.ag_in[ai * 3 + 2];
  const float kexp = P.inv_ar2 * NEG2_LOG2E;
  float agx = 0.f, agy = 0.f, agz = 0.f;

  for (int tb = 0; P.valid && tb < G.T; tb += VA_CH) {
    int t = tb + lane;
    float w = t < G.T ? wrow[t] : 0.f;
    unsigned m = __ballot_sync(0xffffffffu, w != 0.f);
    int nnz = __popc(m);
    if (nnz == 0) continue;
    __syncwarp();
    if (w != 0.f) {
      int slot = __popc(m & ((1u << lane) - 1u));
      nz_t[wid][slot] = t;
      nz_w[wid][slot] = w;
      nz_g[wid][slot] = grow[t];
    }
    __syncwarp();
    unsigned nx = P.hix - P.lox, ny = P.hiy - P.loy;
    unsigned ncols = nx * ny;
    float inv_ny = 1.f / (float)ny;
    for (unsigned cbase = 0; cbase < ncols;) {
      unsigned nkept = compact_columns<ColBufD, true>(buf, P, cbase, ncols, ny, inv_ny, P.Tcut, ox, oy,
                                                      gm.res, gm.dim, lane);
      for (unsigned zc = P.loz & ~3u; zc < P.hiz; zc += 4 * QPASS) {
        __syncwarp();
        fill_ztabs(zt, zc, P, oz, gm.res, kexp, lane);
        __syncwarp();
        unsigned nq = min((unsigned)QPASS, (P.hiz - zc + 3) >> 2);
        for (unsigned c0 = 0; c0 < nkept; c0 += 32) {
          unsigned i = c0 + lane;
          bool have = i < nkept;
          float dxy2 = have ? buf.dxy2[i] : CUDART_NAN_F;
          float dx = have ? buf.dx[i] : 0.f, dy = have ? buf.dy[i] : 0.f;
          const float4* row = reinterpret_cast<const float4*>(diffb + (size_t)(have ? buf.row[i] : 0u) * dim + zc);
          float exy = ex2_approx(dxy2 * kexp);
          float dotxy = fmaf(dx, inx, dy * iny);
          for (unsigned q = 0; q < nq; q++) {
            float4 d2 = zt.dz2[q], e = zt.ez[q], dz = zt.dz[q];
            float lo = zt.lo[q];
            if (!(__fadd_rn(dxy2, lo) <= P.Tcut)) continue;
            float s1[4] = {0.f, 0.f, 0.f, 0.f}, s2[4] = {0.f, 0.f, 0.f, 0.f};
            for (int k = 0; k < nnz; k++) {
              float wk = nz_w[wid][k], gk = nz_g[wid][k];
              float4 dv = __ldg(row + q + (size_t)nz_t[wid][k] * (chan_stride / 4));
              s1[0] = fmaf(wk, dv.x, s1[0]); s1[1] = fmaf(wk, dv.y, s1[1]);
              s1[2] = fmaf(wk, dv.z, s1[2]); s1[3] = fmaf(wk, dv.w, s1[3]);
              s2[0] = fmaf(gk, dv.x, s2[0]); s2[1] = fmaf(gk, dv.y, s2[1]);
              s2[2] = fmaf(gk, dv.z, s2[2]); s2[3] = fmaf(gk, dv.w, s2[3]);
            }
            float d2v[4] = {d2.x, d2.y, d2.z, d2.w}, ev[4] = {e.x, e.y, e.z, e.w}, dzv[4] = {dz.x, dz.y, dz.z, dz.w};
#pragma unroll
            for (int j = 0; j < 4; j++) {
              float rsq = __fadd_rn(dxy2, d2v[j]);
              if (rsq <= P.Tcut) {
                float alpha, beta;
                if (rsq <= P.Tg) {
                  float g = exy * ev[j];
                  alpha = 16.f * g * P.inv_ar2 * P.inv_ar2;
                  beta = -4.f * g * P.inv_ar2;
                } else {
                  float id = rsqrt_approx(rsq);
                  float S = fmaf(gm.D * P.inv_ar, rsq * id, gm.E);
                  beta = S * id * P.inv_ar;
                  alpha = fmaf(gm.D * P.inv_ar2, id * id, -beta * id * id);
                }
                float dzj = dzv[j];
                float ad = alpha * fmaf(dzj, inz, dotxy);
                agx += fmaf(ad, dx, beta * inx) * s1[j] + fmaf(alpha, dx * dx, beta) * s2[j];
                agy += fmaf(ad, dy, beta * iny) * s1[j] + fmaf(alpha, dy * dy, beta) * s2[j];
                agz += fmaf(ad, dzj, beta * inz) * s1[j] + fmaf(alpha, dzj * dzj, beta) * s2[j];
              }
            }
          }
        }
      }
      __syncwarp();
    }
  }
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) {
    agx += __shfl_xor_sync(0xffffffffu, agx, o);
    agy += __shfl_xor_sync(0xffffffffu, agy, o);
    agz += __shfl_xor_sync(0xffffffffu, agz, o);
  }
  if (lane == 0) {
    G.atom_gradients[ai * 3] = agx;
    G.atom_gradients[ai * 3 + 1] = agy;
    G.atom_gradients[ai * 3 + 2] = agz;
  }
}

// atom_gradients[a] = sum over channels in ascending order of partial[a][t] * w[a][t] for w != 0
// (src/grid_maker.cpp:508-515)
__global__ void __launch_bounds__(256) k_reduce_types(BwdArgs G) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= G.nb * G.N) return;
  int bl = i / G.N, a = i - bl * G.N;
  int b = G.b0 + bl;
  const float* w = G.type_vector + ((size_t)b * G.N + a) * G.T;
  const float* p = G.partial + (size_t)i * G.T * 3;
  float gx = 0.f, gy = 0.f, gz = 0.f;
  for (int t = 0; t < G.T; t++) {
    float wt = w[t];
    if (wt != 0.f) {
      if (G.plain_reduce) wt = 1.f;  // backward_gradients: the weight is already inside the partial
      gx = __fadd_rn(gx, __fmul_rn(p[t * 3], wt));
      gy = __fadd_rn(gy, __fmul_rn(p[t * 3 + 1], wt));
      gz = __fadd_rn(gz, __fmul_rn(p[t * 3 + 2], wt));
    }
  }
  size_t ai = (size_t)b * G.N + a;
  G.atom_gradients[ai * 3] = gx;
  G.atom_gradients[ai * 3 + 1] = gy;
  G.atom_gradients[ai * 3 + 2] = gz;
}

// ---------------------------------------------------------------------------------------------
// launchers
// ---------------------------------------------------------------------------------------------

cudaError_t launch_emit(const EmitArgs& A, cudaStream_t st) {
  if (A.gm.rti && A.vec) {
    int n = A.nb * A.T;
    k_chan_params<<<(n + 255) / 256, 256, 0, st>>>(A);
  }
  int n = A.nb * A.N;
  k_emit<<<(n + 255) / 256, 256, 0, st>>>(A);
  return cudaGetLastError();
}

cudaError_t launch_backward(const BwdArgs& G, int mode, cudaStream_t st) {
  long items = (long)G.N * ((mode == 1 || mode == 3) ? G.T : 1);
  if (items == 0 || G.nb == 0) return cudaSuccess;
  dim3 grid((unsigned)((items + BWD2_WARPS - 1) / BWD2_WARPS), G.nb);
  bool bin = G.gm.binary != 0;
  // rows of diff (and of the density, for relevance) start on 16-byte boundaries
  bool quads = G.quads && G.gm.dim % 4 == 0 && (uintptr_t)G.diff % 16 == 0 &&
               (mode != 2 || (uintptr_t)G.density % 16 == 0);
  if (mode == 0) {
    if (quads) k_backward_quads<0, false><<<grid, BWD2_WARPS * 32, 0, st>>>(G);
    else k_backward_warp<0, false><<<grid, BWD2_WARPS * 32, 0, st>>>(G);
  } else if (mode == 1 && quads && !G.gm.rti) {
    // per-atom radii: one work item per atom writes both gradients, no reduction over channels after it
    dim3 ga((unsigned)((G.N + BWD2_WARPS - 1) / BWD2_WARPS), G.nb);
    dim3 gv((unsigned)((G.N + VA_WARPS - 1) / VA_WARPS), G.nb);
    if (G.type_gradients == nullptr) k_backward_quads_atom_ag<<<ga, BWD2_WARPS * 32, 0, st>>>(G);
    else if (bin) k_backward_quads_atom<true><<<gv, VA_WARPS * 32, 0, st>>>(G);
    else k_backward_quads_atom<false><<<gv, VA_WARPS * 32, 0, st>>>(G);
  } else if (mode == 1 && quads && G.type_gradients == nullptr) {
    // radii by channel, no type gradients wanted: only the weighted channels of each atom
    dim3 ga((unsigned)(((long)G.N * nz_groups(G.T) + BWD2_WARPS - 1) / BWD2_WARPS), G.nb);
    if (bin) k_backward_quads_nz<1, true><<<ga, BWD2_WARPS * 32, 0, st>>>(G);
    else k_backward_quads_nz<1, false><<<ga, BWD2_WARPS * 32, 0, st>>>(G);
    int n = G.nb * G.N;
    k_reduce_types<<<(n + 255) / 256, 256, 0, st>>>(G);
  } else if (mode == 1) {
    if (quads && bin) k_backward_quads<1, true><<<grid, BWD2_WARPS * 32, 0, st>>>(G);
    else if (quads) k_backward_quads<1, false><<<grid, BWD2_WARPS * 32, 0, st>>>(G);
    else if (bin) k_backward_warp<1, true><<<grid, BWD2_WARPS * 32, 0, st>>>(G);
    else k_backward_warp<1, false><<<grid, BWD2_WARPS * 32, 0, st>>>(G);
    int n = G.nb * G.N;
    k_reduce_types<<<(n + 255) / 256, 256, 0, st>>>(G);
  } else if (mode == 3 && quads && !G.gm.rti) {
    dim3 ga((unsigned)((G.N + BWD2_WARPS - 1) / BWD2_WARPS), G.nb);
    k_backward_quads_atom_gg<<<ga, BWD2_WARPS * 32, 0, st>>>(G);
  } else if (mode == 3) {
    dim3 ga((unsigned)(((long)G.N * nz_groups(G.T) + BWD2_WARPS - 1) / BWD2_WARPS), G.nb);
    if (quads) k_backward_quads_nz<3, false><<<ga, BWD2_WARPS * 32, 0, st>>>(G);
    else k_backward_warp<3, false><<<grid, BWD2_WARPS * 32, 0, st>>>(G);
    int n = G.nb * G.N;
    k_reduce_types<<<(n + 255) / 256, 256, 0, st>>>(G);
  } else {
    if (quads && bin) k_backward_quads<2, true><<<grid, BWD2_WARPS * 32, 0, st>>>(G);
    else if (quads) k_backward_quads<2, false><<<grid, BWD2_WARPS * 32, 0, st>>>(G);
    else if (bin) k_backward_warp<2, true><<<grid, BWD2_WARPS * 32, 0, st>>>(G);
    else k_backward_warp<2, false><<<grid, BWD2_WARPS * 32, 0, st>>>(G);
  }
  return cudaGetLastError();
}

cudaError_t launch_gradgrad_scatter(const BwdArgs& G, cudaStream_t st) {
  long items = (long)G.N * G.T;
  if (items == 0 || G.nb == 0) return cudaSuccess;
  dim3 grid((unsigned)((items + SCAT_WARPS - 1) / SCAT_WARPS), G.nb);
  if (G.quads && !G.gm.rti && G.gm.dim % 4 == 0 && (uintptr_t)G.out_grid % 16 == 0) {
    dim3 ga((unsigned)((G.N + QS_WARPS - 1) / QS_WARPS), G.nb);
    k_gradgrad_quads_atom<<<ga, QS_WARPS * 32, 0, st>>>(G);
  } else if (G.quads && G.gm.dim % 4 == 0 && (uintptr_t)G.out_grid % 16 == 0) {
    dim3 ga((unsigned)(((long)G.N * nz_groups(G.T) + SCAT_WARPS - 1) / SCAT_WARPS), G.nb);
    k_gradgrad_quads_nz<<<ga, SCAT_WARPS * 32, 0, st>>>(G);
  }
  else
    k_gradgrad_scatter<<<grid, SCAT_WARPS * 32, 0, st>>>(G);
  return cudaGetLastError();
}

cudaError_t launch_forward_scatter(const BwdArgs& G, bool vec, cudaStream_t st) {
  long items = (long)G.N * (vec ? G.T : 1);
  if (items == 0 || G.nb == 0) return cudaSuccess;
  dim3 grid((unsigned)((items + SCAT_WARPS - 1) / SCAT_WARPS), G.nb);
  bool bin = G.gm.binary != 0;
  bool aligned = G.quads && G.gm.dim % 4 == 0 && (uintptr_t)G.out_grid % 16 == 0;
  if (vec && !G.gm.rti && aligned) {
    // per-atom radii: one work item per atom, channels inside
    dim3 ga((unsigned)((G.N + QS_WARPS - 1) / QS_WARPS), G.nb);
    if (bin) k_forward_quads_atom<true, false><<<ga, QS_WARPS * 32, 0, st>>>(G);
    else if (G.precise) k_forward_quads_atom<false, true><<<ga, QS_WARPS * 32, 0, st>>>(G);
    else k_forward_quads_atom<false, false><<<ga, QS_WARPS * 32, 0, st>>>(G);
    return cudaGetLastError();
  }
  if (G.quads && !bin && !G.precise && G.gm.dim % 4 == 0 && (uintptr_t)G.out_grid % 16 == 0) {
    if (vec) {
      // radii by channel: one warp per atom runs the items of its weighted channels
      dim3 ga((unsigned)(((long)G.N * nz_groups(G.T) + SCAT_WARPS - 1) / SCAT_WARPS), G.nb);
      k_forward_quads_nz<<<ga, SCAT_WARPS * 32, 0, st>>>(G);
      return cudaGetLastError();
    }
    dim3 gq((unsigned)((items + QS_WARPS - 1) / QS_WARPS), G.nb);
    k_forward_quads<false><<<gq, QS_WARPS * 32, 0, st>>>(G);
    return cudaGetLastError();
  }
  if (vec) {
    if (bin) k_forward_scatter<true, false, true><<<grid, SCAT_WARPS * 32, 0, st>>>(G);
    else if (G.precise) k_forward_scatter<false, true, true><<<grid, SCAT_WARPS * 32, 0, st>>>(G);
    else k_forward_scatter<false, false, true><<<grid, SCAT_WARPS * 32, 0, st>>>(G);
  } else {
    if (bin) k_forward_scatter<true, false, false><<<grid, SCAT_WARPS * 32, 0, st>>>(G);
    else if (G.precise) k_forward_scatter<false, true, false><<<grid, SCAT_WARPS * 32, 0, st>>>(G);
    else k_forward_scatter<false, false, false><<<grid, SCAT_WARPS * 32, 0, st>>>(G);
  }
  return cudaGetLastError();
}

// Slab height: about 110 KB of one channel per block, so that the slabs being worked on together
// (a few per SM) stay in L2 between their clearing and their last reduction.
}  // namespace lmg
