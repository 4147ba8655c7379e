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
//
// Alternative gather forward (forward mode 0, also for the grid term of backward_gradients in that
// mode): emit also counts the atom into every voxel region its footprint touches;
//   scan   : per-example exclusive scan of the (region, channel) counts
//   fill   : writes atom indices into per-(region, channel) lists
//   forward: one warp per 4x8x4-voxel region; per channel the warp turns its list into a per-lane
//            bit mask of atoms whose footprint crosses the lane's z-column, then every lane walks
//            its own mask and accumulates 4 voxels in registers; each output voxel is written
//            exactly once with a 16-byte store (no memset, no read-modify-write of the grid).
#include "lmg_device.cuh"
#include "lmg_launch.h"

namespace lmg {

// ---------------------------------------------------------------------------------------------
// emit
// ---------------------------------------------------------------------------------------------

__device__ __forceinline__ void region_box(const uint4& c, int& rx0, int& rx1, int& ry0, int& ry1,
                                           int& rz0, int& rz1) {
  unsigned lox = lo16(c.x), loy = hi16(c.x), hix = lo16(c.y), hiy = hi16(c.y);
  unsigned loz = lo16(c.z), hiz = hi16(c.z);
  rx0 = lox / REG_X; rx1 = (hix - 1) / REG_X;
  ry0 = loy / REG_Y; ry1 = (hiy - 1) / REG_Y;
  rz0 = loz / REG_Z; rz1 = (hiz - 1) / REG_Z;
}

// True when the axis-aligned box of region (rx,ry,rz) can hold a voxel within sqrt(Tcull) of the
// atom.  Conservative (the threshold is widened by a few ulps' worth), and a pure function of its
// arguments so that the counting and the filling pass agree.
__device__ __forceinline__ bool region_in_reach(const GMParams& gm, float ox, float oy, float oz,
                                                float ax, float ay, float az, float Tcull,
                                                int rx, int ry, int rz) {
  unsigned last = gm.dim - 1;
  float x0 = voxel_coord(ox, rx * REG_X, gm.res), x1 = voxel_coord(ox, min((unsigned)(rx * REG_X + REG_X - 1), last), gm.res);
  float y0 = voxel_coord(oy, ry * REG_Y, gm.res), y1 = voxel_coord(oy, min((unsigned)(ry * REG_Y + REG_Y - 1), last), gm.res);
  float z0 = voxel_coord(oz, rz * REG_Z, gm.res), z1 = voxel_coord(oz, min((unsigned)(rz * REG_Z + REG_Z - 1), last), gm.res);
  float dx = fmaxf(fmaxf(x0 - ax, ax - x1), 0.f);
  float dy = fmaxf(fmaxf(y0 - ay, ay - y1), 0.f);
  float dz = fmaxf(fmaxf(z0 - az, az - z1), 0.f);
  float d2 = dx * dx + dy * dy + dz * dz;
  return d2 <= Tcull * 1.0001f + 1e-12f;
}

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
      // If even the nearest voxel layers outside [lo.z, hi.z) are farther than the cut-off by
      // their z distance alone, the z test of the footprint can never decide anything.
      bool zfree = true;
      if (loz > 0) {
        float dzl = __fsub_rn(voxel_coord(oz, loz - 1, gm.res), z);
        zfree = zfree && dzl <= 0.f && __fmul_rn(dzl, dzl) > cp.q.w;
      }
      if (hiz < gm.dim) {
        float dzh = __fsub_rn(voxel_coord(oz, hiz, gm.res), z);
        zfree = zfree && dzh >= 0.f && __fmul_rn(dzh, dzh) > cp.q.w;
      }
      r.c = make_uint4(lox | (loy << 16), hix | (hiy << 16), loz | (hiz << 16),
                       (unsigned)chan | ((REC_VALID | (zfree ? REC_ZFREE : 0u)) << 16));
      r.d = make_float4(cp.p.w, cp.q.x, cp.q.y, cp.q.z);
    }
    valid = any;
  }

  if (valid && A.cnt != nullptr) {
    int rx0, rx1, ry0, ry1, rz0, rz1;
    region_box(r.c, rx0, rx1, ry0, ry1, rz0, rz1);
    int nslots = (rx1 - rx0 + 1) * (ry1 - ry0 + 1) * (rz1 - rz0 + 1);
    if (nslots > A.cap) {
      r.c.w |= REC_BIG << 16;
      unsigned p = atomicAdd(&A.bigcount[bl], 1u);
      A.biglist[(size_t)bl * A.N + p] = (unsigned)a;
    } else {
      unsigned* cnt = A.cnt + (size_t)bl * A.M;
      int tb = A.vec ? 1 : A.T;
      int ch = A.vec ? 0 : chan;
      for (int rx = rx0; rx <= rx1; rx++)
        for (int ry = ry0; ry <= ry1; ry++)
          for (int rz = rz0; rz <= rz1; rz++) {
            if (!region_in_reach(gm, ox, oy, oz, r.a.x, r.a.y, r.a.z, r.a.w, rx, ry, rz)) continue;
            int reg = (rx * A.nry + ry) * A.nrz + rz;
            atomicAdd(&cnt[(size_t)reg * tb + ch], 1u);
          }
    }
  }
  A.recs[i] = r;
}

// ---------------------------------------------------------------------------------------------
// scan: in-place exclusive prefix sum of the M counters of each example
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024) k_scan(unsigned* cnt, int M) {
  __shared__ unsigned warp_tot[32];
  __shared__ unsigned carry_s;
  unsigned* c = cnt + (size_t)blockIdx.x * M;
  int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  if (tid == 0) carry_s = 0;
  __syncthreads();
  const int per = 8;
  for (int base = 0; base < M; base += 1024 * per) {
    unsigned v[per];
    unsigned sum = 0;
    int i0 = base + tid * per;
#pragma unroll
    for (int k = 0; k < per; k++) {
      v[k] = (i0 + k < M) ? c[i0 + k] : 0u;
      sum += v[k];
    }
    unsigned inc = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      unsigned n = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += n;
    }
    if (lane == 31) warp_tot[wid] = inc;
    __syncthreads();
    if (wid == 0) {
      unsigned w = warp_tot[lane];
      unsigned winc = w;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        unsigned n = __shfl_up_sync(0xffffffffu, winc, o);
        if (lane >= o) winc += n;
      }
      warp_tot[lane] = winc - w;  // exclusive
    }
    __syncthreads();
    unsigned carry = carry_s;
    unsigned excl = carry + warp_tot[wid] + inc - sum;
#pragma unroll
    for (int k = 0; k < per; k++) {
      if (i0 + k < M) c[i0 + k] = excl;
      excl += v[k];
    }
    __syncthreads();
    if (tid == 1023) carry_s = excl;
    __syncthreads();
  }
}

// ---------------------------------------------------------------------------------------------
// fill: after this kernel cnt[bin] holds the END offset of the bin (begin = end of the bin before)
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) k_fill(EmitArgs A) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= A.nb * A.N) return;
  int bl = i / A.N, a = i - bl * A.N;
  uint4 c = A.recs[i].c;
  unsigned flags = c.w >> 16;
  if (!(flags & REC_VALID) || (flags & REC_BIG)) return;
  float4 ra = A.recs[i].a;
  int b = A.b0 + bl;
  float cx, cy, cz;
  if (A.centers != nullptr) {
    cx = A.centers[b * 3]; cy = A.centers[b * 3 + 1]; cz = A.centers[b * 3 + 2];
  } else {
    cx = A.center_host[0]; cy = A.center_host[1]; cz = A.center_host[2];
  }
  float ox = __fsub_rn(cx, A.gm.half), oy = __fsub_rn(cy, A.gm.half), oz = __fsub_rn(cz, A.gm.half);
  int rx0, rx1, ry0, ry1, rz0, rz1;
  region_box(c, rx0, rx1, ry0, ry1, rz0, rz1);
  unsigned* cnt = A.cnt + (size_t)bl * A.M;
  unsigned* list = A.list + (size_t)bl * A.listcap;
  int tb = A.vec ? 1 : A.T;
  int ch = A.vec ? 0 : (int)(c.w & 0xffffu);
  for (int rx = rx0; rx <= rx1; rx++)
    for (int ry = ry0; ry <= ry1; ry++)
      for (int rzb = rz0; rzb <= rz1; rzb += 4) {
        // four regions per step: their atomics are issued before any result is consumed
        bool in[4];
        unsigned p[4];
#pragma unroll
        for (int k = 0; k < 4; k++) {
          int rz = rzb + k;
          in[k] = rz <= rz1 && region_in_reach(A.gm, ox, oy, oz, ra.x, ra.y, ra.z, ra.w, rx, ry, rz);
        }
#pragma unroll
        for (int k = 0; k < 4; k++) {
          int reg = (rx * A.nry + ry) * A.nrz + rzb + k;
          p[k] = in[k] ? atomicAdd(&cnt[(size_t)reg * tb + ch], 1u) : 0u;
        }
#pragma unroll
        for (int k = 0; k < 4; k++)
          if (in[k]) list[p[k]] = (unsigned)a;
      }
}

// ---------------------------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------------------------

constexpr int FWD_WARPS = 4;        // warps per block of the vector-typed kernel (one region each)
constexpr int FWD_INDEX_WARPS = 8;  // warps sharing one region in the index-typed kernel

// ---------------------------------------------------------------------------------------------
// forward, vector types (and the grid part of backward_gradients)
//
// One warp per region; the region's atom list is shared by all channels, so the warp loops over
// the channels and, for each, stages the atoms that carry weight in that channel.  With
// type-indexed radii the footprint and thresholds of an (atom, channel) pair are built here.
// GRADGRAD evaluates, instead of the density, the derivative of the backward pass with respect
// to the grid gradient (src/grid_maker.cpp:618-634).
// ---------------------------------------------------------------------------------------------

struct __align__(16) Cand {
  float4 a;  // x, y, z, Tcull
  float4 b;  // w, inv_ar2 (or ar when PRECISE), Tg, Tcut (Tbin when BINARY)
  uint4 c;   // lo.x|lo.y<<16, hi.x|hi.y<<16, lo.z|hi.z<<16, bits of 1/ar
  float4 g;  // GRADGRAD: incoming atom gradient x, y, z and type gradient of this channel
};

template <bool BINARY, bool PRECISE, bool GRADGRAD>
__global__ void __launch_bounds__(FWD_WARPS * 32) k_forward_vector(FwdArgs F) {
  __shared__ Cand cand_s[FWD_WARPS][32];
  const GMParams& gm = F.gm;
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  int reg = blockIdx.x * FWD_WARPS + wid;
  int bl = blockIdx.y;
  int b = F.b0 + bl;
  int nreg = F.nrx * F.nry * F.nrz;
  if (reg >= nreg) return;
  Cand* cs = cand_s[wid];

  int rz = reg % F.nrz;
  int ry = (reg / F.nrz) % F.nry;
  int rx = reg / (F.nrz * F.nry);
  unsigned vx = rx * REG_X + (lane >> 3), vy = ry * REG_Y + (lane & 7), vz0 = rz * REG_Z;
  bool col_ok = vx < gm.dim && vy < gm.dim;

  float cx, cy, cz;
  if (F.centers != nullptr) {
    cx = F.centers[b * 3]; cy = F.centers[b * 3 + 1]; cz = F.centers[b * 3 + 2];
  } else {
    cx = F.center_host[0]; cy = F.center_host[1]; cz = F.center_host[2];
  }
  float ox = __fsub_rn(cx, gm.half), oy = __fsub_rn(cy, gm.half), oz = __fsub_rn(cz, gm.half);
  float gx = voxel_coord(ox, vx, gm.res), gy = voxel_coord(oy, vy, gm.res);
  float gz[REG_Z];
#pragma unroll
  for (int k = 0; k < REG_Z; k++) gz[k] = voxel_coord(oz, vz0 + k, gm.res);

  const Rec* recs = F.recs + (size_t)bl * F.N;
  const unsigned* cnt = F.cnt + (size_t)bl * F.M;
  const unsigned* list = F.list + (size_t)bl * F.listcap;
  unsigned nbig = F.bigcount[bl];
  const unsigned* biglist = F.biglist + (size_t)bl * F.N;
  size_t dim = gm.dim;
  float* outb = F.out + (size_t)b * F.T * dim * dim * dim;
  bool vec4_ok = F.vec4_ok;
  unsigned beg = reg == 0 ? 0u : cnt[reg - 1];
  unsigned nlist = cnt[reg] - beg;
  unsigned total = nlist + nbig;  // atoms too large for the lists are visited by every region

  for (int chan = 0; chan < F.T; chan++) {
    float acc[REG_Z];
#pragma unroll
    for (int k = 0; k < REG_Z; k++) acc[k] = 0.f;
    ChanParam cp;
    if (gm.rti) cp = F.chanp[(size_t)bl * F.T + chan];

    for (unsigned base = 0; base < total; base += 32) {
      unsigned n = min(32u, total - base);
      // ---- stage up to 32 candidates ----
      bool have = false;
      if (lane < n) {
        unsigned e = base + lane;
        unsigned ai = e < nlist ? list[beg + e] : biglist[e - nlist];
        const Rec* rp = recs + ai;
        float4 ra = rp->a, rb = rp->b;
        uint4 rc = rp->c;
        Cand cd;
        size_t gi = (size_t)b * F.N + ai;
        float w = F.type_vector[gi * F.T + chan];
        bool use = w != 0.f;
        if (!gm.rti) {
          cd.a = ra;
          cd.b = make_float4(w, PRECISE ? rp->d.z : rb.y, rb.z, BINARY ? rp->d.y : rp->d.x);
          cd.c = make_uint4(rc.x, rc.y, rc.z, __float_as_uint(rb.w));
        } else {
          // per-channel radius: footprint and thresholds of this (atom, channel)
          unsigned lox, hix, loy, hiy, loz, hiz;
          bounds_1d(ox, ra.x, cp.q.z, gm.res, gm.dim, lox, hix);
          bounds_1d(oy, ra.y, cp.q.z, gm.res, gm.dim, loy, hiy);
          bounds_1d(oz, ra.z, cp.q.z, gm.res, gm.dim, loz, hiz);
          cd.a = make_float4(ra.x, ra.y, ra.z, cp.q.w);
          cd.b = make_float4(w, PRECISE ? cp.q.y : cp.p.x, cp.p.y, BINARY ? cp.q.x : cp.p.w);
          cd.c = make_uint4(lox | (loy << 16), hix | (hiy << 16), loz | (hiz << 16),
                            __float_as_uint(cp.p.z));
          use = use && cp.q.y > 0.f;
        }
        if (GRADGRAD) {
          cd.g = make_float4(F.atom_gradients[gi * 3], F.atom_gradients[gi * 3 + 1],
                             F.atom_gradients[gi * 3 + 2], F.type_gradients[gi * F.T + chan]);
        } else {
          cd.g = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        if (!use) cd.a.w = -1.f;  // nothing passes a negative threshold
        cs[lane] = cd;
        have = use;
      }
      __syncwarp();
      // ---- column test: bit i set when candidate i can touch this lane's z-column ----
      unsigned mask = 0;
      if (__any_sync(0xffffffffu, have)) {
        for (unsigned i = 0; i < n; i++) {
          float4 a = cs[i].a;
          uint2 bb = *reinterpret_cast<const uint2*>(&cs[i].c);
          float dx = __fsub_rn(gx, a.x), dy = __fsub_rn(gy, a.y);
          float dxy2 = __fadd_rn(__fmul_rn(dx, dx), __fmul_rn(dy, dy));
          bool p = dxy2 <= a.w;
          p = p && (vx - lo16(bb.x)) < (lo16(bb.y) - lo16(bb.x));
          p = p && (vy - hi16(bb.x)) < (hi16(bb.y) - hi16(bb.x));
          mask |= (p ? 1u : 0u) << i;
        }
      }
      if (!col_ok) mask = 0;
      // ---- each lane walks its own candidates ----
      while (mask) {
        int i = __ffs(mask) - 1;
        mask &= mask - 1;
        float4 a = cs[i].a, bq = cs[i].b;
        uint4 cc = cs[i].c;
        float dx = __fsub_rn(gx, a.x), dy = __fsub_rn(gy, a.y);
        float dxy2 = __fadd_rn(__fmul_rn(dx, dx), __fmul_rn(dy, dy));
        unsigned loz = lo16(cc.z), nz = hi16(cc.z) - loz;
        float4 gg = make_float4(0.f, 0.f, 0.f, 0.f);
        float kD = 0.f, kE = 0.f, k4 = 0.f, dotxy = 0.f;
        if (GRADGRAD) {
          gg = cs[i].g;
          float inv_ar = __uint_as_float(cc.w);
          k4 = -4.f * bq.y; kD = gm.D * bq.y; kE = gm.E * inv_ar;
          dotxy = fmaf(dx, gg.x, dy * gg.y);
        }
#pragma unroll
        for (int k = 0; k < REG_Z; k++) {
          float dz = __fsub_rn(gz[k], a.z);
          float rsq = __fadd_rn(dxy2, __fmul_rn(dz, dz));
          bool inz = (vz0 + k - loz) < nz;
          if (GRADGRAD) {
            // -(w * (d density/d dist)/dist) * (delta . atom gradient) + density * type gradient,
            // only where the voxel is within the cut-off (the reference's isfinite test)
            float e = ex2_approx(rsq * bq.y * NEG2_LOG2E);
            float sq = sqrt_approx(rsq * bq.y);
            float q = fmaxf(fmaf(fmaf(gm.A, sq, gm.B), sq, gm.C), 0.f);
            bool gauss = rsq <= bq.z;
            float val = gauss ? e : q;
            float s = gauss ? k4 * e : fmaf(kE, rsqrt_approx(rsq), kD);
            float dot = fmaf(dz, gg.z, dotxy);
            float gval = fmaf(val, gg.w, -(bq.x * s) * (rsq > 0.f ? dot : 0.f));
            if (inz && rsq <= bq.w) acc[k] += gval;
          } else if (BINARY) {
            if (inz && rsq < bq.w) acc[k] = __fadd_rn(acc[k], bq.x);
          } else {
            float v = PRECISE ? density_precise(rsq, bq.y, bq.z, bq.w, gm.A, gm.B, gm.C)
                              : density_fast(rsq, bq.y, bq.z, bq.w, gm.A, gm.B, gm.C);
            if (PRECISE) {
              if (inz) acc[k] = __fadd_rn(acc[k], __fmul_rn(v, bq.x));
            } else {
              acc[k] = fmaf(inz ? v : 0.f, bq.x, acc[k]);
            }
          }
        }
      }
      __syncwarp();
    }

    // ---- write this channel's 4 voxels ----
    if (col_ok) {
      float* o = outb + (((size_t)chan * dim + vx) * dim + vy) * dim + vz0;
      if (vec4_ok) {
        if (vz0 + REG_Z <= gm.dim) {
          __stcs(reinterpret_cast<float4*>(o), make_float4(acc[0], acc[1], acc[2], acc[3]));
        }
      } else {
#pragma unroll
        for (int k = 0; k < REG_Z; k++)
          if (vz0 + k < gm.dim) o[k] = acc[k];
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// forward, index types: the lists of one region are contiguous over channels, so the warp walks
// them in chunks of 32 atoms regardless of channel.  Each lane keeps the 4 voxels of the channel
// it is currently in and stores them when its next atom belongs to another channel.
// ---------------------------------------------------------------------------------------------

// out[lane j] bit i = in[lane i] bit j
__device__ __forceinline__ unsigned warp_transpose32(unsigned x, int lane) {
  unsigned m = 0x0000ffffu;
#pragma unroll
  for (int j = 16; j >= 1; j >>= 1) {
    unsigned p = __shfl_xor_sync(0xffffffffu, x, j);
    x = (lane & j) ? (((p >> j) & m) | (x & ~m)) : ((x & m) | ((p & m) << j));
    m ^= m << (j >> 1);
  }
  return x;
}

struct __align__(16) CandI {
  float4 a;  // x, y, z, Tcull
  float4 b;  // kexp (ar when PRECISE), 1/ar^2, Tg, Tcut (Tbin when BINARY)
  uint4 c;   // lo.z|hi.z<<16, channel | zfree<<16, unused, unused
};


// Adds one atom's density at the REG_Z voxels of a lane's column.  CHECKZ applies the footprint's
// z range [lo.z, hi.z) (zoff = first voxel - lo.z, nz = hi.z - lo.z) on top of the radial test.
template <bool BINARY, bool PRECISE, bool CHECKZ>
__device__ __forceinline__ void fwd_eval4(float (&acc)[REG_Z], const float (&gz)[REG_Z], float az,
                                          float dxy2, float4 bq, float A_, float B_,
                                          float C_, unsigned zoff, unsigned nz) {
#pragma unroll
  for (int k = 0; k < REG_Z; k++) {
    float dz = __fsub_rn(gz[k], az);
    float rsq = __fadd_rn(dxy2, __fmul_rn(dz, dz));
    bool inz = !CHECKZ || (zoff + k) < nz;
    if (BINARY) {
      if (inz && rsq < bq.w) acc[k] = 1.f;
    } else if (PRECISE) {
      float v = density_precise(rsq, bq.x, bq.z, bq.w, A_, B_, C_);
      if (inz) acc[k] = __fadd_rn(acc[k], v);
    } else {
      // the tail keeps the reference's polynomial and constants so that its rounding residue near
      // the zero at final_radius_multiple cancels against the reference's instead of adding to it
      float g = ex2_approx(rsq * bq.x);
      float sq = sqrt_approx(rsq * bq.y);
      float q = fmaxf(fmaf(fmaf(A_, sq, B_), sq, C_), 0.f);
      float v = rsq <= bq.z ? g : q;
      acc[k] += (inz && rsq <= bq.w) ? v : 0.f;
    }
  }
}

template <bool BINARY, bool PRECISE>
__global__ void __launch_bounds__(FWD_INDEX_WARPS * 32) k_forward_index(FwdArgs F) {
  __shared__ CandI cand_s[FWD_INDEX_WARPS][32];
  const GMParams& gm = F.gm;
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  // one block per region; its warps split the channels so that a crowded region is worked on by
  // several warps, each owning whole channels (no two warps ever write the same voxel)
  // Blocks run example by example; within an example the x-slabs are visited from the middle of
  // the grid outwards.  Molecules sit around the grid centre, so each example starts with its
  // crowded (compute-bound) regions and ends with sparse (store-bound) ones: the end of one example
  // overlaps the start of the next, and the launch as a whole ends with light work.
  // (Measured alternatives: all crowded regions of the batch first, or region-major order with
  // examples fastest, are 10-20 % slower because they separate the two kinds of work.  Persistent
  // warps taking (region, channel range) items from a device-built list were 40 % slower: sparse
  // regions are chains of dependent loads, and many short-lived warps hide those better.)
  int bl = blockIdx.y;
  int b = F.b0 + bl;
  int reg;
  {
    int per_slab = F.nry * F.nrz;
    int s = blockIdx.x / per_slab, rest = blockIdx.x - s * per_slab;
    int mid = (F.nrx - 1) / 2;
    int rxp = mid + ((s & 1) ? (s + 1) / 2 : -(s / 2));
    reg = rxp * per_slab + rest;
  }
  // (Letting one warp take all channels of a sparsely populated region was tried and is slower:
  // the warps that leave early keep the block's registers allocated until the last one is done.)
  const unsigned* cnt = F.cnt + (size_t)bl * F.M;
  int cbeg = (wid * F.T) / FWD_INDEX_WARPS, cend = ((wid + 1) * F.T) / FWD_INDEX_WARPS;
  if (cbeg >= cend) return;
  CandI* cs = cand_s[wid];

  int rz = reg % F.nrz;
  int ry = (reg / F.nrz) % F.nry;
  int rx = reg / (F.nrz * F.nry);
  unsigned x0 = rx * REG_X, y0 = ry * REG_Y;
  unsigned vx = x0 + (lane >> 3), vy = y0 + (lane & 7), vz0 = rz * REG_Z;
  bool col_ok = vx < gm.dim && vy < gm.dim;

  float cx, cy, cz;
  if (F.centers != nullptr) {
    cx = F.centers[b * 3]; cy = F.centers[b * 3 + 1]; cz = F.centers[b * 3 + 2];
  } else {
    cx = F.center_host[0]; cy = F.center_host[1]; cz = F.center_host[2];
  }
  float ox = __fsub_rn(cx, gm.half), oy = __fsub_rn(cy, gm.half), oz = __fsub_rn(cz, gm.half);
  float gx = voxel_coord(ox, vx, gm.res), gy = voxel_coord(oy, vy, gm.res);
  float gz[REG_Z];
#pragma unroll
  for (int k = 0; k < REG_Z; k++) gz[k] = voxel_coord(oz, vz0 + k, gm.res);
  float gxr[REG_X];
#pragma unroll
  for (int k = 0; k < REG_X; k++) gxr[k] = voxel_coord(ox, x0 + k, gm.res);

  const Rec* recs = F.recs + (size_t)bl * F.N;
  const unsigned* list = F.list + (size_t)bl * F.listcap;
  size_t dim = gm.dim;
  float* outb = F.out + (size_t)b * F.T * dim * dim * dim;
  float* ocol = outb + ((size_t)vx * dim + vy) * dim + vz0;  // + chan * dim^3
  size_t chan_stride = dim * dim * dim;
  bool vec4_ok = F.vec4_ok;
  float A_ = gm.A, B_ = gm.B, C_ = gm.C;

  for (int g0 = cbeg; g0 < cend; g0 += 32) {
    int g1 = min(g0 + 32, cend);
    size_t bin0 = (size_t)reg * F.T + g0;
    unsigned beg = bin0 == 0 ? 0u : cnt[bin0 - 1];
    unsigned end = cnt[(size_t)reg * F.T + g1 - 1];
    int cur = -1;
    unsigned written = 0;
    float acc[REG_Z];
#pragma unroll
    for (int k = 0; k < REG_Z; k++) acc[k] = 0.f;

    auto flush = [&]() {
      if (cur >= 0 && col_ok) {
        float* o = ocol + (size_t)cur * chan_stride;
        if (vec4_ok) {
          __stcs(reinterpret_cast<float4*>(o), make_float4(acc[0], acc[1], acc[2], acc[3]));
        } else {
#pragma unroll
          for (int k = 0; k < REG_Z; k++)
            if (vz0 + k < gm.dim) o[k] = acc[k];
        }
        written |= 1u << (cur - g0);
      }
    };

    // Two-deep prefetch: while chunk j is evaluated, the records of chunk j+1 are in flight (their
    // list indices were loaded one chunk earlier) and the list indices of chunk j+2 are requested,
    // so the dependent index -> record gather never stalls the loop.
    float4 pa = make_float4(0.f, 0.f, 0.f, -1.f), pb = pa, pd = pa;
    uint4 pc = make_uint4(0u, 0u, 0u, 0u);
    unsigned nidx = 0;
    if (beg + lane < end) {
      const Rec* rp = recs + list[beg + lane];
      pa = rp->a; pb = rp->b; pc = rp->c; pd = rp->d;
    }
    if (beg + 32 + lane < end) nidx = list[beg + 32 + lane];
    for (unsigned base = beg; base < end; base += 32) {
      unsigned n = min(32u, end - base);
      unsigned bm = 0;
      float4 ra = pa, rb = pb, rd = pd;
      uint4 rc = pc;
      if (base + 32 + lane < end) {
        const Rec* rp = recs + nidx;
        pa = rp->a; pb = rp->b; pc = rp->c; pd = rp->d;
      }
      if (base + 64 + lane < end) nidx = list[base + 64 + lane];
      if (lane < n) {
        CandI cd;
        cd.a = ra;
        cd.b = make_float4(PRECISE ? rd.z : rb.y * NEG2_LOG2E, rb.y, rb.z, BINARY ? rd.y : rd.x);
        cd.c = make_uint4(rc.z, (rc.w & 0xffffu) | ((rc.w >> 16) & REC_ZFREE) << 16, 0u, 0u);
        cs[lane] = cd;
        // columns of this region inside the atom's integer footprint, minus x-rows that are
        // farther than the cut-off by their x distance alone
        int lx = max((int)lo16(rc.x) - (int)x0, 0), hx = min((int)lo16(rc.y) - (int)x0, REG_X);
        int ly = max((int)hi16(rc.x) - (int)y0, 0), hy = min((int)hi16(rc.y) - (int)y0, REG_Y);
        unsigned ym = (hy > ly) ? (((1u << hy) - 1u) & ~((1u << ly) - 1u)) : 0u;
#pragma unroll
        for (int k = 0; k < REG_X; k++) {
          float dxr = __fsub_rn(gxr[k], ra.x);
          bool rowin = k >= lx && k < hx && __fmul_rn(dxr, dxr) <= ra.w;
          if (rowin) bm |= ym << (8 * k);
        }
      }
      __syncwarp();
      unsigned mask = warp_transpose32(bm, lane);
      while (mask) {
        int i = __ffs(mask) - 1;
        mask &= mask - 1;
        float4 a = cs[i].a;
        float4 bq = cs[i].b;
        uint4 cc = cs[i].c;
        int ch = (int)(cc.y & 0xffffu);
        if (ch != cur) {
          flush();
          cur = ch;
#pragma unroll
          for (int k = 0; k < REG_Z; k++) acc[k] = 0.f;
        }
        float dx = __fsub_rn(gx, a.x), dy = __fsub_rn(gy, a.y);
        float dxy2 = __fadd_rn(__fmul_rn(dx, dx), __fmul_rn(dy, dy));
        if (!(dxy2 <= a.w)) continue;
        // the footprint's z range only matters for atoms flagged as needing it (exact ties at the
        // cut-off, truncated Gaussians); everywhere else the radial test already implies it
        if (cc.y >> 16) {
          fwd_eval4<BINARY, PRECISE, false>(acc, gz, a.z, dxy2, bq, A_, B_, C_, 0u, 0u);
        } else {
          unsigned loz = lo16(cc.x);
          fwd_eval4<BINARY, PRECISE, true>(acc, gz, a.z, dxy2, bq, A_, B_, C_, vz0 - loz, hi16(cc.x) - loz);
        }
      }
      __syncwarp();
    }
    flush();
    // channels of this group that no atom of this column touched are zero
    if (col_ok) {
      for (int c = g0; c < g1; c++) {
        if (!((written >> (c - g0)) & 1u)) {
          float* o = ocol + (size_t)c * chan_stride;
          if (vec4_ok) {
            __stcs(reinterpret_cast<float4*>(o), make_float4(0.f, 0.f, 0.f, 0.f));
          } else {
#pragma unroll
            for (int k = 0; k < REG_Z; k++)
              if (vz0 + k < gm.dim) o[k] = 0.f;
          }
        }
      }
    }
  }
}

// Atoms whose footprint spans more regions than the list capacity (far larger than the expected
// radius) are not binned; after the main kernel one block per such atom adds its density into
// the finished grid.  This path only exists so that any radius is handled correctly.
template <bool BINARY, bool PRECISE>
__global__ void __launch_bounds__(128) k_forward_big(FwdArgs F) {
  const GMParams& gm = F.gm;
  int bl = blockIdx.y;
  int b = F.b0 + bl;
  unsigned nbig = F.bigcount[bl];
  if (nbig == 0) return;
  float cx, cy, cz;
  if (F.centers != nullptr) {
    cx = F.centers[b * 3]; cy = F.centers[b * 3 + 1]; cz = F.centers[b * 3 + 2];
  } else {
    cx = F.center_host[0]; cy = F.center_host[1]; cz = F.center_host[2];
  }
  float ox = __fsub_rn(cx, gm.half), oy = __fsub_rn(cy, gm.half), oz = __fsub_rn(cz, gm.half);
  size_t dim = gm.dim;
  for (unsigned e = blockIdx.x; e < nbig; e += gridDim.x) {
    const Rec* rp = F.recs + (size_t)bl * F.N + F.biglist[(size_t)bl * F.N + e];
    float4 ra = rp->a, rb = rp->b, rd = rp->d;
    uint4 rc = rp->c;
    unsigned lox = lo16(rc.x), loy = hi16(rc.x), hix = lo16(rc.y), hiy = hi16(rc.y);
    unsigned loz = lo16(rc.z), hiz = hi16(rc.z);
    unsigned nx = hix - lox, ny = hiy - loy, nz = hiz - loz;
    float* o = F.out + ((size_t)b * F.T + (rc.w & 0xffffu)) * dim * dim * dim;
    size_t total = (size_t)nx * ny * nz;
    for (size_t v = threadIdx.x; v < total; v += blockDim.x) {
      unsigned z = loz + (unsigned)(v % nz), y = loy + (unsigned)((v / nz) % ny), x = lox + (unsigned)(v / ((size_t)nz * ny));
      float dx = __fsub_rn(voxel_coord(ox, x, gm.res), ra.x);
      float dy = __fsub_rn(voxel_coord(oy, y, gm.res), ra.y);
      float dz = __fsub_rn(voxel_coord(oz, z, gm.res), ra.z);
      float rsq = __fadd_rn(__fadd_rn(__fmul_rn(dx, dx), __fmul_rn(dy, dy)), __fmul_rn(dz, dz));
      float* p = o + ((size_t)x * dim + y) * dim + z;
      if (BINARY) {
        if (rsq < rd.y) *p = 1.f;
      } else {
        float val = PRECISE ? density_precise(rsq, rd.z, rb.z, rd.x, gm.A, gm.B, gm.C)
                            : density_fast(rsq, rb.y, rb.z, rd.x, gm.A, gm.B, gm.C);
        if (val != 0.f) atomicAdd(p, val);
      }
    }
  }
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
constexpr int BWD2_COLS = 256;  // compacted columns held per warp at a time
constexpr int ZSTEPS = 4;       // z positions per lane and chunk; a chunk covers 4*ZSTEPS voxels

struct ColBuf {
  unsigned row[BWD2_COLS];  // x*dim + y
  float dxy2[BWD2_COLS];    // (gx-ax)^2 + (gy-ay)^2
};
struct ColBufD {
  unsigned row[BWD2_COLS];
  float dxy2[BWD2_COLS];
  float dx[BWD2_COLS];  // gx-ax
  float dy[BWD2_COLS];
};

// Appends the columns of [cbase, ncols) whose squared distance in the xy plane is <= Tcull to the
// buffer until it is (nearly) full; returns how many it holds and advances cbase.
template <class BUF, bool WITH_D>
__device__ __forceinline__ unsigned compact_columns(BUF& buf, const ItemParams& P, unsigned& cbase,
                                                    unsigned ncols, unsigned ny, float inv_ny, float Tcull,
                                                    float ox, float oy, float res, unsigned dim, int lane) {
  unsigned nkept = 0;
  while (cbase < ncols && nkept + 32 <= BWD2_COLS) {
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
}

__device__ __forceinline__ void red_add_v4(float* p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}

// Sweep over the compacted columns of a footprint with the lanes laid out as (column, z-quad): ZQ
// lanes along z hold one aligned quad each, 32/ZQ columns per step.  A lane's z terms live in
// registers for the whole item, and the lanes of a column touch neighbouring 16-byte pieces of one
// line, so a warp's reduction reaches 32/ZQ rows instead of 32 (the scatter kernels are bound by the
// number of distinct lines their reductions touch).  `quad(i, dxy2, exy, d2v, ev, dzv, off)` is called
// by every lane whose quad can hold a voxel of the item: i = column slot, off = row*dim + z of the quad.
template <int ZQ, class BUF, class QuadFn>
__device__ __forceinline__ void qlane_sweep(const ItemParams& P, const BUF& buf, unsigned nkept, size_t dim,
                                            float oz, float res, float kexp, float Tcull, int lane,
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
      ev[j] = ex2_approx(d2v[j] * kexp);
      lo = fminf(lo, d2v[j]);  // fminf skips the NaN entries
    }
    const size_t zoff = zc + 4 * zq;
    for (unsigned c0 = 0; c0 < nkept; c0 += CPI) {
      unsigned i = c0 + cl;
      float dxy2 = i < nkept ? buf.dxy2[i] : CUDART_NAN_F;
      if (!(__fadd_rn(dxy2, lo) <= Tcull)) continue;  // also false for NaN: no column, or no z in range
      quad(i, dxy2, ex2_approx(dxy2 * kexp), d2v, ev, dzv, (size_t)buf.row[i] * dim + zoff);
    }
  }
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
    if (quad_span(P) <= 4) qlane_sweep<4>(P, buf, nkept, dim, oz, gm.res, kexp, P.Tcut, lane, quad);
    else qlane_sweep<8>(P, buf, nkept, dim, oz, gm.res, kexp, P.Tcut, lane, quad);
    __syncwarp();
  }
}

template <bool VEC>
__global__ void __launch_bounds__(SCAT_WARPS * 32) k_forward_quads(BwdArgs G) {
  __shared__ ColBuf bufs[SCAT_WARPS];
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  int item = blockIdx.x * SCAT_WARPS + wid;
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
  const float k4 = 4.f * P.inv_ar2, kD = -gm.D * P.inv_ar2, kE = -gm.E * P.inv_ar;
  const float ta = gm.ta, ntb = -gm.tb;

  if (P.valid) {
    unsigned nx = P.hix - P.lox, ny = P.hiy - P.loy;
    unsigned ncols = nx * ny;
    float inv_ny = 1.f / (float)ny;
    for (unsigned cbase = 0; cbase < ncols;) {
      unsigned nkept = compact_columns<ColBufD, true>(buf, P, cbase, ncols, ny, inv_ny, Tcull, ox, oy,
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
          for (unsigned q0 = 0; q0 < nq; q0 += 4) {
            // up to four quads of the column are requested together, then used
            float4 dv[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
              dv[u] = make_float4(0.f, 0.f, 0.f, 0.f);
              if (q0 + u < nq) {
                float4 d2 = zt.dz2[q0 + u];
                float lo = fminf(fminf(d2.x, d2.y), fminf(d2.z, d2.w));  // fminf skips the NaN entries
                if (__fadd_rn(dxy2, lo) <= Tcull) dv[u] = __ldg(row + q0 + u);
              }
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
                  float lo = fminf(fminf(d2.x, d2.y), fminf(d2.z, d2.w));
                  if (__fadd_rn(dxy2, lo) <= Tcull) {
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
                    float sg = rsq <= P.Tg ? exy4 * ev[j] : fmaf(kE, rsqrt_approx(rsq), kD);
                    float f = (want_ag && rsq <= P.Tcut) ? sg * dvv[j] : 0.f;
                    fsum += f;
                    agz = fmaf(f, dzv[j], agz);
                  }
                  if (MODE == 1) {
                    float v;
                    if (BINARY) {
                      v = rsq < P.Tbin ? 1.f : 0.f;
                    } else {
                      float tq = fminf(fmaf(ta, sqrt_approx(rsq * P.inv_ar2), ntb), 0.f);
                      v = rsq <= P.Tg ? g : tq * tq;
                      v = rsq <= P.Tcut ? v : 0.f;
                    }
                    tg = fmaf(v, dvv[j], tg);
                  }
                  if (MODE == 2) {
                    float v = BINARY ? (rsq < P.Tbin ? 1.f : 0.f)
                                     : density_precise(rsq, P.ar, P.Tg, P.Tcut, gm.A, gm.B, gm.C);
                    if (v > 0.f && dev[j] > 0.f) tg += __fdiv_rn(__fmul_rn(dvv[j], v), dev[j]);
                  }
                  if (MODE == 3) {
                    if (rsq <= P.Tcut) {
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
                      float dzj = dzv[j], dvj = dvv[j];
                      float dot = fmaf(dzj, inz, dotxy);
                      float wa = P.w * alpha * dot;
                      float wb = P.w * beta;
                      float tt = alpha * intg;
                      float bt = beta * intg;
                      agx = fmaf(dvj, fmaf(wa, dx, fmaf(wb, inx, fmaf(tt, dx * dx, bt))), agx);
                      agy = fmaf(dvj, fmaf(wa, dy, fmaf(wb, iny, fmaf(tt, dy * dy, bt))), agy);
                      agz = fmaf(dvj, fmaf(wa, dzj, fmaf(wb, inz, fmaf(tt, dzj * dzj, bt))), agz);
                    }
                  }
                }
              }
            }
          }
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
__global__ void __launch_bounds__(SCAT_WARPS * 32) k_forward_quads_atom(BwdArgs G) {
  __shared__ ColBuf bufs[SCAT_WARPS];
  __shared__ ZTabs ztabs[SCAT_WARPS];
  __shared__ int nz_t[SCAT_WARPS][VA_CH];
  __shared__ float nz_w[SCAT_WARPS][VA_CH];
  const GMParams& gm = G.gm;
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  int item = blockIdx.x * SCAT_WARPS + wid;
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
          if (quad_span(P) <= 4) qlane_sweep<4>(P, buf, nkept, dim, oz, gm.res, kexp, Tcull, lane, quad);
          else qlane_sweep<8>(P, buf, nkept, dim, oz, gm.res, kexp, Tcull, lane, quad);
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
// A lane keeps the type gradients of a round's channels in registers; rounds of VA_BCH channels.
constexpr int VA_BCH = 16;

template <bool BINARY>
__global__ void __launch_bounds__(BWD2_WARPS * 32) k_backward_quads_atom(BwdArgs G) {
  __shared__ ColBufD bufs[BWD2_WARPS];
  __shared__ ZTabs ztabs[BWD2_WARPS];
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
  const float Tcull = fmaxf(P.Tcut, BINARY ? P.Tbin : -1.f);
  const float kexp = P.inv_ar2 * NEG2_LOG2E;
  const float k4 = 4.f * P.inv_ar2, kD = -gm.D * P.inv_ar2, kE = -gm.E * P.inv_ar;
  const float ta = gm.ta, ntb = -gm.tb;
  float agx = 0.f, agy = 0.f, agz = 0.f;

  for (int tb = 0; tb < G.T; tb += VA_BCH) {
    const int nch = min(VA_BCH, G.T - tb);
    float wch[VA_BCH], tgacc[VA_BCH];
#pragma unroll
    for (int c = 0; c < VA_BCH; c++) {
      wch[c] = c < nch ? wrow[tb + c] : 0.f;
      tgacc[c] = 0.f;
    }
    if (P.valid) {
      unsigned nx = P.hix - P.lox, ny = P.hiy - P.loy;
      unsigned ncols = nx * ny;
      float inv_ny = 1.f / (float)ny;
      for (unsigned cbase = 0; cbase < ncols;) {
        unsigned nkept = compact_columns<ColBufD, true>(buf, P, cbase, ncols, ny, inv_ny, Tcull, ox, oy,
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
            const float* row = diffb + (size_t)(have ? buf.row[i] : 0u) * dim + zc;
            float exy = ex2_approx(dxy2 * kexp);
            float fsum = 0.f;
            for (unsigned q = 0; q < nq; q++) {
              float4 d2 = zt.dz2[q], e = zt.ez[q], dz = zt.dz[q];
              float lo = fminf(fminf(d2.x, d2.y), fminf(d2.z, d2.w));  // fminf skips the NaN entries
              if (!(__fadd_rn(dxy2, lo) <= Tcull)) continue;            // no voxel of this lane's quad
              float d2v[4] = {d2.x, d2.y, d2.z, d2.w}, ev[4] = {e.x, e.y, e.z, e.w};
              float dzv[4] = {dz.x, dz.y, dz.z, dz.w};
              float v[4], sg[4], dsum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
              for (int j = 0; j < 4; j++) {
                float rsq = __fadd_rn(dxy2, d2v[j]);
                float g = exy * ev[j];
                float s1 = rsq <= P.Tg ? k4 * g : fmaf(kE, rsqrt_approx(rsq), kD);
                sg[j] = rsq <= P.Tcut ? s1 : 0.f;
                if (BINARY) {
                  v[j] = rsq < P.Tbin ? 1.f : 0.f;
                } else {
                  float tq = fminf(fmaf(ta, sqrt_approx(rsq * P.inv_ar2), ntb), 0.f);
                  float val = rsq <= P.Tg ? g : tq * tq;
                  v[j] = rsq <= P.Tcut ? val : 0.f;
                }
              }
              const float4* qp = reinterpret_cast<const float4*>(row) + q;
#pragma unroll
              for (int c4 = 0; c4 < VA_BCH; c4 += 4) {
                // four channels requested together, then used
                float4 dv[4];
#pragma unroll
                for (int u = 0; u < 4; u++)
                  dv[u] = (c4 + u < nch) ? __ldg(qp + (size_t)(tb + c4 + u) * (chan_stride / 4))
                                         : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int u = 0; u < 4; u++) {
                  float wk = wch[c4 + u];
                  tgacc[c4 + u] = fmaf(v[0], dv[u].x, fmaf(v[1], dv[u].y, fmaf(v[2], dv[u].z,
                                       fmaf(v[3], dv[u].w, tgacc[c4 + u]))));
                  dsum[0] = fmaf(wk, dv[u].x, dsum[0]);
                  dsum[1] = fmaf(wk, dv[u].y, dsum[1]);
                  dsum[2] = fmaf(wk, dv[u].z, dsum[2]);
                  dsum[3] = fmaf(wk, dv[u].w, dsum[3]);
                }
              }
#pragma unroll
              for (int j = 0; j < 4; j++) {
                float f = sg[j] * dsum[j];
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
            float lo = fminf(fminf(d2.x, d2.y), fminf(d2.z, d2.w));  // fminf skips the NaN entries
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
__global__ void __launch_bounds__(SCAT_WARPS * 32) k_gradgrad_quads_atom(BwdArgs G) {
  __shared__ ColBufD bufs[SCAT_WARPS];
  __shared__ ZTabs ztabs[SCAT_WARPS];
  __shared__ int nz_t[SCAT_WARPS][VA_CH];
  __shared__ float nz_w[SCAT_WARPS][VA_CH], nz_g[SCAT_WARPS][VA_CH];
  const GMParams& gm = G.gm;
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  int item = blockIdx.x * SCAT_WARPS + wid;
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
            float lo = fminf(fminf(d2.x, d2.y), fminf(d2.z, d2.w));  // fminf skips the NaN entries
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

cudaError_t launch_scan_fill(const EmitArgs& A, cudaStream_t st) {
  k_scan<<<A.nb, 1024, 0, st>>>(A.cnt, A.M);
  int n = A.nb * A.N;
  k_fill<<<(n + 255) / 256, 256, 0, st>>>(A);
  return cudaGetLastError();
}

template <bool BINARY, bool PRECISE>
static void launch_forward_t(const FwdArgs& F, dim3 grid, cudaStream_t st) {
  if (F.vec) {
    k_forward_vector<BINARY, PRECISE, false><<<grid, FWD_WARPS * 32, 0, st>>>(F);
  } else {
    dim3 gidx(F.nrx * F.nry * F.nrz, F.nb);
    k_forward_index<BINARY, PRECISE><<<gidx, FWD_INDEX_WARPS * 32, 0, st>>>(F);
    dim3 gbig(min(F.N, 32), F.nb);
    k_forward_big<BINARY, PRECISE><<<gbig, 128, 0, st>>>(F);
  }
}

cudaError_t launch_forward(const FwdArgs& F, cudaStream_t st) {
  int nreg = F.nrx * F.nry * F.nrz;
  dim3 grid((nreg + FWD_WARPS - 1) / FWD_WARPS, F.nb);
  if (F.gradgrad) {
    k_forward_vector<false, false, true><<<grid, FWD_WARPS * 32, 0, st>>>(F);
    return cudaGetLastError();
  }
  if (F.gm.binary)
    launch_forward_t<true, false>(F, grid, st);
  else if (F.precise)
    launch_forward_t<false, true>(F, grid, st);
  else
    launch_forward_t<false, false>(F, grid, st);
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
    if (G.type_gradients == nullptr) k_backward_quads_atom_ag<<<ga, BWD2_WARPS * 32, 0, st>>>(G);
    else if (bin) k_backward_quads_atom<true><<<ga, BWD2_WARPS * 32, 0, st>>>(G);
    else k_backward_quads_atom<false><<<ga, BWD2_WARPS * 32, 0, st>>>(G);
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
    dim3 ga((unsigned)((G.N + SCAT_WARPS - 1) / SCAT_WARPS), G.nb);
    k_gradgrad_quads_atom<<<ga, SCAT_WARPS * 32, 0, st>>>(G);
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
    dim3 ga((unsigned)((G.N + SCAT_WARPS - 1) / SCAT_WARPS), G.nb);
    if (bin) k_forward_quads_atom<true, false><<<ga, SCAT_WARPS * 32, 0, st>>>(G);
    else if (G.precise) k_forward_quads_atom<false, true><<<ga, SCAT_WARPS * 32, 0, st>>>(G);
    else k_forward_quads_atom<false, false><<<ga, SCAT_WARPS * 32, 0, st>>>(G);
    return cudaGetLastError();
  }
  if (G.quads && !bin && !G.precise && G.gm.dim % 4 == 0 && (uintptr_t)G.out_grid % 16 == 0) {
    if (vec) {
      // radii by channel: one warp per atom runs the items of its weighted channels
      dim3 ga((unsigned)(((long)G.N * nz_groups(G.T) + SCAT_WARPS - 1) / SCAT_WARPS), G.nb);
      k_forward_quads_nz<<<ga, SCAT_WARPS * 32, 0, st>>>(G);
      return cudaGetLastError();
    }
    k_forward_quads<false><<<grid, SCAT_WARPS * 32, 0, st>>>(G);
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

}  // namespace lmg
