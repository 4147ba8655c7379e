/* TEST INFRASTRUCTURE ONLY - never linked into or called from the product library.
 *
 * Plain-C restatement of the CPU algorithm of libmolgrid's gridding path, used as
 * the parity checker for the CUDA kernels.  Each function names the reference
 * file:line it follows (paths relative to the libmolgrid tree).  The arithmetic is
 * kept operation for operation (float vs double intermediates, evaluation order,
 * no fused multiply-add: build with -ffp-contract=off) so that results are
 * bit-identical to the reference's own CPU build; tests/test_oracle.py pins that
 * against the compiled reference (oracle/_ref) and against the committed golden
 * vectors under tests/golden/.
 *
 * Return codes mirror the reference's exceptions: 0 ok, 1 std::out_of_range,
 * 2 std::invalid_argument.  lmgo_last_error() gives a message.
 */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

static __thread char g_err[256];

const char* lmgo_last_error(void) { return g_err; }

static int fail(int code, const char* msg) {
  snprintf(g_err, sizeof g_err, "%s", msg);
  return code;
}

/* GridMaker state: include/libmolgrid/grid_maker.h:36-48 */
typedef struct {
  float resolution, dimension, radius_scale, gaussian_radius_multiple, final_radius_multiple;
  float A, B, C, D, E;
  int binary, radii_type_indexed;
  unsigned dim;
} gridmaker;

/* GridMaker::initialize, src/grid_maker.cpp:15-36.
 * Note the quirk kept here: when grm < 0 the stored multiple becomes |grm| but the
 * coefficient expressions below still use the caller's (negative) grm.
 * Unqualified exp() on a float argument resolves to the double function there. */
static void gm_init(gridmaker* g, const float* p) {
  float res = p[0], d = p[1], rscale = p[4], grm = p[5];
  g->resolution = res;
  g->dimension = d;
  g->binary = p[2] != 0;
  g->radii_type_indexed = p[3] != 0;
  g->radius_scale = rscale;
  g->gaussian_radius_multiple = grm;
  if (g->gaussian_radius_multiple < 0) {
    g->gaussian_radius_multiple *= -1;
    g->final_radius_multiple = g->gaussian_radius_multiple;
  } else {
    g->final_radius_multiple = (1 + 2 * grm * grm) / (2 * grm);
  }
  g->dim = (unsigned)(roundf(d / res) + 1);
  g->A = exp(-2 * grm * grm) * 4 * grm * grm;
  g->B = -exp(-2 * grm * grm) * (4 * grm + 8 * grm * grm * grm);
  g->C = exp(-2 * grm * grm) * (4 * grm * grm * grm * grm + 4 * grm * grm + 1);
  g->D = 8 * grm * grm * exp(-2.0 * grm * grm);
  g->E = -(4 * grm + 8 * grm * grm * grm) * exp(-2 * grm * grm);
}

int lmgo_consts(const float* gmp, float* out8) {
  gridmaker g;
  gm_init(&g, gmp);
  out8[0] = g.A; out8[1] = g.B; out8[2] = g.C; out8[3] = g.D; out8[4] = g.E;
  out8[5] = g.final_radius_multiple; out8[6] = (float)g.dim; out8[7] = g.gaussian_radius_multiple;
  return 0;
}

/* GridMaker::get_grid_origin, src/grid_maker.cpp:100-107 */
static void grid_origin(const gridmaker* g, const float* center, float* o) {
  float half = g->dimension / 2.0;
  o[0] = center[0] - half;
  o[1] = center[1] - half;
  o[2] = center[2] - half;
}

/* GridMaker::get_bounds_1d, src/grid_maker.cu:66-79: half-open [lo, hi) voxel range */
static void bounds_1d(const gridmaker* g, float origin, float coord, float densityrad,
                      unsigned* lo, unsigned* hi) {
  *lo = 0;
  *hi = 0;
  float low = coord - densityrad - origin;
  if (low > 0) *lo = (unsigned)floorf(low / g->resolution);
  float high = coord + densityrad - origin;
  if (high > 0) {
    unsigned c = (unsigned)ceilf(high / g->resolution);
    *hi = g->dim < c ? g->dim : c;
  }
}

/* sqDistance, src/grid_maker.cu:82-92: grid point minus atom, summed x then y then z */
static float sq_distance(float gx, float gy, float gz, float x, float y, float z) {
  float ret;
  float tmp = gx - x;
  ret = tmp * tmp;
  tmp = gy - y;
  ret += tmp * tmp;
  tmp = gz - z;
  ret += tmp * tmp;
  return ret;
}

/* GridMaker::calc_point<false>, src/grid_maker.cu:95-118 */
static float calc_point_density(const gridmaker* g, float ax, float ay, float az, float ar,
                                float gx, float gy, float gz) {
  float rsq = sq_distance(gx, gy, gz, ax, ay, az);
  ar *= g->radius_scale;
  float dist = sqrtf(rsq);
  if (dist > ar * g->final_radius_multiple) {
    return 0.0;
  } else if (dist <= ar * g->gaussian_radius_multiple) {
    float ex = -2.0 * dist * dist / (ar * ar);
    return expf(ex);
  } else {
    float dr = dist / ar;
    float q = (g->A * dr + g->B) * dr + g->C;
    return q > 0 ? q : 0;
  }
}

/* GridMaker::calc_point<true>, src/grid_maker.cu:120-130 */
static float calc_point_binary(const gridmaker* g, float ax, float ay, float az, float ar,
                               float gx, float gy, float gz) {
  float rsq = sq_distance(gx, gy, gz, ax, ay, az);
  ar *= g->radius_scale;
  if (rsq < ar * ar) return 1.0;
  return 0.0;
}

static int check_dims(const gridmaker* g, unsigned n, unsigned ntypes) {
  (void)g; (void)n; (void)ntypes;
  return 0;
}

/* CPU forward, index types: src/grid_maker.cpp:153-212 */
int lmgo_forward_index(const float* gmp, const float* center, unsigned n, const float* coords,
                       const float* types, const float* radii, unsigned ntypes, float* out) {
  gridmaker g;
  gm_init(&g, gmp);
  size_t dim = g.dim;
  memset(out, 0, sizeof(float) * ntypes * dim * dim * dim);
  if (check_dims(&g, n, ntypes)) return 1;
  if (g.radii_type_indexed) return fail(2, "Type indexed radii not supported with index types.");
  float o[3];
  grid_origin(&g, center, o);
  for (size_t a = 0; a < n; a++) {
    int64_t atype = (int64_t)floorf(types[a]);
    if (atype >= (int64_t)ntypes) return fail(1, "Type index larger than allowed");
    if (atype >= 0 && atype < (int64_t)ntypes) {
      float ax = coords[3 * a], ay = coords[3 * a + 1], az = coords[3 * a + 2];
      float radius = radii[a];
      float densityrad = radius * g.radius_scale * g.final_radius_multiple;
      unsigned lo[3], hi[3];
      bounds_1d(&g, o[0], ax, densityrad, &lo[0], &hi[0]);
      bounds_1d(&g, o[1], ay, densityrad, &lo[1], &hi[1]);
      bounds_1d(&g, o[2], az, densityrad, &lo[2], &hi[2]);
      for (size_t i = lo[0]; i < hi[0]; i++) {
        for (size_t j = lo[1]; j < hi[1]; j++) {
          for (size_t k = lo[2]; k < hi[2]; k++) {
            float gx = o[0] + i * g.resolution;
            float gy = o[1] + j * g.resolution;
            float gz = o[2] + k * g.resolution;
            size_t off = (((atype * dim) + i) * dim + j) * dim + k;
            if (g.binary) {
              float val = calc_point_binary(&g, ax, ay, az, radius, gx, gy, gz);
              if (val != 0) out[off] = 1.0;
            } else {
              float val = calc_point_density(&g, ax, ay, az, radius, gx, gy, gz);
              out[off] += val;
            }
          }
        }
      }
    }
  }
  return 0;
}

/* check_vector_args, src/grid_maker.cpp:67-88 (the radii size rule) */
static int check_vector_radii(const gridmaker* g, unsigned n, unsigned ntypes, unsigned nradii) {
  if (g->radii_type_indexed) {
    if (nradii != ntypes) return fail(1, "radii does not match number of types");
  } else {
    if (nradii != n) return fail(1, "radii does not match number of atoms");
  }
  return 0;
}

/* CPU forward, vector types: src/grid_maker.cpp:214-271 */
int lmgo_forward_vector(const float* gmp, const float* center, unsigned n, unsigned ntypes,
                        const float* coords, const float* tv, const float* radii, unsigned nradii,
                        float* out) {
  gridmaker g;
  gm_init(&g, gmp);
  size_t dim = g.dim;
  memset(out, 0, sizeof(float) * ntypes * dim * dim * dim);
  if (check_vector_radii(&g, n, ntypes, nradii)) return 1;
  float o[3];
  grid_origin(&g, center, o);
  for (size_t a = 0; a < n; a++) {
    for (size_t t = 0; t < ntypes; t++) {
      float tmult = tv[a * ntypes + t];
      if (tmult != 0) {
        float ax = coords[3 * a], ay = coords[3 * a + 1], az = coords[3 * a + 2];
        float radius = g.radii_type_indexed ? radii[t] : radii[a];
        float densityrad = radius * g.radius_scale * g.final_radius_multiple;
        unsigned lo[3], hi[3];
        bounds_1d(&g, o[0], ax, densityrad, &lo[0], &hi[0]);
        bounds_1d(&g, o[1], ay, densityrad, &lo[1], &hi[1]);
        bounds_1d(&g, o[2], az, densityrad, &lo[2], &hi[2]);
        for (size_t i = lo[0]; i < hi[0]; i++) {
          for (size_t j = lo[1]; j < hi[1]; j++) {
            for (size_t k = lo[2]; k < hi[2]; k++) {
              float gx = o[0] + i * g.resolution;
              float gy = o[1] + j * g.resolution;
              float gz = o[2] + k * g.resolution;
              size_t off = (((t * dim) + i) * dim + j) * dim + k;
              if (g.binary) {
                float val = calc_point_binary(&g, ax, ay, az, radius, gx, gy, gz);
                if (val != 0) out[off] += tmult;
              } else {
                float val = calc_point_density(&g, ax, ay, az, radius, gx, gy, gz);
                out[off] += val * tmult;
              }
            }
          }
        }
      }
    }
  }
  return 0;
}

/* GridMaker::density_grad_dist, src/grid_maker.cu:881-896 (ar already includes radius_scale) */
static float density_grad_dist(const gridmaker* g, float dist, float ar) {
  float agrad_dist = 0.0;
  float dist2 = dist * dist;
  if (dist > ar * g->final_radius_multiple) {
    return NAN;
  } else if (dist <= ar * g->gaussian_radius_multiple) {
    float ex = -2.0 * dist2 / (ar * ar);
    float coef = -4.0 * dist / (ar * ar);
    agrad_dist = coef * expf(ex);
  } else {
    agrad_dist = (g->D * dist / ar + g->E) / ar;
  }
  return agrad_dist;
}

/* GridMaker::accumulate_atom_gradient, src/grid_maker.cu:898-919 */
static void accumulate_atom_gradient(const gridmaker* g, float ax, float ay, float az, float x,
                                     float y, float z, float ar, float gridval, float* agrad) {
  float dist_x = x - ax;
  float dist_y = y - ay;
  float dist_z = z - az;
  float dist2 = dist_x * dist_x + dist_y * dist_y + dist_z * dist_z;
  /* this file is compiled by nvcc there, whose host pass resolves sqrt(float) to the
   * single-precision overload; the result is then widened to double */
  double dist = sqrtf(dist2);
  ar *= g->radius_scale;
  float agrad_dist = density_grad_dist(g, dist, ar);
  if (dist > 0 && isfinite(agrad_dist)) {
    agrad[0] += -(dist_x / dist) * (agrad_dist * gridval);
    agrad[1] += -(dist_y / dist) * (agrad_dist * gridval);
    agrad[2] += -(dist_z / dist) * (agrad_dist * gridval);
  }
}

/* GridMaker::calc_atom_gradient_cpu, src/grid_maker.cpp:325-354 */
static void calc_atom_gradient(const gridmaker* g, const float* o, const float* a,
                               const float* diff /* one channel */, float radius, float* agrad) {
  agrad[0] = agrad[1] = agrad[2] = 0;
  float r = radius * g->radius_scale * g->final_radius_multiple;
  unsigned lo[3], hi[3];
  size_t dim = g->dim;
  bounds_1d(g, o[0], a[0], r, &lo[0], &hi[0]);
  bounds_1d(g, o[1], a[1], r, &lo[1], &hi[1]);
  bounds_1d(g, o[2], a[2], r, &lo[2], &hi[2]);
  for (unsigned i = lo[0]; i < hi[0]; ++i)
    for (unsigned j = lo[1]; j < hi[1]; ++j)
      for (unsigned k = lo[2]; k < hi[2]; ++k) {
        float x = o[0] + i * g->resolution;
        float y = o[1] + j * g->resolution;
        float z = o[2] + k * g->resolution;
        accumulate_atom_gradient(g, a[0], a[1], a[2], x, y, z, radius,
                                 diff[(i * dim + j) * dim + k], agrad);
      }
}

/* GridMaker::calc_type_gradient_cpu, src/grid_maker.cpp:357-389 */
static float calc_type_gradient(const gridmaker* g, const float* o, const float* a,
                                const float* diff, float radius) {
  float r = radius * g->radius_scale * g->final_radius_multiple;
  unsigned lo[3], hi[3];
  size_t dim = g->dim;
  bounds_1d(g, o[0], a[0], r, &lo[0], &hi[0]);
  bounds_1d(g, o[1], a[1], r, &lo[1], &hi[1]);
  bounds_1d(g, o[2], a[2], r, &lo[2], &hi[2]);
  float ret = 0;
  for (unsigned i = lo[0]; i < hi[0]; ++i)
    for (unsigned j = lo[1]; j < hi[1]; ++j)
      for (unsigned k = lo[2]; k < hi[2]; ++k) {
        float x = o[0] + i * g->resolution;
        float y = o[1] + j * g->resolution;
        float z = o[2] + k * g->resolution;
        float val = g->binary ? calc_point_binary(g, a[0], a[1], a[2], radius, x, y, z)
                              : calc_point_density(g, a[0], a[1], a[2], radius, x, y, z);
        ret += val * diff[(i * dim + j) * dim + k];
      }
  return ret;
}

/* CPU backward, index types: src/grid_maker.cpp:436-467 */
int lmgo_backward_index(const float* gmp, const float* center, unsigned n, const float* coords,
                        const float* types, const float* radii, unsigned ntypes, const float* diff,
                        float* atom_gradients) {
  gridmaker g;
  gm_init(&g, gmp);
  memset(atom_gradients, 0, sizeof(float) * 3 * n);
  if (g.radii_type_indexed) return fail(2, "Type indexed radii not supported with index types.");
  float o[3];
  grid_origin(&g, center, o);
  size_t chan = (size_t)g.dim * g.dim * g.dim;
  for (unsigned i = 0; i < n; ++i) {
    int whichgrid = (int)roundf(types[i]);
    if (whichgrid >= 0) {
      if ((unsigned)whichgrid >= ntypes) return fail(2, "Incorrect channel size for diff");
      float ag[3];
      calc_atom_gradient(&g, o, coords + 3 * i, diff + chan * whichgrid, radii[i], ag);
      atom_gradients[3 * i] = ag[0];
      atom_gradients[3 * i + 1] = ag[1];
      atom_gradients[3 * i + 2] = ag[2];
    }
  }
  return 0;
}

/* CPU backward, vector types: src/grid_maker.cpp:477-519 */
int lmgo_backward_vector(const float* gmp, const float* center, unsigned n, unsigned ntypes,
                         const float* coords, const float* tv, const float* radii, unsigned nradii,
                         const float* diff, float* atom_gradients, float* type_gradients) {
  gridmaker g;
  gm_init(&g, gmp);
  memset(atom_gradients, 0, sizeof(float) * 3 * n);
  memset(type_gradients, 0, sizeof(float) * (size_t)ntypes * n);
  if (g.radii_type_indexed) {
    if (ntypes != nradii) return fail(2, "Radii dimension doesn't equal number of types");
  } else {
    if (n != nradii) return fail(2, "Radii dimension doesn't equal number of coordinates");
  }
  float o[3];
  grid_origin(&g, center, o);
  size_t chan = (size_t)g.dim * g.dim * g.dim;
  for (unsigned i = 0; i < n; ++i) {
    float radius = 0;
    if (!g.radii_type_indexed) radius = radii[i];
    for (unsigned t = 0; t < ntypes; t++) {
      float tmult = tv[(size_t)i * ntypes + t];
      if (g.radii_type_indexed) radius = radii[t];
      if (tmult != 0) {
        float ag[3];
        calc_atom_gradient(&g, o, coords + 3 * i, diff + chan * t, radius, ag);
        atom_gradients[3 * i] += ag[0] * tmult;
        atom_gradients[3 * i + 1] += ag[1] * tmult;
        atom_gradients[3 * i + 2] += ag[2] * tmult;
      }
      type_gradients[(size_t)i * ntypes + t] =
          calc_type_gradient(&g, o, coords + 3 * i, diff + chan * t, radius);
    }
  }
  return 0;
}

/* GridMaker::calc_atom_relevance_cpu, src/grid_maker.cpp:391-433; backward_relevance :684-704 */
int lmgo_backward_relevance(const float* gmp, const float* center, unsigned n, const float* coords,
                            const float* types, const float* radii, unsigned ntypes,
                            const float* density, const float* diff, float* relevance) {
  gridmaker g;
  gm_init(&g, gmp);
  (void)ntypes;
  memset(relevance, 0, sizeof(float) * n);
  float o[3];
  grid_origin(&g, center, o);
  size_t dim = g.dim, chan = dim * dim * dim;
  for (unsigned a = 0; a < n; ++a) {
    int whichgrid = (int)roundf(types[a]);
    if (whichgrid < 0) continue;
    const float* c = coords + 3 * a;
    const float* den = density + chan * whichgrid;
    const float* dif = diff + chan * whichgrid;
    float radius = radii[a];
    float ret = 0;
    float r = radius * g.radius_scale * g.final_radius_multiple;
    unsigned lo[3], hi[3];
    bounds_1d(&g, o[0], c[0], r, &lo[0], &hi[0]);
    bounds_1d(&g, o[1], c[1], r, &lo[1], &hi[1]);
    bounds_1d(&g, o[2], c[2], r, &lo[2], &hi[2]);
    for (unsigned i = lo[0]; i < hi[0]; ++i)
      for (unsigned j = lo[1]; j < hi[1]; ++j)
        for (unsigned k = lo[2]; k < hi[2]; ++k) {
          float x = o[0] + i * g.resolution;
          float y = o[1] + j * g.resolution;
          float z = o[2] + k * g.resolution;
          float val = g.binary ? calc_point_binary(&g, c[0], c[1], c[2], radius, x, y, z)
                               : calc_point_density(&g, c[0], c[1], c[2], radius, x, y, z);
          if (val > 0) {
            float denseval = den[(i * dim + j) * dim + k];
            float gridval = dif[(i * dim + j) * dim + k];
            if (denseval > 0) ret += gridval * val / denseval;
          }
        }
    relevance[a] = ret;
  }
  return 0;
}

/* GridMaker::type_grad_grad / atom_density_grad_grad (identical bodies), src/grid_maker.cu:812-856 */
static float density_grad_grad(const gridmaker* g, float a, float x, float dist, float r) {
  float ret = 0.0;
  float dist2 = dist * dist;
  if (dist > r * g->final_radius_multiple) {
    return 0;
  } else if (dist <= r * g->gaussian_radius_multiple) {
    float r2 = r * r;
    float ex = -2.0 * dist2 / r2;
    ret = 16 * (a - x) * (a - x) * expf(ex) / (r2 * r2) - 4 * expf(ex) / (r2);
  } else {
    float ax = a - x;
    float ax2 = ax * ax;
    float term1 = -(g->E + g->D * dist / r) * ax2 / (pow(dist2, 1.5) * r);
    float term2 = g->D * ax2 / (dist2 * r * r);
    float term3 = (g->E + g->D * dist / r) / (dist * r);
    ret = term1 + term2 + term3;
  }
  return ret;
}

/* GridMaker::atom_density_grad_grad_other, src/grid_maker.cu:860-878 */
static float density_grad_grad_other(const gridmaker* g, float a, float x, float b, float y,
                                     float dist, float r) {
  float ret = 0.0;
  float dist2 = dist * dist;
  if (dist > r * g->final_radius_multiple) {
    return 0;
  } else if (dist <= r * g->gaussian_radius_multiple) {
    float r2 = r * r;
    float ex = -2.0 * dist2 / r2;
    ret = 16 * (a - x) * (b - y) * expf(ex) / (r2 * r2);
  } else {
    float ax = a - x;
    float by = b - y;
    float term1 = -(g->E + g->D * dist / r) * ax * by / (pow(dist2, 1.5) * r);
    float term2 = g->D * ax * by / (dist2 * r * r);
    ret = term1 + term2;
  }
  return ret;
}

/* CPU backward_gradients: src/grid_maker.cpp:529-672 */
int lmgo_backward_gradients(const float* gmp, const float* center, unsigned n, unsigned ntypes,
                            const float* coords, const float* tv, const float* radii,
                            unsigned nradii, const float* diff, const float* atom_gradients,
                            const float* type_gradients, float* diffdiff, float* atom_diffdiff,
                            float* type_diffdiff) {
  gridmaker g;
  gm_init(&g, gmp);
  size_t dim = g.dim, chan = dim * dim * dim;
  if (check_vector_radii(&g, n, ntypes, nradii)) return 1;
  if (g.binary) return fail(2, "Binary densities not supported");
  memset(atom_diffdiff, 0, sizeof(float) * 3 * n);
  memset(type_diffdiff, 0, sizeof(float) * (size_t)ntypes * n);
  memset(diffdiff, 0, sizeof(float) * chan * ntypes);
  float o[3];
  grid_origin(&g, center, o);
  for (size_t aidx = 0; aidx < n; ++aidx) {
    for (size_t tidx = 0; tidx < ntypes; tidx++) {
      float tmult = tv[aidx * ntypes + tidx];
      if (tmult != 0) {
        const float* diffG = diff + chan * tidx;
        float ax = coords[3 * aidx], ay = coords[3 * aidx + 1], az = coords[3 * aidx + 2];
        float agx = atom_gradients[3 * aidx], agy = atom_gradients[3 * aidx + 1],
              agz = atom_gradients[3 * aidx + 2];
        float tgrad = type_gradients[aidx * ntypes + tidx];
        float radius = g.radii_type_indexed ? radii[tidx] : radii[aidx];
        float ar = radius * g.radius_scale;
        float densityrad = radius * g.radius_scale * g.final_radius_multiple;
        unsigned lo[3], hi[3];
        bounds_1d(&g, o[0], ax, densityrad, &lo[0], &hi[0]);
        bounds_1d(&g, o[1], ay, densityrad, &lo[1], &hi[1]);
        bounds_1d(&g, o[2], az, densityrad, &lo[2], &hi[2]);
        float addx = 0, addy = 0, addz = 0;
        for (size_t i = lo[0]; i < hi[0]; i++) {
          for (size_t j = lo[1]; j < hi[1]; j++) {
            for (size_t k = lo[2]; k < hi[2]; k++) {
              float x = o[0] + i * g.resolution;
              float y = o[1] + j * g.resolution;
              float z = o[2] + k * g.resolution;
              float G = diffG[(i * dim + j) * dim + k];
              size_t off = (((tidx * dim) + i) * dim + j) * dim + k;
              float dist_x = x - ax;
              float dist_y = y - ay;
              float dist_z = z - az;
              float dist2 = dist_x * dist_x + dist_y * dist_y + dist_z * dist_z;
              double dist = sqrt(dist2);
              float agrad_dist = density_grad_dist(&g, dist, ar);
              if (isfinite(agrad_dist)) {
                float gval = 0.0;
                if (dist > 0) {
                  gval += -(dist_x / dist) * (agrad_dist * agx);
                  gval += -(dist_y / dist) * (agrad_dist * agy);
                  gval += -(dist_z / dist) * (agrad_dist * agz);
                  gval *= tmult;
                }
                float val = calc_point_density(&g, ax, ay, az, radius, x, y, z);
                gval += val * tgrad;
                diffdiff[off] += gval;

                addx += density_grad_grad(&g, ax, x, dist, ar) * G * tmult * agx;
                addx += density_grad_grad_other(&g, ax, x, ay, y, dist, ar) * G * tmult * agy;
                addx += density_grad_grad_other(&g, ax, x, az, z, dist, ar) * G * tmult * agz;
                addx += density_grad_grad(&g, ax, x, dist, ar) * G * tgrad;

                addy += density_grad_grad_other(&g, ay, y, ax, x, dist, ar) * G * tmult * agx;
                addy += density_grad_grad(&g, ay, y, dist, ar) * G * tmult * agy;
                addy += density_grad_grad_other(&g, ay, y, az, z, dist, ar) * G * tmult * agz;
                addy += density_grad_grad(&g, ay, y, dist, ar) * G * tgrad;

                addz += density_grad_grad_other(&g, az, z, ax, x, dist, ar) * G * tmult * agx;
                addz += density_grad_grad_other(&g, az, z, ay, y, dist, ar) * G * tmult * agy;
                addz += density_grad_grad(&g, az, z, dist, ar) * G * tmult * agz;
                addz += density_grad_grad(&g, az, z, dist, ar) * G * tgrad;
              }
            }
          }
        }
        atom_diffdiff[3 * aidx] += addx;
        atom_diffdiff[3 * aidx + 1] += addy;
        atom_diffdiff[3 * aidx + 2] += addz;
      }
    }
  }
  return 0;
}

/* ---- Quaternion, include/libmolgrid/quaternion.h:17-167 (all float, left to right) ---- */
typedef struct { float a, b, c, d; } quat;

/* operator*, quaternion.h:82-91 */
static quat q_mul(quat l, quat r) {
  quat o;
  o.a = +l.a * r.a - l.b * r.b - l.c * r.c - l.d * r.d;
  o.b = +l.a * r.b + l.b * r.a + l.c * r.d - l.d * r.c;
  o.c = +l.a * r.c - l.b * r.d + l.c * r.a + l.d * r.b;
  o.d = +l.a * r.d + l.b * r.c - l.c * r.b + l.d * r.a;
  return o;
}

/* operator/(Quaternion), quaternion.h:106-120 */
static quat q_div(quat l, quat r) {
  float den = r.a * r.a + r.b * r.b + r.c * r.c + r.d * r.d;
  quat o;
  o.a = (+l.a * r.a + l.b * r.b + l.c * r.c + l.d * r.d) / den;
  o.b = (-l.a * r.b + l.b * r.a - l.c * r.d + l.d * r.c) / den;
  o.c = (-l.a * r.c + l.b * r.d + l.c * r.a - l.d * r.b) / den;
  o.d = (-l.a * r.d - l.b * r.c + l.c * r.b + l.d * r.a) / den;
  return o;
}

/* inverse, quaternion.h:163-166 */
static quat q_inverse(quat q) {
  float nsq = q.a * q.a + q.b * q.b + q.c * q.c + q.d * q.d;
  quat o = {q.a / nsq, -q.b / nsq, -q.c / nsq, -q.d / nsq};
  return o;
}

/* rotate, quaternion.h:145-149: this * p * (conj() / norm()) */
static void q_rotate(quat q, float x, float y, float z, float* out) {
  quat p = {0, x, y, z};
  float norm = q.a * q.a + q.b * q.b + q.c * q.c + q.d * q.d;
  quat cn = {q.a / norm, -q.b / norm, -q.c / norm, -q.d / norm};
  p = q_mul(q_mul(q, p), cn);
  out[0] = p.b;
  out[1] = p.c;
  out[2] = p.d;
}

/* transform, quaternion.h:152-159 */
static void q_transform(quat q, float x, float y, float z, const float* center,
                        const float* translate, float* out) {
  float pt[3];
  q_rotate(q, x - center[0], y - center[1], z - center[2], pt);
  out[0] = pt[0] + center[0] + translate[0];
  out[1] = pt[1] + center[1] + translate[1];
  out[2] = pt[2] + center[2] + translate[2];
}

int lmgo_quaternion_ops(const float* qa, const float* qb, const float* pt, float* out15) {
  quat a = {qa[0], qa[1], qa[2], qa[3]}, b = {qb[0], qb[1], qb[2], qb[3]};
  quat r[3] = {q_mul(a, b), q_div(a, b), q_inverse(a)};
  for (int i = 0; i < 3; i++) {
    out15[4 * i] = r[i].a; out15[4 * i + 1] = r[i].b;
    out15[4 * i + 2] = r[i].c; out15[4 * i + 3] = r[i].d;
  }
  q_rotate(a, pt[0], pt[1], pt[2], out15 + 12);
  return 0;
}

/* Transform::forward (CPU), src/transform.cpp:57-79; tr = {q[4], center[3], translate[3]} */
int lmgo_transform_forward(const float* tr, unsigned n, const float* in, float* out,
                           int dotranslate) {
  quat q = {tr[0], tr[1], tr[2], tr[3]};
  const float zero[3] = {0, 0, 0};
  for (unsigned i = 0; i < n; i++) {
    float x = in[3 * i], y = in[3 * i + 1], z = in[3 * i + 2];
    float o[3];
    q_transform(q, x, y, z, tr + 4, dotranslate ? tr + 7 : zero, o);
    out[3 * i] = o[0];
    out[3 * i + 1] = o[1];
    out[3 * i + 2] = o[2];
  }
  return 0;
}

/* Transform::backward (CPU), src/transform.cpp:85-108 */
int lmgo_transform_backward(const float* tr, unsigned n, const float* in, float* out,
                            int dotranslate) {
  quat q = {tr[0], tr[1], tr[2], tr[3]};
  quat inv = q_inverse(q);
  const float* c = tr + 4;
  const float* t = tr + 7;
  float un[3];
  if (dotranslate) {
    un[0] = -t[0] - c[0]; un[1] = -t[1] - c[1]; un[2] = -t[2] - c[2];
  } else {
    un[0] = -c[0]; un[1] = -c[1]; un[2] = -c[2];
  }
  for (unsigned i = 0; i < n; i++) {
    float x = in[3 * i] + un[0], y = in[3 * i + 1] + un[1], z = in[3 * i + 2] + un[2];
    float o[3];
    q_rotate(inv, x, y, z, o);
    out[3 * i] = o[0] + c[0];
    out[3 * i + 1] = o[1] + c[1];
    out[3 * i + 2] = o[2] + c[2];
  }
  return 0;
}

/* GridInterpolater::get_pt, src/grid_interpolater.cu:16-22 */
static float get_pt(const float* in, int dim, int x, int y, int z) {
  if (x < 0 || x >= dim || y < 0 || y >= dim || z < 0 || z >= dim) return 0;
  return in[((size_t)x * dim + y) * dim + z];
}

/* GridInterpolater::interpolate, src/grid_interpolater.cu:26-58 */
static float interpolate(const float* in, int dim, float gx, float gy, float gz) {
  int xl = (int)floorf(gx), xh = (int)ceilf(gx);
  int yl = (int)floorf(gy), yh = (int)ceilf(gy);
  int zl = (int)floorf(gz), zh = (int)ceilf(gz);
  float p000 = get_pt(in, dim, xl, yl, zl);
  float p001 = get_pt(in, dim, xl, yl, zh);
  float p010 = get_pt(in, dim, xl, yh, zl);
  float p011 = get_pt(in, dim, xl, yh, zh);
  float p100 = get_pt(in, dim, xh, yl, zl);
  float p101 = get_pt(in, dim, xh, yl, zh);
  float p110 = get_pt(in, dim, xh, yh, zl);
  float p111 = get_pt(in, dim, xh, yh, zh);
  float xd = xh > xl ? (gx - xl) / (xh - xl) : 0;
  float yd = yh > yl ? (gy - yl) / (yh - yl) : 0;
  float zd = zh > zl ? (gz - zl) / (zh - zl) : 0;
  float c00 = p000 * (1 - xd) + p100 * xd;
  float c01 = p001 * (1 - xd) + p101 * xd;
  float c10 = p010 * (1 - xd) + p110 * xd;
  float c11 = p011 * (1 - xd) + p111 * xd;
  float c0 = c00 * (1 - yd) + c10 * yd;
  float c1 = c01 * (1 - yd) + c11 * yd;
  return c0 * (1 - zd) + c1 * zd;
}

/* GridInterpolater::forward (CPU), src/grid_interpolater.cpp:16-48;
 * gi = {in_resolution, in_dimension, out_resolution, out_dimension}, dims per grid_interpolater.h:59-64 */
int lmgo_interpolate(const float* gi, const float* in_center, unsigned nchannels, const float* in,
                     const float* tr, const float* out_center, float* out) {
  float in_res = gi[0], in_dimension = gi[1], out_res = gi[2], out_dimension = gi[3];
  unsigned in_dim = (unsigned)(roundf(in_dimension / in_res) + 1);
  unsigned out_dim = (unsigned)(roundf(out_dimension / out_res) + 1);
  if (in == out) return fail(2, "Input and output grid can not be the same in GridInterpolator.");
  const float* center = tr + 4;
  float in_radius = in_dimension / 2.0;
  float out_radius = out_dimension / 2.0;
  float in_origin[3] = {in_center[0] - in_radius, in_center[1] - in_radius, in_center[2] - in_radius};
  float out_origin[3] = {out_center[0] - out_radius, out_center[1] - out_radius,
                         out_center[2] - out_radius};
  quat q = {tr[0], tr[1], tr[2], tr[3]};
  quat inv = q_inverse(q);
  const float* t = tr + 7;
  float un[3] = {-t[0] - center[0], -t[1] - center[1], -t[2] - center[2]};
  size_t ichan = (size_t)in_dim * in_dim * in_dim, ochan = (size_t)out_dim * out_dim * out_dim;
  for (unsigned i = 0; i < out_dim; i++)
    for (unsigned j = 0; j < out_dim; j++)
      for (unsigned k = 0; k < out_dim; k++) {
        /* grid2cart, grid_interpolater.h:194-198 */
        float ox = out_origin[0] + i * out_res;
        float oy = out_origin[1] + j * out_res;
        float oz = out_origin[2] + k * out_res;
        float np[3];
        q_rotate(inv, ox + un[0], oy + un[1], oz + un[2], np);
        /* cart2grid, grid_interpolater.h:189-192 */
        float gx = (np[0] + center[0] - in_origin[0]) / in_res;
        float gy = (np[1] + center[1] - in_origin[1]) / in_res;
        float gz = (np[2] + center[2] - in_origin[2]) / in_res;
        for (unsigned c = 0; c < nchannels; c++)
          out[c * ochan + ((size_t)i * out_dim + j) * out_dim + k] =
              interpolate(in + c * ichan, (int)in_dim, gx, gy, gz);
      }
  return 0;
}
