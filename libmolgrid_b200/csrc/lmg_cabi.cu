// Host side of the C ABI declared in include/lmg_b200.h: argument checks, workspace carving,
// pass splitting and kernel launches.  Nothing here computes results on the CPU.
#include <cmath>
#include <cstdio>
#include <cstring>
#include <random>
#include <string>
#include <vector>

#include <nvtx3/nvToolsExt.h>

#include "../../include/lmg_b200.h"
#include "lmg_launch.h"
#include "lmg_misc.h"

namespace {

thread_local std::string g_err;
std::default_random_engine g_engine;  // same engine type as libmolgrid::random_engine
int g_precise = -1;                   // -1 auto, 0 fast density, 1 reference-order density
int g_interp_tiled = 1;               // tensor-copy staged interpolation where the input allows it
int g_quads = 1;                      // aligned-quad kernels where the grid allows them

// ---- optional per-kernel timing (bench support; off by default) --------------------------------
// When enabled, the forward and backward kernels of each pass are bracketed by CUDA events on the
// launching stream; lmg_profile_collect() synchronises and returns the summed durations.
struct ProfRec { cudaEvent_t e0, e1; int kind; };
std::vector<ProfRec> g_prof;
size_t g_prof_used = 0;
bool g_prof_on = false;
long g_launches = 0;  // kernels launched by this library since load (memsets not counted)

ProfRec* prof_begin(int kind, cudaStream_t st) {
  if (!g_prof_on || g_prof_used >= g_prof.size()) return nullptr;
  ProfRec* r = &g_prof[g_prof_used++];
  r->kind = kind;
  cudaEventRecord(r->e0, st);
  return r;
}
void prof_end(ProfRec* r, cudaStream_t st) {
  if (r != nullptr) cudaEventRecord(r->e1, st);
}

// A named range on the calling thread for the stages of a pass (visible in timeline tools; a
// no-op when no tool is attached).
struct Range {
  explicit Range(const char* name) { nvtxRangePushA(name); }
  ~Range() { nvtxRangePop(); }
};

int fail(int code, const std::string& msg) {
  g_err = msg;
  return code;
}

int cuda_fail(cudaError_t e, const char* what) {
  return fail(LMG_ERR_CUDA, std::string("CUDA Error: ") + what + ": " + cudaGetErrorString(e));
}

size_t align_up(size_t v, size_t a = 256) { return (v + a - 1) / a * a; }

// Tensor maps over the interpolater's input seen as {z, y, x, example*channel}: one per box size
// {itile_z(iz), itile_xy(iy), itile_xy(ix), 1}, zero fill outside.  The encoder is a driver entry point; false
// if it is not there.
bool make_input_maps(lmg::InterpMaps* maps, const float* in, unsigned dim, size_t nchan) {
  typedef CUresult (*Encode)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                             const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                             CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static Encode encode = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return (Encode)p;
  }();
  if (encode == nullptr) return false;
  // the maps depend on the address and the extents alone: a caller that interpolates from the same
  // buffer again (a training loop) gets the maps of its last call back
  struct Last {
    const float* in = nullptr;
    unsigned dim = 0;
    size_t nchan = 0;
    lmg::InterpMaps maps;
  };
  static thread_local Last last;
  if (last.in == in && last.dim == dim && last.nchan == nchan && in != nullptr) {
    *maps = last.maps;
    return true;
  }
  last.in = nullptr;
  cuuint64_t d = dim;
  cuuint64_t gdim[4] = {d, d, d, (cuuint64_t)nchan};
  cuuint64_t gstride[3] = {d * 4, d * d * 4, d * d * d * 4};  // bytes, dimensions 1..3
  cuuint32_t estride[4] = {1, 1, 1, 1};
  for (int ix = 0; ix < lmg::ITILE_NXY; ix++)
    for (int iy = 0; iy < lmg::ITILE_NXY; iy++)
      for (int iz = 0; iz < lmg::ITILE_NZ; iz++) {
        cuuint32_t boxdim[4] = {(cuuint32_t)lmg::itile_z(iz), (cuuint32_t)lmg::itile_xy(iy),
                                (cuuint32_t)lmg::itile_xy(ix), 1};
        CUresult r = encode(&maps->m[(ix * lmg::ITILE_NXY + iy) * lmg::ITILE_NZ + iz], CU_TENSOR_MAP_DATA_TYPE_FLOAT32,
                            4, const_cast<float*>(in), gdim, gstride, boxdim, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return false;
      }
  last.maps = *maps;
  last.in = in;
  last.dim = dim;
  last.nchan = nchan;
  return true;
}

}  // namespace

namespace lmg {

GMParams to_params(const lmg_gridmaker* g) {
  GMParams p;
  p.res = g->resolution;
  p.half = (float)(g->dimension / 2.0);  // src/grid_maker.cpp:101
  p.rscale = g->radius_scale;
  p.G = g->gaussian_radius_multiple;
  p.finalm = g->final_radius_multiple;
  p.A = g->A; p.B = g->B; p.C = g->C; p.D = g->D; p.E = g->E;
  {
    double G = g->gaussian_radius_multiple, eg = std::exp(-G * G);
    bool truncated = g->final_radius_multiple == g->gaussian_radius_multiple;
    p.ta = truncated ? 0.f : (float)(2.0 * G * eg);
    p.tb = truncated ? 0.f : (float)((1.0 + 2.0 * G * G) * eg);
  }
  p.dim = g->dim;
  p.binary = g->binary;
  p.rti = g->radii_type_indexed;
  return p;
}

Xform to_xform(const lmg_transform* t) {
  Xform X;
  for (int i = 0; i < 4; i++) X.q[i] = t->q[i];
  for (int i = 0; i < 3; i++) { X.c[i] = t->center[i]; X.t[i] = t->translate[i]; }
  return X;
}

void fill_emit(EmitArgs& E, const lmg_gridmaker* g, const lmg_atoms* a) {
  std::memset(&E, 0, sizeof E);
  E.gm = to_params(g);
  E.N = a->max_atoms;
  E.T = a->ntypes;
  E.vec = a->type_vector != nullptr;
  E.n_atoms = a->n_atoms;
  E.coords = a->coords;
  E.type_index = a->type_index;
  E.type_vector = a->type_vector;
  E.radii = a->radii;
  E.centers = a->centers;
  for (int i = 0; i < 3; i++) E.center_host[i] = a->center_host[i];
  E.transforms = reinterpret_cast<const Xform*>(a->transforms);
  if (a->transforms == nullptr && a->transform_host != nullptr) {
    E.xform_host = to_xform(a->transform_host);
    E.has_xform_host = 1;
  }
  E.check_types = 1;
}

int quads_setting() { return g_quads; }

}  // namespace lmg

namespace {

using lmg::fill_emit;
using lmg::to_params;
using lmg::to_xform;

// Scratch layout of one pass over nb examples.
struct Layout {
  size_t status, recs, chanp, partial, total;
  size_t per_example;
};

constexpr size_t STATUS_BYTES = 256;

Layout layout(const lmg_gridmaker* g, int op, int nb, int N, int T, int vec) {
  Layout L;
  std::memset(&L, 0, sizeof L);
  size_t recs = align_up((size_t)N * sizeof(lmg::Rec));
  size_t chanp = (vec && g->radii_type_indexed) ? align_up((size_t)T * sizeof(lmg::ChanParam)) : 0;
  size_t partial = (vec && (op == LMG_OP_BACKWARD || op == LMG_OP_BACKWARD_GRADIENTS))
                       ? align_up((size_t)N * T * 3 * 4) : 0;
  L.per_example = recs + chanp + partial;
  size_t o = STATUS_BYTES;
  L.status = 0;
  L.recs = o; o += recs * nb;
  L.chanp = o; o += chanp * nb;
  L.partial = o; o += partial * nb;
  L.total = o;
  return L;
}

int check_common(const lmg_gridmaker* g, const lmg_atoms* a, const void* ws) {
  if (g == nullptr || a == nullptr) return fail(LMG_ERR_INVALID_ARGUMENT, "null settings or atoms");
  if (a->batch < 0 || a->max_atoms < 0 || a->ntypes <= 0)
    return fail(LMG_ERR_INVALID_ARGUMENT, "negative batch/atom count or no types");
  if (a->batch > 0 && a->max_atoms > 0 && (a->coords == nullptr || a->radii == nullptr))
    return fail(LMG_ERR_INVALID_ARGUMENT, "coords/radii missing memory");
  if ((a->type_index == nullptr) == (a->type_vector == nullptr) && a->batch > 0 && a->max_atoms > 0)
    return fail(LMG_ERR_INVALID_ARGUMENT, "exactly one of type_index and type_vector must be given");
  if (a->ntypes > 65535) return fail(LMG_ERR_INVALID_ARGUMENT, "more than 65535 types");
  if (g->dim > 65535) return fail(LMG_ERR_OUT_OF_RANGE, "grid dimension above 65535 points");
  // src/grid_maker.cpp:160-162, :443-445
  if (a->type_index != nullptr && g->radii_type_indexed)
    return fail(LMG_ERR_INVALID_ARGUMENT, "Type indexed radii not supported with index types.");
  if (ws == nullptr) return fail(LMG_ERR_WORKSPACE, "workspace missing");
  return LMG_OK;
}

void carve(lmg::EmitArgs& E, const Layout& L, char* ws) {
  E.status = reinterpret_cast<int*>(ws + L.status);
  E.recs = reinterpret_cast<lmg::Rec*>(ws + L.recs);
  E.chanp = reinterpret_cast<lmg::ChanParam*>(ws + L.chanp);
}

// number of examples per pass that fit the workspace; 0 if none
int examples_per_pass(const Layout& one, size_t ws_bytes, int batch) {
  if (ws_bytes < STATUS_BYTES + one.per_example) return 0;
  size_t fit = (ws_bytes - STATUS_BYTES) / one.per_example;
  // the example index is the y coordinate of every launch grid
  return (int)std::min<size_t>(std::min<size_t>(fit, (size_t)batch), 65535);
}

bool use_precise(const lmg_gridmaker* g) {
  if (g_precise >= 0) return g_precise != 0;
  // the fast exponential loses relative accuracy in proportion to the exponent's size (2*G^2)
  return g->gaussian_radius_multiple > 2.0f;
}

}  // namespace

extern "C" {

const char* lmg_last_error(void) { return g_err.c_str(); }
// lets the library's other translation units report through lmg_last_error()
void lmg_internal_set_error(const char* msg) { g_err = msg ? msg : ""; }
int lmg_version(void) { return 100; }

void lmg_set_random_seed(unsigned seed) { g_engine.seed(seed); }

// Bench support (not part of the reference interface): per-kernel durations and launch counts.
int lmg_profile_enable(int max_records) {
  for (auto& r : g_prof) { cudaEventDestroy(r.e0); cudaEventDestroy(r.e1); }
  g_prof.clear();
  g_prof_used = 0;
  g_prof_on = max_records > 0;
  for (int i = 0; i < max_records; i++) {
    ProfRec r;
    r.kind = 0;
    if (cudaEventCreate(&r.e0) != cudaSuccess || cudaEventCreate(&r.e1) != cudaSuccess)
      return fail(LMG_ERR_CUDA, "creating profiling events");
    g_prof.push_back(r);
  }
  return LMG_OK;
}

// ms[k], count[k] for k = 0 (forward kernel), 1 (backward kernels), 2 (zero fill of the forward
// output); resets the records
int lmg_profile_collect(double* ms, int* count) {
  for (int k = 0; k < 3; k++) { ms[k] = 0; count[k] = 0; }
  for (size_t i = 0; i < g_prof_used; i++) {
    cudaError_t e = cudaEventSynchronize(g_prof[i].e1);
    float t = 0;
    if (e == cudaSuccess) e = cudaEventElapsedTime(&t, g_prof[i].e0, g_prof[i].e1);
    if (e != cudaSuccess) return cuda_fail(e, "reading profiling events");
    ms[g_prof[i].kind] += t;
    count[g_prof[i].kind] += 1;
  }
  g_prof_used = 0;
  return LMG_OK;
}

long lmg_launch_count(void) { return g_launches; }

// Tuning knobs (not part of the reference interface).
void lmg_set_precise(int mode) { g_precise = mode; }
void lmg_set_quads(int on) { g_quads = on; }

int lmg_gridmaker_init(lmg_gridmaker* g, float res, float d, int bin, int rti, float rscale, float grm) {
  if (g == nullptr) return fail(LMG_ERR_INVALID_ARGUMENT, "null settings");
  g->resolution = res;
  g->dimension = d;
  g->radius_scale = rscale;
  g->gaussian_radius_multiple = grm;
  g->binary = bin != 0;
  g->radii_type_indexed = rti != 0;
  if (g->gaussian_radius_multiple < 0) {
    // a negative multiple asks for a truncated Gaussian without the quadratic tail
    g->gaussian_radius_multiple *= -1;
    g->final_radius_multiple = g->gaussian_radius_multiple;
  } else {
    g->final_radius_multiple = (1 + 2 * grm * grm) / (2 * grm);
  }
  g->dim = (unsigned)(std::round(d / res) + 1);
  // The reference evaluates these with the double-precision exponential of a float argument and
  // keeps the caller's sign of grm; the products run in double and are rounded once to float.
  double e = ::exp((double)(-2 * grm * grm));
  g->A = (float)(e * 4 * grm * grm);
  g->B = (float)(-e * (4 * grm + 8 * grm * grm * grm));
  g->C = (float)(e * (4 * grm * grm * grm * grm + 4 * grm * grm + 1));
  g->D = (float)(8 * grm * grm * ::exp(-2.0 * grm * grm));
  g->E = (float)(-(4 * grm + 8 * grm * grm * grm) * e);
  return LMG_OK;
}

int lmg_interpolater_init(lmg_interpolater* gi, float inres, float indim, float outres, float outdim) {
  if (gi == nullptr) return fail(LMG_ERR_INVALID_ARGUMENT, "null settings");
  gi->in_resolution = inres;
  gi->in_dimension = indim;
  gi->out_resolution = outres;
  gi->out_dimension = outdim;
  gi->in_dim = (unsigned)(std::round(indim / inres) + 1);
  gi->out_dim = (unsigned)(std::round(outdim / outres) + 1);
  return LMG_OK;
}

int lmg_transform_random(lmg_transform* t, const float center[3], float random_translate,
                         int random_rotate) {
  if (t == nullptr || center == nullptr) return fail(LMG_ERR_INVALID_ARGUMENT, "null transform");
  for (int i = 0; i < 3; i++) t->center[i] = center[i];
  // three translation draws are always consumed, then three more for a rotation
  std::uniform_real_distribution<double> sym(-1.0, 1);
  for (int i = 0; i < 3; i++) t->translate[i] = (float)(sym(g_engine) * random_translate);
  t->q[0] = 1; t->q[1] = 0; t->q[2] = 0; t->q[3] = 0;
  if (random_rotate) {
    // uniform random unit quaternion from three uniform variates
    std::uniform_real_distribution<double> unit(0, 1);
    double u1 = unit(g_engine), u2 = unit(g_engine), u3 = unit(g_engine);
    double s1 = std::sqrt(1 - u1), s2 = std::sqrt(u1);
    t->q[0] = (float)(s1 * std::sin(2 * M_PI * u2));
    t->q[1] = (float)(s1 * std::cos(2 * M_PI * u2));
    t->q[2] = (float)(s2 * std::sin(2 * M_PI * u3));
    t->q[3] = (float)(s2 * std::cos(2 * M_PI * u3));
  }
  return LMG_OK;
}

int lmg_transform_random_batch(lmg_transform* t, int n, const float center[3], float random_translate,
                               int random_rotate) {
  if (n < 0) return fail(LMG_ERR_INVALID_ARGUMENT, "negative size");
  for (int i = 0; i < n; i++) {
    int rc = lmg_transform_random(&t[i], center, random_translate, random_rotate);
    if (rc) return rc;
  }
  return LMG_OK;
}

size_t lmg_workspace_bytes(const lmg_gridmaker* g, int op, int batch, int max_atoms, int ntypes,
                           int vector_types) {
  if (g == nullptr || batch < 0 || max_atoms < 0 || ntypes <= 0) return 0;
  return layout(g, op, batch > 0 ? batch : 1, max_atoms, ntypes, vector_types).total;
}

int lmg_check_status(void* workspace, void* stream) {
  if (workspace == nullptr) return fail(LMG_ERR_WORKSPACE, "workspace missing");
  int st = 0;
  cudaError_t e = cudaMemcpyAsync(&st, workspace, sizeof st, cudaMemcpyDeviceToHost, (cudaStream_t)stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
  if (e != cudaSuccess) return cuda_fail(e, "reading status");
  if (st == 1) return fail(LMG_ERR_OUT_OF_RANGE, "Type index larger than allowed");
  if (st == 2) return fail(LMG_ERR_INVALID_ARGUMENT, "Incorrect channel size for diff");
  return LMG_OK;
}

int lmg_forward(const lmg_gridmaker* g, const lmg_atoms* a, float* out, void* workspace,
                size_t workspace_bytes, void* stream) {
  int rc = check_common(g, a, workspace);
  if (rc) return rc;
  if (a->batch == 0) return LMG_OK;
  if (out == nullptr) return fail(LMG_ERR_INVALID_ARGUMENT, "Output grid not allocated");
  cudaStream_t st = (cudaStream_t)stream;
  char* ws = (char*)workspace;
  int vec = a->type_vector != nullptr;
  size_t grid_elems = (size_t)a->ntypes * g->dim * g->dim * g->dim;
  cudaError_t e = cudaMemsetAsync(ws, 0, STATUS_BYTES, st);
  if (e != cudaSuccess) return cuda_fail(e, "clearing status");
  if (a->max_atoms == 0 || g->dim == 0) {
    e = cudaMemsetAsync(out, 0, grid_elems * a->batch * sizeof(float), st);
    return e == cudaSuccess ? LMG_OK : cuda_fail(e, "zeroing output");
  }
  Layout one = layout(g, LMG_OP_FORWARD, 1, a->max_atoms, a->ntypes, vec);
  int per_pass = examples_per_pass(one, workspace_bytes, a->batch);
  if (per_pass == 0)
    return fail(LMG_ERR_WORKSPACE, "workspace too small for one example: need " +
                                       std::to_string(STATUS_BYTES + one.per_example) + " bytes");
  // One zero fill of the whole output, then per pass one emit and one scatter launch.  (Measured
  // and dropped: filling on an auxiliary stream one chunk ahead of the scatter - the library's fill
  // kernels occupy every SM, so the scatter blocks merely queue behind them; and letting each
  // scatter launch clear the next chunk of examples - ten small launches lose more in ramp-up and
  // tail than the overlap gains.)
  Range whole("lmg_forward");
  ProfRec* pr_fill = prof_begin(2, st);
  {
    Range r("zero fill");
    e = cudaMemsetAsync(out, 0, grid_elems * a->batch * sizeof(float), st);
  }
  prof_end(pr_fill, st);
  if (e != cudaSuccess) return cuda_fail(e, "zeroing output");
  for (int b0 = 0; b0 < a->batch; b0 += per_pass) {
    int nb = std::min(per_pass, a->batch - b0);
    Layout L = layout(g, LMG_OP_FORWARD, nb, a->max_atoms, a->ntypes, vec);
    lmg::EmitArgs E;
    fill_emit(E, g, a);
    carve(E, L, ws);
    E.b0 = b0; E.nb = nb;
    E.round_types = 0;
    {
      Range r("emit");
      e = lmg::launch_emit(E, st);
    }
    if (e != cudaSuccess) return cuda_fail(e, "emit");
    lmg::BwdArgs S;
    std::memset(&S, 0, sizeof S);
    S.gm = E.gm; S.b0 = b0; S.nb = nb; S.N = E.N; S.T = E.T;
    S.type_vector = a->type_vector;
    S.centers = a->centers;
    for (int i = 0; i < 3; i++) S.center_host[i] = a->center_host[i];
    S.recs = E.recs; S.chanp = E.chanp;
    S.out_grid = out;
    S.precise = use_precise(g);
    S.quads = g_quads;
    ProfRec* pr = prof_begin(0, st);
    {
      Range r("forward scatter");
      e = lmg::launch_forward_scatter(S, vec != 0, st);
    }
    prof_end(pr, st);
    g_launches += 2 + ((vec && g->radii_type_indexed) ? 1 : 0);
    if (e != cudaSuccess) return cuda_fail(e, "forward scatter");
  }
  return LMG_OK;
}

static int backward_common(const lmg_gridmaker* g, const lmg_atoms* a, int op, int mode,
                           const float* diff, const float* density, float* atom_gradients,
                           float* type_gradients, float* relevance, void* workspace,
                           size_t workspace_bytes, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  char* ws = (char*)workspace;
  int vec = a->type_vector != nullptr;
  cudaError_t e = cudaMemsetAsync(ws, 0, STATUS_BYTES, st);
  if (e != cudaSuccess) return cuda_fail(e, "clearing status");
  if (a->max_atoms == 0) return LMG_OK;
  Layout one = layout(g, op, 1, a->max_atoms, a->ntypes, vec);
  int per_pass = examples_per_pass(one, workspace_bytes, a->batch);
  if (per_pass == 0)
    return fail(LMG_ERR_WORKSPACE, "workspace too small for one example: need " +
                                       std::to_string(STATUS_BYTES + one.per_example) + " bytes");
  for (int b0 = 0; b0 < a->batch; b0 += per_pass) {
    int nb = std::min(per_pass, a->batch - b0);
    Layout L = layout(g, op, nb, a->max_atoms, a->ntypes, vec);
    lmg::EmitArgs E;
    fill_emit(E, g, a);
    carve(E, L, ws);
    E.b0 = b0; E.nb = nb;
    E.round_types = 1;
    {
      Range r("emit");
      e = lmg::launch_emit(E, st);
    }
    if (e != cudaSuccess) return cuda_fail(e, "emit");
    lmg::BwdArgs B;
    std::memset(&B, 0, sizeof B);
    B.gm = E.gm; B.b0 = b0; B.nb = nb; B.N = E.N; B.T = E.T;
    B.type_vector = a->type_vector;
    B.centers = a->centers;
    for (int i = 0; i < 3; i++) B.center_host[i] = a->center_host[i];
    B.recs = E.recs; B.chanp = E.chanp;
    B.diff = diff; B.density = density;
    B.atom_gradients = atom_gradients; B.type_gradients = type_gradients; B.relevance = relevance;
    B.partial = reinterpret_cast<float*>(ws + L.partial);
    B.quads = g_quads;
    g_launches += 1 + ((vec && g->radii_type_indexed) ? 1 : 0);
    ProfRec* pr = prof_begin(1, st);
    {
      Range r(mode == 2 ? "backward relevance" : "backward");
      e = lmg::launch_backward(B, mode, st);
    }
    prof_end(pr, st);
    g_launches += mode == 1 ? 2 : 1;
    if (e != cudaSuccess) return cuda_fail(e, "backward");
  }
  return LMG_OK;
}

int lmg_backward(const lmg_gridmaker* g, const lmg_atoms* a, const float* diff, float* atom_gradients,
                 float* type_gradients, void* workspace, size_t workspace_bytes, void* stream) {
  int rc = check_common(g, a, workspace);
  if (rc) return rc;
  if (a->batch == 0 || a->max_atoms == 0) return LMG_OK;  // no atom, no gradient row to write
  int vec = a->type_vector != nullptr;
  if (diff == nullptr || atom_gradients == nullptr)
    return fail(LMG_ERR_INVALID_ARGUMENT, "diff/atom_gradients missing memory");
  if (!vec && type_gradients != nullptr)
    return fail(LMG_ERR_INVALID_ARGUMENT, "type_gradients given with index types");
  return backward_common(g, a, LMG_OP_BACKWARD, vec ? 1 : 0, diff, nullptr, atom_gradients,
                         type_gradients, nullptr, workspace, workspace_bytes, stream);
}

int lmg_backward_relevance(const lmg_gridmaker* g, const lmg_atoms* a, const float* density,
                           const float* diff, float* relevance, void* workspace,
                           size_t workspace_bytes, void* stream) {
  int rc = check_common(g, a, workspace);
  if (rc) return rc;
  if (a->batch == 0 || a->max_atoms == 0) return LMG_OK;  // no atom, no relevance to write
  if (a->type_index == nullptr)
    return fail(LMG_ERR_INVALID_ARGUMENT, "backward_relevance needs index types");
  if (density == nullptr || diff == nullptr || relevance == nullptr)
    return fail(LMG_ERR_INVALID_ARGUMENT, "density/diff/relevance missing memory");
  return backward_common(g, a, LMG_OP_BACKWARD_RELEVANCE, 2, diff, density, nullptr, nullptr,
                         relevance, workspace, workspace_bytes, stream);
}

int lmg_backward_gradients(const lmg_gridmaker* g, const lmg_atoms* a, const float* diff,
                           const float* atom_gradients, const float* type_gradients, float* diffdiff,
                           float* atom_diffdiff, float* type_diffdiff, void* workspace,
                           size_t workspace_bytes, void* stream) {
  int rc = check_common(g, a, workspace);
  if (rc) return rc;
  // src/grid_maker.cpp:559 and the vector-types-only overload set (include/libmolgrid/grid_maker.h:463-547)
  if (g->binary) return fail(LMG_ERR_INVALID_ARGUMENT, "Binary densities not supported");
  if (a->batch == 0) return LMG_OK;
  if (a->max_atoms == 0) {
    // no atoms: the gradient of the grid gradient is zero, the per-atom outputs are empty
    if (diffdiff == nullptr) return fail(LMG_ERR_INVALID_ARGUMENT, "backward_gradients argument missing memory");
    size_t bytes = (size_t)a->batch * a->ntypes * g->dim * g->dim * g->dim * sizeof(float);
    cudaError_t e0 = cudaMemsetAsync(diffdiff, 0, bytes, (cudaStream_t)stream);
    return e0 == cudaSuccess ? LMG_OK : cuda_fail(e0, "zeroing diffdiff");
  }
  if (a->type_vector == nullptr)
    return fail(LMG_ERR_INVALID_ARGUMENT, "backward_gradients needs vector types");
  if (diff == nullptr || atom_gradients == nullptr || type_gradients == nullptr || diffdiff == nullptr ||
      atom_diffdiff == nullptr || type_diffdiff == nullptr)
    return fail(LMG_ERR_INVALID_ARGUMENT, "backward_gradients argument missing memory");
  cudaStream_t st = (cudaStream_t)stream;
  char* ws = (char*)workspace;
  size_t grid_elems = (size_t)a->ntypes * g->dim * g->dim * g->dim;
  cudaError_t e = cudaMemsetAsync(ws, 0, STATUS_BYTES, st);
  if (e != cudaSuccess) return cuda_fail(e, "clearing status");
  // type_diffdiff is identically zero: the density is linear in the type weights
  e = cudaMemsetAsync(type_diffdiff, 0, (size_t)a->batch * a->max_atoms * a->ntypes * sizeof(float), st);
  if (e != cudaSuccess) return cuda_fail(e, "zeroing type_diffdiff");
  if (a->max_atoms == 0 || g->dim == 0) {
    e = cudaMemsetAsync(diffdiff, 0, grid_elems * a->batch * sizeof(float), st);
    return e == cudaSuccess ? LMG_OK : cuda_fail(e, "zeroing output");
  }
  Layout one = layout(g, LMG_OP_BACKWARD_GRADIENTS, 1, a->max_atoms, a->ntypes, 1);
  int per_pass = examples_per_pass(one, workspace_bytes, a->batch);
  if (per_pass == 0)
    return fail(LMG_ERR_WORKSPACE, "workspace too small for one example: need " +
                                       std::to_string(STATUS_BYTES + one.per_example) + " bytes");
  e = cudaMemsetAsync(diffdiff, 0, grid_elems * a->batch * sizeof(float), st);
  if (e != cudaSuccess) return cuda_fail(e, "zeroing output");
  for (int b0 = 0; b0 < a->batch; b0 += per_pass) {
    int nb = std::min(per_pass, a->batch - b0);
    Layout L = layout(g, LMG_OP_BACKWARD_GRADIENTS, nb, a->max_atoms, a->ntypes, 1);
    lmg::EmitArgs E;
    fill_emit(E, g, a);
    carve(E, L, ws);
    E.b0 = b0; E.nb = nb;
    E.round_types = 0;
    // atom part (atom_diffdiff) and, by scatter, the grid part (diffdiff)
    lmg::BwdArgs B;
    std::memset(&B, 0, sizeof B);
    B.gm = E.gm; B.b0 = b0; B.nb = nb; B.N = E.N; B.T = E.T;
    B.type_vector = a->type_vector;
    B.centers = a->centers;
    for (int i = 0; i < 3; i++) B.center_host[i] = a->center_host[i];
    B.recs = E.recs; B.chanp = E.chanp;
    B.diff = diff;
    B.atom_gradients = atom_diffdiff;
    B.ag_in = atom_gradients; B.tg_in = type_gradients;
    B.plain_reduce = 1;
    B.partial = reinterpret_cast<float*>(ws + L.partial);
    B.out_grid = diffdiff;
    B.quads = g_quads;
    e = lmg::launch_emit(E, st);
    if (e != cudaSuccess) return cuda_fail(e, "emit");
    e = lmg::launch_gradgrad_scatter(B, st);
    if (e != cudaSuccess) return cuda_fail(e, "backward_gradients grid");
    e = lmg::launch_backward(B, 3, st);
    if (e != cudaSuccess) return cuda_fail(e, "backward_gradients atoms");
    g_launches += 4 + (g->radii_type_indexed ? 1 : 0);
  }
  return LMG_OK;
}

static int transform_common(const lmg_transform* t, int n, const float* in, float* out, int dotranslate,
                            bool forward, void* stream) {
  if (t == nullptr) return fail(LMG_ERR_INVALID_ARGUMENT, "null transform");
  if (n < 0) return fail(LMG_ERR_INVALID_ARGUMENT, "negative size");
  if (n == 0) return LMG_OK;
  // Transform::checkGrids, include/libmolgrid/transform.h:130-147
  if (in == nullptr) return fail(LMG_ERR_INVALID_ARGUMENT, "Input coordinates missing memory");
  if (out == nullptr) return fail(LMG_ERR_INVALID_ARGUMENT, "Output coordinates missing memory");
  cudaError_t e = lmg::launch_transform(to_xform(t), n, in, out, dotranslate, forward, (cudaStream_t)stream);
  return e == cudaSuccess ? LMG_OK : cuda_fail(e, "transform");
}

int lmg_transform_forward(const lmg_transform* t, int n, const float* in, float* out, int dotranslate,
                          void* stream) {
  return transform_common(t, n, in, out, dotranslate, true, stream);
}

int lmg_transform_backward(const lmg_transform* t, int n, const float* in, float* out, int dotranslate,
                           void* stream) {
  return transform_common(t, n, in, out, dotranslate, false, stream);
}

unsigned lmg_tma_timeouts(void) {
  unsigned n = 0;
  return lmg::read_tma_timeouts(&n) == cudaSuccess ? n : 0xffffffffu;
}

void lmg_set_interp_tiled(int on) { g_interp_tiled = on; }

int lmg_interpolate(const lmg_interpolater* gi, int batch, int nchannels, const float* in,
                    const lmg_transform* transforms, const float* in_centers, const float* out_centers,
                    float* out, void* stream) {
  if (gi == nullptr || transforms == nullptr || in_centers == nullptr || out_centers == nullptr)
    return fail(LMG_ERR_INVALID_ARGUMENT, "null interpolater arguments");
  if (batch < 0 || nchannels < 0) return fail(LMG_ERR_INVALID_ARGUMENT, "negative size");
  // GridInterpolater::checkGrids, src/grid_interpolater.cpp:55-76
  if (in == out && in != nullptr)
    return fail(LMG_ERR_INVALID_ARGUMENT, "Input and output grid can not be the same in GridInterpolator.");
  if (in == nullptr) return fail(LMG_ERR_INVALID_ARGUMENT, "Input grid not allocated");
  if (out == nullptr) return fail(LMG_ERR_INVALID_ARGUMENT, "Output grid not allocated");
  lmg::InterpArgs I;
  I.in_res = gi->in_resolution;
  I.out_res = gi->out_resolution;
  I.in_half = (float)(gi->in_dimension / 2.0);
  I.out_half = (float)(gi->out_dimension / 2.0);
  I.in_dim = gi->in_dim;
  I.out_dim = gi->out_dim;
  I.K = nchannels;
  I.in = in;
  I.out = out;
  // The tiled kernel stages boxes of the input through tensor copies: rows of the input must start
  // on 16-byte boundaries, and an 8^3 output tile must map into a 16x16x20 box of input voxels under
  // any rotation (8*sqrt(3)*out_res/in_res + 2 <= 16).
  lmg::InterpMaps maps;
  bool tiled = g_interp_tiled && batch > 0 && nchannels > 0 && gi->in_dim > 0 &&
               (uintptr_t)in % 16 == 0 && (gi->in_dim * sizeof(float)) % 16 == 0 &&
               gi->out_resolution <= 1.008f * gi->in_resolution &&
               (size_t)batch * nchannels < (size_t)1 << 31 &&
               make_input_maps(&maps, in, gi->in_dim, (size_t)batch * nchannels);
  for (int b0 = 0; b0 < batch; b0 += lmg::INTERP_MAX_EX) {
    int nb = std::min(lmg::INTERP_MAX_EX, batch - b0);
    I.b0 = b0;
    for (int i = 0; i < nb; i++) {
      I.ex[i].X = to_xform(&transforms[b0 + i]);
      for (int k = 0; k < 3; k++) {
        I.ex[i].in_center[k] = in_centers[(size_t)(b0 + i) * 3 + k];
        I.ex[i].out_center[k] = out_centers[(size_t)(b0 + i) * 3 + k];
      }
    }
    cudaError_t e = tiled ? lmg::launch_interpolate_tiled(maps, I, nb, (cudaStream_t)stream)
                          : lmg::launch_interpolate(I, nb, (cudaStream_t)stream);
    g_launches += 1;
    if (e != cudaSuccess) return cuda_fail(e, "interpolate");
  }
  return LMG_OK;
}

int lmg_interpolate_backward(const lmg_interpolater* gi, int batch, int nchannels, const float* grad_out,
                             const lmg_transform* transforms, const float* in_centers,
                             const float* out_centers, float* grad_in, void* stream) {
  if (gi == nullptr || transforms == nullptr || in_centers == nullptr || out_centers == nullptr)
    return fail(LMG_ERR_INVALID_ARGUMENT, "null interpolater arguments");
  if (batch < 0 || nchannels < 0) return fail(LMG_ERR_INVALID_ARGUMENT, "negative size");
  if (grad_out == grad_in && grad_out != nullptr)
    return fail(LMG_ERR_INVALID_ARGUMENT, "Input and output grid can not be the same in GridInterpolator.");
  if (grad_out == nullptr) return fail(LMG_ERR_INVALID_ARGUMENT, "Output gradient grid not allocated");
  if (grad_in == nullptr) return fail(LMG_ERR_INVALID_ARGUMENT, "Input gradient grid not allocated");
  cudaStream_t st = (cudaStream_t)stream;
  size_t in_elems = (size_t)nchannels * gi->in_dim * gi->in_dim * gi->in_dim;
  cudaError_t e = cudaMemsetAsync(grad_in, 0, in_elems * batch * sizeof(float), st);
  if (e != cudaSuccess) return cuda_fail(e, "zeroing the input gradient");
  lmg::InterpArgs I;
  I.in_res = gi->in_resolution;
  I.out_res = gi->out_resolution;
  I.in_half = (float)(gi->in_dimension / 2.0);
  I.out_half = (float)(gi->out_dimension / 2.0);
  I.in_dim = gi->in_dim;
  I.out_dim = gi->out_dim;
  I.K = nchannels;
  I.in = grad_out;
  I.out = grad_in;
  for (int b0 = 0; b0 < batch; b0 += lmg::INTERP_MAX_EX) {
    int nb = std::min(lmg::INTERP_MAX_EX, batch - b0);
    I.b0 = b0;
    for (int i = 0; i < nb; i++) {
      I.ex[i].X = to_xform(&transforms[b0 + i]);
      for (int k = 0; k < 3; k++) {
        I.ex[i].in_center[k] = in_centers[(size_t)(b0 + i) * 3 + k];
        I.ex[i].out_center[k] = out_centers[(size_t)(b0 + i) * 3 + k];
      }
    }
    e = lmg::launch_interpolate_backward(I, nb, st);
    g_launches += 1;
    if (e != cudaSuccess) return cuda_fail(e, "interpolate backward");
  }
  return LMG_OK;
}

}  // extern "C"
