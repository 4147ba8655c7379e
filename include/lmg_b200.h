/* lmg_b200.h - C ABI of the B200 (sm_100a) gridding library, liblmg_b200.so.
 *
 * These entry points are what a binding of libmolgrid's gridding path calls instead of
 * the reference's own CUDA overloads.  Each declaration names the reference interface it
 * replaces (paths relative to the libmolgrid tree).  Conventions:
 *
 *  - Every array argument is a DEVICE pointer to dense row-major fp32 unless its comment
 *    says "host".  Grids are [T][D][D][D] per example with Z fastest, as in the reference
 *    (include/libmolgrid/grid.h:119-128); batches add a leading example dimension.
 *  - Nothing is allocated on the caller's behalf: kernels take their scratch memory from
 *    the caller-provided workspace (size from lmg_workspace_bytes).  Outputs are fully
 *    overwritten.
 *  - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream, which is
 *    what the reference always uses).  No call synchronises the host unless it says so.
 *  - Return value: LMG_OK or an LMG_ERR_* code; lmg_last_error() (thread-local) describes
 *    the last failure.  The codes map back to the reference's exceptions:
 *    LMG_ERR_OUT_OF_RANGE <-> std::out_of_range, LMG_ERR_INVALID_ARGUMENT <->
 *    std::invalid_argument, LMG_ERR_CUDA <-> std::runtime_error (LMG_CUDA_CHECK,
 *    include/libmolgrid/common.h:41-47).  Nothing throws across this boundary.
 *  - There is no CPU fallback: without a CUDA device every compute call fails with
 *    LMG_ERR_CUDA.
 */
#ifndef LMG_B200_H_
#define LMG_B200_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  LMG_OK = 0,
  LMG_ERR_OUT_OF_RANGE = 1,
  LMG_ERR_INVALID_ARGUMENT = 2,
  LMG_ERR_CUDA = 3,
  LMG_ERR_WORKSPACE = 4
};

/* GridMaker settings and derived constants.
 * Replaces the data members of libmolgrid::GridMaker (include/libmolgrid/grid_maker.h:36-48). */
typedef struct lmg_gridmaker {
  float resolution;
  float dimension;
  float radius_scale;
  float gaussian_radius_multiple; /* stored non-negative, as the reference does */
  float final_radius_multiple;
  float A, B, C, D, E;
  unsigned dim; /* grid points per side */
  int binary;
  int radii_type_indexed;
} lmg_gridmaker;

/* Fills *g exactly as GridMaker::GridMaker + GridMaker::initialize do
 * (include/libmolgrid/grid_maker.h:70-74, src/grid_maker.cpp:15-36), on the host. */
int lmg_gridmaker_init(lmg_gridmaker* g, float resolution, float dimension, int binary,
                       int radii_type_indexed, float radius_scale, float gaussian_radius_multiple);

/* Rotation about `center` followed by a translation.
 * Replaces libmolgrid::Transform's state (include/libmolgrid/transform.h:28-31);
 * q = (real, i, j, k) as libmolgrid::Quaternion stores it (include/libmolgrid/quaternion.h:22-26). */
typedef struct lmg_transform {
  float q[4];
  float center[3];
  float translate[3];
} lmg_transform;

/* Fills *t with a random transform drawn exactly as Transform::Transform(float3, float, bool)
 * does (src/transform.cpp:13-33) from the library's engine; lmg_set_random_seed reseeds it
 * (python/bindings.in.cpp:400, src/libmolgrid.cpp:11).  Host only. */
int lmg_transform_random(lmg_transform* t, const float center[3], float random_translate,
                         int random_rotate);
/* n such transforms drawn one after the other into t[n] (the loop of
 * include/libmolgrid/grid_maker.h:194-201, one Transform per example in order). */
int lmg_transform_random_batch(lmg_transform* t, int n, const float center[3], float random_translate,
                               int random_rotate);
void lmg_set_random_seed(unsigned seed);

/* The atoms of a batch of `batch` examples, padded to `max_atoms` per example: the argument
 * set of the reference's batched raw-tensor overloads (include/libmolgrid/grid_maker.h:265-301)
 * with the per-example Transform of forward(Example, Transform, Grid)
 * (src/grid_maker.cpp:109-116) folded in.  batch == 1 gives the single-example overloads. */
typedef struct lmg_atoms {
  int batch;
  int max_atoms;
  int ntypes;                /* channels of the grid (and length of a type vector) */
  const int* n_atoms;        /* [batch] valid atoms per example, or NULL: all max_atoms */
  const float* coords;       /* [batch][max_atoms][3] */
  const float* type_index;   /* [batch][max_atoms], or NULL when type_vector is given */
  const float* type_vector;  /* [batch][max_atoms][ntypes], or NULL */
  const float* radii;        /* [batch][max_atoms], or [batch][ntypes] if radii_type_indexed */
  const float* centers;      /* [batch][3] grid centres, or NULL: use center_host for all */
  float center_host[3];      /* host value */
  const lmg_transform* transforms; /* [batch] applied to coords before gridding, or NULL */
  const lmg_transform* transform_host; /* host: one transform for every example, or NULL;
                                          ignored when `transforms` is given */
} lmg_atoms;

enum {
  LMG_OP_FORWARD = 0,
  LMG_OP_BACKWARD = 1,
  LMG_OP_BACKWARD_GRADIENTS = 2,
  LMG_OP_BACKWARD_RELEVANCE = 3
};

/* Scratch bytes that let the given op process the whole batch in one pass.  A smaller
 * workspace makes the op run the batch in several passes; it fails with LMG_ERR_WORKSPACE
 * only if not even one example fits.  `vector_types` != 0 for type_vector input. */
size_t lmg_workspace_bytes(const lmg_gridmaker* g, int op, int batch, int max_atoms, int ntypes,
                           int vector_types);

/* Density (or binary occupancy) grids out[batch][ntypes][D][D][D].
 * Replaces GridMaker::forward for index types (src/grid_maker.cu:260-289, CPU :153-212),
 * vector types (src/grid_maker.cu:402-441, CPU :214-271) and their batched / Transform
 * overloads (include/libmolgrid/grid_maker.h:194-201,265-301, src/grid_maker.cpp:109-141).
 * Results follow the reference's CPU path. */
int lmg_forward(const lmg_gridmaker* g, const lmg_atoms* atoms, float* out, void* workspace,
                size_t workspace_bytes, void* stream);

/* Atom gradients atom_gradients[batch][max_atoms][3] from grid gradients
 * diff[batch][ntypes][D][D][D]; with vector types also type_gradients[batch][max_atoms][ntypes]
 * (must be NULL for index types).
 * Replaces GridMaker::backward (src/grid_maker.cu:576-642, CPU src/grid_maker.cpp:436-519).
 * Inputs without atoms or without examples (max_atoms == 0 or batch == 0) are accepted by every
 * pass, as the reference's loops over zero atoms are: lmg_forward and lmg_backward_gradients still
 * clear their grids, the per-atom outputs (which are empty) are not touched and may be NULL. */
int lmg_backward(const lmg_gridmaker* g, const lmg_atoms* atoms, const float* diff,
                 float* atom_gradients, float* type_gradients, void* workspace,
                 size_t workspace_bytes, void* stream);
/* With vector types, type_gradients may be NULL when only the atom gradients are wanted (types that
 * are inputs rather than parameters); the reference always computes both.  With per-atom radii the
 * kernels then read only the channels in which an atom carries weight. */

/* Second-order pass for vector types: from diff and the incoming atom_gradients /
 * type_gradients produce diffdiff[batch][ntypes][D][D][D], atom_diffdiff[batch][max_atoms][3]
 * and type_diffdiff[batch][max_atoms][ntypes] (identically zero).
 * Replaces GridMaker::backward_gradients (src/grid_maker.cu:755-803, CPU
 * src/grid_maker.cpp:529-672). */
int lmg_backward_gradients(const lmg_gridmaker* g, const lmg_atoms* atoms, const float* diff,
                           const float* atom_gradients, const float* type_gradients,
                           float* diffdiff, float* atom_diffdiff, float* type_diffdiff,
                           void* workspace, size_t workspace_bytes, void* stream);

/* Per-atom relevance relevance[batch][max_atoms] from a density grid and a relevance grid,
 * index types only.
 * Replaces GridMaker::backward_relevance (src/grid_maker.cu:974-992, CPU
 * src/grid_maker.cpp:684-704). */
int lmg_backward_relevance(const lmg_gridmaker* g, const lmg_atoms* atoms, const float* density,
                           const float* diff, float* relevance, void* workspace,
                           size_t workspace_bytes, void* stream);

/* lmg_backward for index types without a workspace and without any allocation.
 * No counterpart in the reference.  It exists for hosts that cannot allocate device memory for
 * a plug-in: applications that hand the whole GPU to their own memory manager at start-up (a later
 * cudaMalloc fails there), or that ban allocation calls from their steady-state loop because
 * cudaMalloc may synchronise the device.  The atom records live in a fixed array inside the
 * library image instead (about 1 MB, held by every GPU that loads the library until exit).
 *  - batch * max_atoms must not exceed lmg_static_max_atoms() (16384); beyond that the call fails
 *    with LMG_ERR_WORKSPACE and launches nothing.  Index types only.
 *  - All calls on one device share that array, which keeps the previous call's contents; each
 *    call clears the status word and rewrites every record slot first, so consecutive calls on one
 *    stream are independent, while calls that can overlap on the GPU race and must be serialised by
 *    the caller.
 *  - The first call on each device resolves the array's device address; make it outside any stream
 *    capture.
 *  - A type index >= ntypes is not an error of the call itself (the data lives on the device): the
 *    atom's gradient stays zero and a status word is set in the fixed array.
 *    lmg_static_check_status(stream) waits for the stream, reads that word (a 4-byte copy, nothing
 *    allocated) and returns LMG_ERR_INVALID_ARGUMENT for it, as lmg_check_status does for
 *    lmg_backward.  It reports the last lmg_backward_static call on the current device.
 * Results are those of lmg_backward, bit for bit (the same kernels run). */
int lmg_backward_static(const lmg_gridmaker* g, const lmg_atoms* atoms, const float* diff,
                        float* atom_gradients, void* stream);
size_t lmg_static_max_atoms(void);
int lmg_static_check_status(void* stream);

/* out[n][3] = transform applied to in[n][3]; in-place is allowed; `t` is a host struct.
 * dotranslate == 0 rotates about the centre only.
 * Replaces Transform::forward / Transform::backward on Grid2fCUDA
 * (src/transform.cu:66-93, CPU src/transform.cpp:57-108). */
int lmg_transform_forward(const lmg_transform* t, int n, const float* in, float* out,
                          int dotranslate, void* stream);
int lmg_transform_backward(const lmg_transform* t, int n, const float* in, float* out,
                           int dotranslate, void* stream);

/* GridInterpolater settings.
 * Replaces libmolgrid::GridInterpolater's members (include/libmolgrid/grid_interpolater.h:33-38,59-64). */
typedef struct lmg_interpolater {
  float in_resolution, in_dimension, out_resolution, out_dimension;
  unsigned in_dim, out_dim;
} lmg_interpolater;

int lmg_interpolater_init(lmg_interpolater* gi, float in_resolution, float in_dimension,
                          float out_resolution, float out_dimension);

/* Trilinear resample out[batch][nchannels][Dout]^3 of in[batch][nchannels][Din]^3 under one
 * transform per example.  transforms[batch], in_centers[batch][3] and out_centers[batch][3]
 * are HOST arrays (the reference takes them by value); they are copied into the launch.
 * Replaces GridInterpolater::forward (src/grid_interpolater.cu:134-166, CPU
 * src/grid_interpolater.cpp:16-48). */
int lmg_interpolate(const lmg_interpolater* gi, int batch, int nchannels, const float* in,
                    const lmg_transform* transforms, const float* in_centers,
                    const float* out_centers, float* out, void* stream);

/* Adjoint of lmg_interpolate: grad_in[batch][nchannels][Din]^3 (fully overwritten) from
 * grad_out[batch][nchannels][Dout]^3 with the same transforms and centres.  The reference has no
 * backward pass for GridInterpolater ("TODO: backwards", include/libmolgrid/grid_interpolater.h:179);
 * this is the transpose of the forward pass's trilinear weights. */
int lmg_interpolate_backward(const lmg_interpolater* gi, int batch, int nchannels, const float* grad_out,
                             const lmg_transform* transforms, const float* in_centers,
                             const float* out_centers, float* grad_in, void* stream);

/* ---- batch assembly from pre-typed atom records --------------------------------------------
 * A record is the 16-byte {float x, y, z; int type} of the reference's .gninatypes / .molcache2 files
 * (src/coord_cache.cpp:82-148).  One call turns the records of a whole batch into the padded batch
 * arrays lmg_forward / lmg_backward read: per coordinate set it looks channel and radius up in the
 * typer's tables (AtomIndexTyper::get_int_type, src/atom_typer.cpp:167-178; type numbers outside
 * [0, LMG_RECORD_TYPES) use the GenericMetal row), adds the set's type offset (Example::merge_coordinates,
 * src/example.cpp:69-100) and writes the atoms to their slots of the example.  Atoms whose mapped type
 * is negative keep their slot with type -1 and radius 0 (the reference drops them; the gridding
 * kernels skip them, so grids and gradients agree).  Optionally each example's grid centre - the mean
 * of the mapped atoms of its centre set, the reference's default for forward(Example, grid)
 * (src/grid_maker.cpp:126-137, src/coordinateset.cpp:228-243) - is written to centers[batch][3]
 * and into transforms[batch].center.  All pointers are device pointers. */
#define LMG_RECORD_TYPES 28
typedef struct lmg_record_set {
  long long first_record; /* index of the set's first record in `records` */
  int count;              /* records in the set */
  int example;            /* destination example */
  int typer;              /* row block of type_map / type_radius that applies */
  int type_offset;        /* added to mapped types: the types of earlier sets of the example */
  int dst_atom;           /* first atom slot of the set within the example */
  int is_center_set;      /* 1 for the set whose mean is the example's grid centre */
} lmg_record_set;

/* type_map[ntypers][LMG_RECORD_TYPES] (channel or -1) and type_radius[ntypers][LMG_RECORD_TYPES];
 * max_set_records = the largest `count`; *status (device int) becomes 1 if a set does not fit
 * max_atoms.  centers and transforms may be NULL. */
int lmg_decode_records(const void* records, const lmg_record_set* sets, int nsets, const int* type_map,
                       const float* type_radius, int batch, int max_atoms, int max_set_records,
                       float* coords, float* type_index, float* radii, float* centers,
                       lmg_transform* transforms, int* status, void* stream);

/* Host-side helper of batch staging (no device work): copies n chunks, chunk i being bytes[i]
 * bytes at host address src[i], back to back into dst (normally pinned memory that one
 * host-to-device copy then moves).  The counterpart of the per-atom push_back loops of
 * Example::merge_coordinates (src/example.cpp:84-96) for raw records. */
int lmg_gather_host(void* dst, size_t dst_bytes, int n, const unsigned long long* src,
                    const long long* bytes);

/* sum[ntypes] (+)= the per-type totals of one coordinate set on the device: with type vectors
 * type_vector[n][ntypes] the column sums, formed atom by atom in order; with type indices
 * type_index[n] the number of atoms whose rounded index is the type (negative indices are skipped).
 * zerofirst != 0 clears sum first.  *status (device int, may be NULL) becomes 1 if an index is
 * >= ntypes, the CPU path's out_of_range.  Exactly one of type_index / type_vector is given.
 * Replaces CoordinateSet::sum_types on Grid1fCUDA (src/coordinateset.cu:21-57); the results are
 * those of the CPU overload (src/coordinateset.cpp:352-374), which the reference's own GPU kernel
 * for type indices does not reproduce (it adds the index instead of 1 and overwrites sum). */
int lmg_sum_types(const float* type_index, const float* type_vector, int n, int ntypes, float* sum,
                  int zerofirst, int* status, void* stream);

/* Reads back (synchronising `stream`) the status word that kernels of the last call that used
 * `workspace` wrote: 0, or LMG_ERR_OUT_OF_RANGE / LMG_ERR_INVALID_ARGUMENT when an atom's type
 * index was >= ntypes - the data-dependent checks of src/grid_maker.cpp:172 and :458-460,
 * which the reference makes on the host while it loops over atoms. */
int lmg_check_status(void* workspace, void* stream);

const char* lmg_last_error(void);
int lmg_version(void);

#ifdef __cplusplus
}
#endif
#endif /* LMG_B200_H_ */
