// Argument blocks passed by value to the gridding kernels, and their host-side launchers.
#pragma once
#include <cuda_runtime.h>

#include "lmg_device.cuh"

namespace lmg {

// A pass covers examples [b0, b0+nb) of the caller's batch; scratch arrays are indexed by the
// example's position in the pass (bl = b - b0), caller arrays by b.
struct EmitArgs {
  GMParams gm;
  int b0, nb, N, T;
  int vec;          // type vectors (1) or type indices (0)
  int round_types;  // 1: round the type index (backward passes), 0: floor (forward)
  int check_types;  // report type >= T through the status word
  const int* n_atoms;
  const float* coords;
  const float* type_index;
  const float* type_vector;
  const float* radii;
  const float* centers;
  float center_host[3];
  const Xform* transforms;
  Xform xform_host;
  int has_xform_host;
  // scratch
  Rec* recs;          // [nb][N]
  ChanParam* chanp;   // [nb][T], type-indexed radii only
  int* status;
};

struct BwdArgs {
  GMParams gm;
  int b0, nb, N, T;
  const float* type_vector;
  const float* centers;
  float center_host[3];
  const Rec* recs;
  const ChanParam* chanp;
  const float* diff;
  const float* density;
  float* atom_gradients;
  float* type_gradients;
  float* relevance;
  float* partial;  // [nb][N][T][3] scratch, vector types
  // backward_gradients (mode 3): incoming gradients, and a reduction without the weight factor
  const float* ag_in;  // [B][N][3]
  const float* tg_in;  // [B][N][T]
  int plain_reduce;
  float* out_grid;     // forward by scatter: [B][T][D][D][D], zero-filled before the launch
  int precise;
  int quads;           // rows are walked in aligned quads of four voxels when the grid allows it
};

cudaError_t launch_emit(const EmitArgs& A, cudaStream_t st);
cudaError_t launch_backward(const BwdArgs& G, int mode, cudaStream_t st);
cudaError_t launch_forward_scatter(const BwdArgs& G, bool vec, cudaStream_t st);
cudaError_t launch_gradgrad_scatter(const BwdArgs& G, cudaStream_t st);

}  // namespace lmg

// Host-side helpers shared by the entry points (defined with the C ABI).
struct lmg_gridmaker;
struct lmg_atoms;
struct lmg_transform;
namespace lmg {
GMParams to_params(const lmg_gridmaker* g);
Xform to_xform(const lmg_transform* t);
// input side of a pass: settings, sizes, the caller's arrays, per-example or single transform
void fill_emit(EmitArgs& E, const lmg_gridmaker* g, const lmg_atoms* a);
int quads_setting();  // current value of the aligned-quad kernel switch
}  // namespace lmg
