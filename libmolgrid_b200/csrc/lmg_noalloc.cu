// lmg_backward_static: the index-typed backward pass for callers that cannot provide a workspace
// because they cannot allocate device memory at all.
//
// Some hosts give the whole GPU to their own memory manager when they start (a framework that
// reserves all device memory up front, an embedding application with a fixed device budget), so a
// later cudaMalloc from a plug-in simply fails; others forbid allocation calls inside their
// steady-state loop because cudaMalloc may synchronise the device.  For them the atom records that
// the backward kernel needs live in the fixed array below instead of a caller-provided buffer.
//
// What that implies for the caller:
//   * The array is part of the library image: every GPU that loads the library holds
//     LMG_STATIC_BYTES (about 1 MB) until the process exits, whether or not this entry point is used.
//   * batch * max_atoms may not exceed LMG_STATIC_MAX_ATOMS; larger requests are refused with
//     LMG_ERR_WORKSPACE and nothing is launched.
//   * All calls on a device share the one array and it keeps whatever the previous call left.
//     The status word is cleared and every record slot is rewritten at the start of each call, so
//     calls issued one after another on the same stream are independent; calls that can overlap on
//     the GPU (different streams, different host threads) race on it and must be serialised by the
//     caller.
//   * A type index >= ntypes leaves that atom's gradient at zero and sets a status word in the
//     array; lmg_static_check_status(stream) reads it back (the counterpart of lmg_check_status,
//     which needs a workspace pointer this path does not have).
//   * The first call on each device looks up the array's device address (cudaGetSymbolAddress).
//     Make that first call outside any stream capture; later calls only launch work.
//   * Nothing here calls cudaMalloc, cudaFree or any other allocating routine.
#include <cstring>
#include <mutex>
#include <string>

#include "../../include/lmg_b200.h"
#include "lmg_launch.h"

extern "C" void lmg_internal_set_error(const char* msg);

namespace {

constexpr size_t STATIC_STATUS_BYTES = 256;
constexpr size_t STATIC_MAX_ATOMS = 16384;
constexpr size_t STATIC_BYTES = STATIC_STATUS_BYTES + STATIC_MAX_ATOMS * sizeof(lmg::Rec);

// In host code this name is only a handle for the runtime; the address a kernel can use comes
// from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_static_scratch[STATIC_BYTES];

constexpr int MAX_DEVICES = 64;
void* g_scratch_ptr[MAX_DEVICES] = {};
std::mutex g_setup_mutex;

int fail(int code, const std::string& msg) {
  lmg_internal_set_error(msg.c_str());
  return code;
}

// Device address of the array on the current device, resolved once per device.
int scratch_for_current_device(char** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(LMG_ERR_CUDA, std::string("CUDA Error: ") + cudaGetErrorString(e));
  if (dev < 0 || dev >= MAX_DEVICES) return fail(LMG_ERR_CUDA, "device index out of range");
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || p == nullptr)
      return fail(LMG_ERR_CUDA, std::string("CUDA Error: cudaGetSymbolAddress: ") + cudaGetErrorString(e));
    g_scratch_ptr[dev] = p;
  }
  *out = static_cast<char*>(g_scratch_ptr[dev]);
  return LMG_OK;
}

}  // namespace

extern "C" {

size_t lmg_static_max_atoms(void) { return STATIC_MAX_ATOMS; }

int lmg_backward_static(const lmg_gridmaker* g, const lmg_atoms* a, const float* diff,
                        float* atom_gradients, void* stream) {
  if (g == nullptr || a == nullptr) return fail(LMG_ERR_INVALID_ARGUMENT, "null settings or atoms");
  if (a->batch < 0 || a->max_atoms < 0 || a->ntypes <= 0 || a->ntypes > 65535)
    return fail(LMG_ERR_INVALID_ARGUMENT, "bad batch, atom or type count");
  if (a->type_vector != nullptr || (a->type_index == nullptr && a->batch > 0 && a->max_atoms > 0))
    return fail(LMG_ERR_INVALID_ARGUMENT, "lmg_backward_static takes index types only");
  if (g->radii_type_indexed)
    return fail(LMG_ERR_INVALID_ARGUMENT, "Type indexed radii not supported with index types.");
  if (g->dim > 65535) return fail(LMG_ERR_OUT_OF_RANGE, "grid dimension above 65535 points");
  size_t total = (size_t)a->batch * (size_t)a->max_atoms;
  if (total > STATIC_MAX_ATOMS)
    return fail(LMG_ERR_WORKSPACE,
                "lmg_backward_static handles at most " + std::to_string(STATIC_MAX_ATOMS) +
                    " atoms per call (batch * max_atoms = " + std::to_string(total) +
                    "); use lmg_backward with a workspace for larger batches");
  if (total == 0) return LMG_OK;
  if (a->coords == nullptr || a->radii == nullptr || diff == nullptr || atom_gradients == nullptr)
    return fail(LMG_ERR_INVALID_ARGUMENT, "coords/radii/diff/atom_gradients missing memory");

  char* ws = nullptr;
  int rc = scratch_for_current_device(&ws);
  if (rc != LMG_OK) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  // the status word must start at zero; the record slots are all rewritten by the first kernel
  cudaError_t e = cudaMemsetAsync(ws, 0, STATIC_STATUS_BYTES, st);
  if (e != cudaSuccess) return fail(LMG_ERR_CUDA, std::string("CUDA Error: ") + cudaGetErrorString(e));

  lmg::EmitArgs E;
  lmg::fill_emit(E, g, a);
  E.gm.rti = 0;
  E.b0 = 0; E.nb = a->batch;
  E.round_types = 1;
  E.status = reinterpret_cast<int*>(ws);
  E.recs = reinterpret_cast<lmg::Rec*>(ws + STATIC_STATUS_BYTES);
  e = lmg::launch_emit(E, st);
  if (e != cudaSuccess) return fail(LMG_ERR_CUDA, std::string("CUDA Error: emit: ") + cudaGetErrorString(e));

  lmg::BwdArgs B;
  std::memset(&B, 0, sizeof B);
  B.gm = E.gm;
  B.b0 = 0; B.nb = a->batch; B.N = a->max_atoms; B.T = a->ntypes;
  B.centers = a->centers;
  for (int i = 0; i < 3; i++) B.center_host[i] = a->center_host[i];
  B.recs = E.recs;
  B.diff = diff;
  B.atom_gradients = atom_gradients;
  B.quads = lmg::quads_setting();  // the aligned-quad kernel where the grid allows it (the launcher checks)
  e = lmg::launch_backward(B, 0, st);
  if (e != cudaSuccess) return fail(LMG_ERR_CUDA, std::string("CUDA Error: backward: ") + cudaGetErrorString(e));
  return LMG_OK;
}

// The data-dependent check of lmg_backward (a type index >= ntypes) for the static entry point:
// reads the status word that the last lmg_backward_static call on this device and stream left in
// the fixed array.  A 4-byte device-to-host copy and a stream synchronisation; allocates nothing.
int lmg_static_check_status(void* stream) {
  char* ws = nullptr;
  int rc = scratch_for_current_device(&ws);
  if (rc != LMG_OK) return rc;
  int st = 0;
  cudaError_t e = cudaMemcpyAsync(&st, ws, sizeof st, cudaMemcpyDeviceToHost, (cudaStream_t)stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
  if (e != cudaSuccess) return fail(LMG_ERR_CUDA, std::string("CUDA Error: reading status: ") + cudaGetErrorString(e));
  if (st == 1) return fail(LMG_ERR_OUT_OF_RANGE, "Type index larger than allowed");
  if (st == 2) return fail(LMG_ERR_INVALID_ARGUMENT, "Incorrect channel size for diff");
  return LMG_OK;
}

}  // extern "C"
