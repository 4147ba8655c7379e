// Batch assembly on the device: raw pre-typed atom records -> the padded batch arrays the gridding
// kernels read.
//
// The reference builds a batch on the host: per file it maps record types to channels and radii
// (src/coord_cache.cpp:82-148 with AtomIndexTyper::get_int_type, src/atom_typer.cpp:167-178 and
// include/libmolgrid/atom_typer.h:363-368), drops unmapped atoms, merges the sets of an example with
// type offsets (src/example.cpp:69-100) and copies every example to the GPU on its own.  Here the
// records of a whole batch travel in one copy and one kernel does the lookup, the merge and the
// padding; a second kernel takes each example's grid centre, the mean of its last set
// (src/grid_maker.cpp:126-137, src/coordinateset.cpp:228-243).
//
// Unmapped atoms keep their slot with type -1 and radius 0 instead of being dropped: the gridding
// kernels skip such atoms, so grids and gradients are those of the reference; the centre is taken
// over mapped atoms only, in record order, with the reference's float accumulation.
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstring>
#include <string>

#include "../../include/lmg_b200.h"

extern "C" void lmg_internal_set_error(const char* msg);

namespace {

struct Record {
  float x, y, z;
  int type;
};

int fail(int code, const std::string& msg) {
  lmg_internal_set_error(msg.c_str());
  return code;
}

constexpr int GENERIC_METAL = 26;  // GninaIndexTyper::GenericMetal, the type of unknown numbers

__device__ __forceinline__ int table_row(int raw) {
  return (raw >= 0 && raw < LMG_RECORD_TYPES) ? raw : GENERIC_METAL;
}

__global__ void __launch_bounds__(256) k_decode_records(const Record* rec, const lmg_record_set* sets,
                                                        const int* type_map, const float* type_radius,
                                                        int max_atoms, float* coords, float* type_index,
                                                        float* radii, int* status) {
  const lmg_record_set S = sets[blockIdx.y];
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < S.count; i += gridDim.x * blockDim.x) {
    int slot = S.dst_atom + i;
    if (slot < 0 || slot >= max_atoms) {
      atomicExch(status, 1);  // the descriptor table does not fit the arrays
      continue;
    }
    Record r = rec[S.first_record + i];
    int row = S.typer * LMG_RECORD_TYPES + table_row(r.type);
    int t = type_map[row];
    size_t a = (size_t)S.example * max_atoms + slot;
    coords[a * 3] = r.x;
    coords[a * 3 + 1] = r.y;
    coords[a * 3 + 2] = r.z;
    type_index[a] = t >= 0 ? (float)(t + S.type_offset) : -1.f;
    radii[a] = t >= 0 ? type_radius[row] : 0.f;
  }
}

// one thread per example: mean of the mapped atoms of its centre set, summed in record order
__global__ void __launch_bounds__(128) k_batch_centers(const Record* rec, const lmg_record_set* sets, int nsets,
                                                       const int* type_map, int batch, float* centers,
                                                       lmg_transform* transforms) {
  int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= batch) return;
  float sx = 0.f, sy = 0.f, sz = 0.f;
  int n = 0;
  for (int s = 0; s < nsets; s++) {
    const lmg_record_set S = sets[s];
    if (S.example != b || !S.is_center_set) continue;
    for (int i = 0; i < S.count; i++) {
      Record r = rec[S.first_record + i];
      if (type_map[S.typer * LMG_RECORD_TYPES + table_row(r.type)] < 0) continue;
      sx = __fadd_rn(sx, r.x);
      sy = __fadd_rn(sy, r.y);
      sz = __fadd_rn(sz, r.z);
      n++;
    }
  }
  if (n > 0) {
    float fn = (float)n;
    sx = __fdiv_rn(sx, fn);
    sy = __fdiv_rn(sy, fn);
    sz = __fdiv_rn(sz, fn);
  }
  if (centers != nullptr) {
    centers[b * 3] = sx;
    centers[b * 3 + 1] = sy;
    centers[b * 3 + 2] = sz;
  }
  if (transforms != nullptr) {
    transforms[b].center[0] = sx;
    transforms[b].center[1] = sy;
    transforms[b].center[2] = sz;
  }
}

// CoordinateSet::sum_types for vector types: one thread per type walks the atoms in order, so the
// sum is formed in the order of the CPU loop (src/coordinateset.cpp:364-371) and agrees bit for bit;
// neighbouring threads read neighbouring floats of a row.
__global__ void __launch_bounds__(128) k_sum_vector_types(const float* __restrict__ tv, int n, int T,
                                                          float* __restrict__ sum) {
  int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  float s = sum[t];
  for (int i = 0; i < n; i++) s = __fadd_rn(s, tv[(size_t)i * T + t]);
  sum[t] = s;
}

// ... for index types: a block per type counts the atoms whose rounded index is that type
// (src/coordinateset.cpp:357-362; the count is exact, so the order does not matter); block 0 also
// reports an index >= T through the status word.
__global__ void __launch_bounds__(256) k_sum_index_types(const float* __restrict__ ti, int n, int T,
                                                         float* __restrict__ sum, int* status) {
  __shared__ unsigned s_count;
  if (threadIdx.x == 0) s_count = 0;
  __syncthreads();
  const float t = (float)blockIdx.x;
  unsigned mine = 0;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    float r = roundf(ti[i]);
    mine += r == t;
    if (blockIdx.x == 0 && r >= (float)T && status != nullptr) atomicMax(status, 1);
  }
  mine = __reduce_add_sync(0xffffffffu, mine);
  if ((threadIdx.x & 31) == 0 && mine) atomicAdd(&s_count, mine);
  __syncthreads();
  if (threadIdx.x == 0) sum[blockIdx.x] = __fadd_rn(sum[blockIdx.x], (float)s_count);
}

}  // namespace

// Host-side half of batch staging: n chunks of bytes (the raw records of n examples) copied back to
// back into `dst` (pinned memory).  Plain memcpy on the calling thread; the Python caller releases
// the interpreter lock for the duration, so several batches can be staged at the same time.
extern "C" int lmg_gather_host(void* dst, size_t dst_bytes, int n, const unsigned long long* src,
                               const long long* bytes) {
  if (n < 0) return fail(LMG_ERR_INVALID_ARGUMENT, "negative size");
  if (n == 0) return LMG_OK;
  if (dst == nullptr || src == nullptr || bytes == nullptr)
    return fail(LMG_ERR_INVALID_ARGUMENT, "gather argument missing memory");
  size_t o = 0;
  for (int i = 0; i < n; i++) {
    if (bytes[i] < 0 || o + (size_t)bytes[i] > dst_bytes)
      return fail(LMG_ERR_INVALID_ARGUMENT, "gathered chunks do not fit the destination");
    if (bytes[i] > 0) std::memcpy(static_cast<char*>(dst) + o, reinterpret_cast<const void*>(src[i]), (size_t)bytes[i]);
    o += (size_t)bytes[i];
  }
  return LMG_OK;
}

extern "C" int lmg_sum_types(const float* type_index, const float* type_vector, int n, int ntypes, float* sum,
                             int zerofirst, int* status, void* stream) {
  if (n < 0 || ntypes < 0) return fail(LMG_ERR_INVALID_ARGUMENT, "negative size");
  if (ntypes == 0) return LMG_OK;
  if (sum == nullptr) return fail(LMG_ERR_INVALID_ARGUMENT, "Type sum output missing memory");
  if ((type_index == nullptr) == (type_vector == nullptr) && n > 0)
    return fail(LMG_ERR_INVALID_ARGUMENT, "exactly one of type_index and type_vector must be given");
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e = cudaSuccess;
  if (zerofirst) e = cudaMemsetAsync(sum, 0, sizeof(float) * (size_t)ntypes, st);
  if (e == cudaSuccess && status != nullptr) e = cudaMemsetAsync(status, 0, sizeof(int), st);
  if (e == cudaSuccess && n > 0) {
    if (type_vector != nullptr)
      k_sum_vector_types<<<(ntypes + 127) / 128, 128, 0, st>>>(type_vector, n, ntypes, sum);
    else
      k_sum_index_types<<<ntypes, 256, 0, st>>>(type_index, n, ntypes, sum, status);
    e = cudaGetLastError();
  }
  if (e != cudaSuccess) return fail(LMG_ERR_CUDA, std::string("summing types: ") + cudaGetErrorString(e));
  return LMG_OK;
}

extern "C" int lmg_decode_records(const void* records, const lmg_record_set* sets, int nsets,
                                  const int* type_map, const float* type_radius, int batch, int max_atoms,
                                  int max_set_records, float* coords, float* type_index, float* radii,
                                  float* centers, lmg_transform* transforms, int* status, void* stream) {
  if (nsets < 0 || batch < 0 || max_atoms < 0 || max_set_records < 0)
    return fail(LMG_ERR_INVALID_ARGUMENT, "negative size");
  if (batch == 0 || nsets == 0) return LMG_OK;
  if (records == nullptr || sets == nullptr || type_map == nullptr || type_radius == nullptr)
    return fail(LMG_ERR_INVALID_ARGUMENT, "record batch argument missing memory");
  if (coords == nullptr || type_index == nullptr || radii == nullptr || status == nullptr)
    return fail(LMG_ERR_INVALID_ARGUMENT, "batch arrays missing memory");
  if (nsets > 65535) return fail(LMG_ERR_INVALID_ARGUMENT, "more than 65535 coordinate sets in one batch");
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e = cudaMemsetAsync(status, 0, sizeof(int), st);
  if (e == cudaSuccess && max_set_records > 0 && max_atoms > 0) {
    int bx = (max_set_records + 255) / 256;
    if (bx > 64) bx = 64;  // large sets loop
    dim3 grid(bx, nsets);
    k_decode_records<<<grid, 256, 0, st>>>((const Record*)records, sets, type_map, type_radius, max_atoms, coords,
                                           type_index, radii, status);
    e = cudaGetLastError();
  }
  if (e == cudaSuccess && (centers != nullptr || transforms != nullptr)) {
    k_batch_centers<<<(batch + 127) / 128, 128, 0, st>>>((const Record*)records, sets, nsets, type_map, batch,
                                                         centers, transforms);
    e = cudaGetLastError();
  }
  if (e != cudaSuccess) return fail(LMG_ERR_CUDA, std::string("decoding records: ") + cudaGetErrorString(e));
  return LMG_OK;
}
