// Gather (rank-2 data, rank-2 int64 indices) for sm_100a.
//
// Reference nests: kernels/gather/naive_runtime_sized.py:26-49 and
// accera/python/accera/test/dsl_tests.py:1596-1601, 1642-1647
//   axis 0: output[i,j,k] = data[indices[i,j], k]
//   axis 1: output[i,j,k] = data[i, indices[j,k]]
// The reference has no GPU kernel for it.  Axis 0 is a row copy and is pure HBM
// traffic: every output row is moved as 128-bit vectors, four loads in flight
// per thread before the first store, the table read through the read-only path
// (duplicated indices hit L2) and the output written with streaming stores.
// Axis 1 gathers single elements and is handled element-wise.
//
// An index outside [0, dim) is never dereferenced: the destination is zero-
// filled and a counter in the status buffer is bumped for the host to report.
#include "accb_internal.h"

namespace accb {
namespace {

constexpr int kBlock = 256;
constexpr int kUnroll = 4;

// One block copies one chunk of kBlock * kUnroll vectors of one output row.
__global__ void __launch_bounds__(kBlock)
gather_rows_vec_kernel(const uint4* __restrict__ data, const int64_t* __restrict__ indices,
                       uint4* __restrict__ output, int64_t n_rows_in, int64_t vec_per_row,
                       int64_t chunks_per_row, int* __restrict__ status, int launch_id)
{
    pdl_enter();
    const int64_t row = blockIdx.x / chunks_per_row;
    const int64_t chunk = blockIdx.x % chunks_per_row;
    const int64_t src_row = indices[row];
    const bool ok = (src_row >= 0) && (src_row < n_rows_in);
    if (!ok && threadIdx.x == 0 && chunk == 0) { atomicAdd(status + ST_GATHER_COUNT, 1); status[ST_GATHER_ID] = launch_id; }
    const uint4* src = data + (ok ? src_row : 0) * vec_per_row;
    uint4* dst = output + row * vec_per_row;
    const int64_t v0 = chunk * (kBlock * kUnroll) + threadIdx.x;
    uint4 r[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
        const int64_t v = v0 + u * kBlock;
        r[u] = (ok && v < vec_per_row) ? __ldg(src + v) : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
        const int64_t v = v0 + u * kBlock;
        if (v < vec_per_row) __stcs(dst + v, r[u]);
    }
}

// Element-wise form, any element width: thread e handles output element e.
//   axis 0: e = row * d1 + k  ->  data[indices[row] * d1 + k]
//   axis 1: e = i * n_idx + jk ->  data[i * d1 + indices[jk]]
template <typename T>
__global__ void __launch_bounds__(kBlock)
gather_elem_kernel(const T* __restrict__ data, const int64_t* __restrict__ indices, T* __restrict__ output,
                   int64_t d0, int64_t d1, int64_t n_idx, int axis, int64_t total, int* __restrict__ status, int launch_id)
{
    pdl_enter();
    for (int64_t e = (int64_t)blockIdx.x * kBlock + threadIdx.x; e < total; e += (int64_t)gridDim.x * kBlock) {
        int64_t src;
        bool ok;
        if (axis == 0) {
            const int64_t row = e / d1, k = e - row * d1;
            const int64_t ix = indices[row];
            ok = (ix >= 0) && (ix < d0);
            src = ix * d1 + k;
            if (!ok && k == 0) { atomicAdd(status + ST_GATHER_COUNT, 1); status[ST_GATHER_ID] = launch_id; }
        } else {
            const int64_t i = e / n_idx, jk = e - i * n_idx;
            const int64_t ix = indices[jk];
            ok = (ix >= 0) && (ix < d1);
            src = i * d1 + ix;
            if (!ok && i == 0) { atomicAdd(status + ST_GATHER_COUNT, 1); status[ST_GATHER_ID] = launch_id; }
        }
        output[e] = ok ? __ldg(data + src) : T(0);
    }
}

template <typename T>
cudaError_t launch_elem(const void* data, const int64_t* indices, void* output, int64_t d0, int64_t d1, int64_t n_idx,
                        int axis, int64_t total, int* status, int launch_id, cudaStream_t stream)
{
    int64_t blocks = (total + kBlock - 1) / kBlock;
    if (blocks > 148 * 64) blocks = 148 * 64;   // grid-stride beyond this
    const cudaError_t e = launch_pdl(gather_elem_kernel<T>, dim3((unsigned)blocks), dim3(kBlock), stream, (const T*)data, indices,
                                     (T*)output, d0, d1, n_idx, axis, total, status, launch_id);
    return e != cudaSuccess ? e : cudaGetLastError();
}

}  // namespace

int launch_gather(const void* data, int64_t d0, int64_t d1, const int64_t* indices, int64_t i0, int64_t i1,
                  void* output, int axis, int elem_bytes, int* status, int launch_id, cudaStream_t stream, const char** err)
{
    const int64_t n_idx = i0 * i1;
    const int64_t total = (axis == 0) ? n_idx * d1 : d0 * n_idx;
    if (total == 0) return 0;
    cudaError_t e;
    const int64_t row_bytes = d1 * elem_bytes;
    const bool vec = (axis == 0) && (row_bytes % 16 == 0) && (row_bytes >= 512) &&
                     ((reinterpret_cast<uintptr_t>(data) & 15) == 0) && ((reinterpret_cast<uintptr_t>(output) & 15) == 0);
    if (vec) {
        const int64_t vpr = row_bytes / 16;
        const int64_t cpr = (vpr + kBlock * kUnroll - 1) / (kBlock * kUnroll);
        if (n_idx * cpr > 0x7fffffff) { *err = "gather: too many rows for this kernel's grid"; return ACCB_ERR_ARG; }
        e = launch_pdl(gather_rows_vec_kernel, dim3((unsigned)(n_idx * cpr)), dim3(kBlock), stream, (const uint4*)data, indices,
                       (uint4*)output, d0, vpr, cpr, status, launch_id);
        if (e == cudaSuccess) e = cudaGetLastError();
    } else {
        switch (elem_bytes) {
        case 1: e = launch_elem<uint8_t>(data, indices, output, d0, d1, n_idx, axis, total, status, launch_id, stream); break;
        case 2: e = launch_elem<uint16_t>(data, indices, output, d0, d1, n_idx, axis, total, status, launch_id, stream); break;
        case 4: e = launch_elem<uint32_t>(data, indices, output, d0, d1, n_idx, axis, total, status, launch_id, stream); break;
        case 8: e = launch_elem<uint64_t>(data, indices, output, d0, d1, n_idx, axis, total, status, launch_id, stream); break;
        default: *err = "gather: elem_bytes must be 1, 2, 4 or 8"; return ACCB_ERR_ARG;
        }
    }
    if (e != cudaSuccess) { *err = cudaGetErrorString(e); return ACCB_ERR_CUDA; }
    note_launches(1);
    return 1;
}

}  // namespace accb
