// Second pass of a K-split tensor-core GEMM: adds the fp32 / int32 partial results of the K slices in slice
// order and applies the epilogue,
//     C <- epi(alpha * (P[0] + P[1] + ... + P[S-1]) + beta * C + bias)
// The partials are dense row-major M x N matrices, one after the other.  Pure HBM streaming: every thread takes
// four consecutive columns (one 16-byte load per slice).
//
// The reference has no counterpart: its generated kernels give every output tile to one thread block and walk
// the whole K there (accera/transforms/src/exec/ExecutionPlanToAffineLoweringPass.cpp:5986-6533).  A problem with few
// output tiles and a long K leaves most of a 148-SM part idle that way.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "accb_internal.h"

namespace accb {
namespace {

template <typename T> __device__ __forceinline__ float load_as_float(const T* p) { return (float)*p; }
template <typename T> __device__ __forceinline__ void store_from_float(T* p, float v) { *p = (T)v; }

template <typename TC>
__global__ void __launch_bounds__(256)
splitk_reduce_f32_kernel(const float* __restrict__ partial, int slices, int64_t m, int64_t n, TC* __restrict__ C, int64_t cs0,
                         int64_t cs1, float alpha, float beta, const float* __restrict__ bias, int relu)
{
    pdl_enter();    // may be resident while the launch that writes the partial sums still runs: wait for it before reading
    const int64_t groups_per_row = (n + 3) / 4;
    const int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (g >= m * groups_per_row) return;
    const int64_t row = g / groups_per_row, col0 = (g - row * groups_per_row) * 4;
    const int64_t plane = m * n;
    const float* src = partial + row * n + col0;
    float acc[4] = { 0.f, 0.f, 0.f, 0.f };
    const bool vec = (n % 4 == 0);
    for (int s = 0; s < slices; ++s) {
        if (vec) {
            const float4 v = __ldcs(reinterpret_cast<const float4*>(src + (int64_t)s * plane));
            acc[0] += v.x; acc[1] += v.y; acc[2] += v.z; acc[3] += v.w;
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) if (col0 + j < n) acc[j] += src[(int64_t)s * plane + j];
        }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        if (col0 + j >= n) break;
        TC* d = C + row * cs0 + (col0 + j) * cs1;
        float x = alpha * acc[j];
        if (beta != 0.0f) x += beta * load_as_float(d);
        if (bias) x += __ldg(bias + col0 + j);
        if (relu) x = fmaxf(x, 0.0f);
        store_from_float(d, x);
    }
}

__global__ void __launch_bounds__(256)
splitk_reduce_s32_kernel(const int* __restrict__ partial, int slices, int64_t m, int64_t n, int* __restrict__ C, int64_t cs0,
                         int64_t cs1, int add_c, int relu)
{
    pdl_enter();
    const int64_t groups_per_row = (n + 3) / 4;
    const int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (g >= m * groups_per_row) return;
    const int64_t row = g / groups_per_row, col0 = (g - row * groups_per_row) * 4;
    const int64_t plane = m * n;
    const int* src = partial + row * n + col0;
    int acc[4] = { 0, 0, 0, 0 };
    const bool vec = (n % 4 == 0);
    for (int s = 0; s < slices; ++s) {
        if (vec) {
            const int4 v = __ldcs(reinterpret_cast<const int4*>(src + (int64_t)s * plane));
            acc[0] += v.x; acc[1] += v.y; acc[2] += v.z; acc[3] += v.w;
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) if (col0 + j < n) acc[j] += src[(int64_t)s * plane + j];
        }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        if (col0 + j >= n) break;
        int* d = C + row * cs0 + (col0 + j) * cs1;
        int x = acc[j];
        if (add_c) x += *d;
        if (relu) x = max(x, 0);
        *d = x;
    }
}

}  // namespace

int launch_splitk_reduce(const void* partial, int slices, const accb_gemm_desc& d, void* c, const float* bias,
                         cudaStream_t stream, const char** err)
{
    const int64_t groups = d.m * ((d.n + 3) / 4);
    const int64_t blocks = (groups + 255) / 256;
    if (blocks > 0x7fffffff) { *err = "split-K reduction: problem too large"; return ACCB_ERR_ARG; }
    const int relu = d.epilogue == ACCB_EPI_RELU;
    const unsigned gsz = (unsigned)blocks;
    switch (d.c_type) {
    case ACCB_F32:
        (void)launch_pdl(splitk_reduce_f32_kernel<float>, dim3(gsz), dim3(256), stream, (const float*)partial, slices, d.m, d.n, (float*)c,
                         d.c_stride[0], d.c_stride[1], d.alpha, d.beta, bias, relu);
        break;
    case ACCB_F16:
        (void)launch_pdl(splitk_reduce_f32_kernel<__half>, dim3(gsz), dim3(256), stream, (const float*)partial, slices, d.m, d.n, (__half*)c,
                         d.c_stride[0], d.c_stride[1], d.alpha, d.beta, bias, relu);
        break;
    case ACCB_BF16:
        (void)launch_pdl(splitk_reduce_f32_kernel<__nv_bfloat16>, dim3(gsz), dim3(256), stream, (const float*)partial, slices, d.m, d.n,
                         (__nv_bfloat16*)c, d.c_stride[0], d.c_stride[1], d.alpha, d.beta, bias, relu);
        break;
    case ACCB_S32:
        (void)launch_pdl(splitk_reduce_s32_kernel, dim3(gsz), dim3(256), stream, (const int*)partial, slices, d.m, d.n, (int*)c, d.c_stride[0],
                         d.c_stride[1], (int)(d.beta != 0.0f), relu);
        break;
    default:
        *err = "split-K reduction: unsupported output type";
        return ACCB_ERR_ARG;
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { *err = cudaGetErrorString(e); return ACCB_ERR_CUDA; }
    note_launches(1);
    return 1;
}

}  // namespace accb
