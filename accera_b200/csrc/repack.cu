// Copies a GEMM operand whose rows are not 16-byte aligned into a buffer with an aligned pitch, so that the
// tensor-core path (TMA needs 16-byte aligned rows) can take it.  One kernel does the whole job - the copy, the zero
// columns that pad a row to the new width and the zero rows that pad K - and is launched with programmatic stream
// serialization, so that in a stream of GEMM calls it overlaps the tail of the kernel before it.
#include <cuda_runtime.h>
#include <stdint.h>

#include "accb_internal.h"

namespace accb {
namespace {

// One thread per 16-byte vector of the destination.  The source row starts on an element boundary only, so it is
// read element by element (consecutive threads read consecutive addresses); T is an unsigned type of the element size.
template <typename T>
__global__ void __launch_bounds__(256)
repack_rows_kernel(const uint8_t* __restrict__ src, int64_t src_pitch, int64_t rows, int64_t width,
                   uint8_t* __restrict__ dst, int64_t dst_pitch, int64_t dst_rows)
{
    pdl_enter();
    constexpr int kPer = 16 / (int)sizeof(T);
    const int64_t vec_per_row = dst_pitch / 16;
    const int64_t total = dst_rows * vec_per_row;
    for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < total; v += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = v / vec_per_row, c0 = (v - r * vec_per_row) * kPer;
        alignas(16) T e[kPer];
        const T* s = reinterpret_cast<const T*>(src + r * src_pitch);
#pragma unroll
        for (int i = 0; i < kPer; ++i) e[i] = (r < rows && c0 + i < width) ? s[c0 + i] : T(0);
        *reinterpret_cast<uint4*>(dst + r * dst_pitch + (c0 / kPer) * 16) = *reinterpret_cast<const uint4*>(e);
    }
}

}  // namespace

// src: `rows` rows of `width` elements of `elem_bytes` (1, 2 or 4) bytes, `src_pitch` BYTES apart; dst: `dst_rows` >= rows
// rows, `dst_pitch` bytes apart (a multiple of 16 covering `width` elements), 16-byte aligned; everything in dst that is
// not copied is set to zero.  Returns launches made or a negative ACCB_ERR_*.
int launch_repack_rows(const void* src, int64_t src_pitch, int64_t rows, int64_t width, int elem_bytes, void* dst,
                       int64_t dst_pitch, int64_t dst_rows, cudaStream_t stream, const char** err)
{
    const int64_t total = dst_rows * (dst_pitch / 16);
    if (total <= 0) return 0;
    int64_t blocks = (total + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;           // grid-stride beyond this
    cudaError_t e;
    const uint8_t* s = static_cast<const uint8_t*>(src);
    uint8_t* d = static_cast<uint8_t*>(dst);
    switch (elem_bytes) {
    case 1: e = launch_pdl(repack_rows_kernel<uint8_t>, dim3((unsigned)blocks), dim3(256), stream, s, src_pitch, rows, width, d, dst_pitch, dst_rows); break;
    case 2: e = launch_pdl(repack_rows_kernel<uint16_t>, dim3((unsigned)blocks), dim3(256), stream, s, src_pitch, rows, width, d, dst_pitch, dst_rows); break;
    case 4: e = launch_pdl(repack_rows_kernel<uint32_t>, dim3((unsigned)blocks), dim3(256), stream, s, src_pitch, rows, width, d, dst_pitch, dst_rows); break;
    default: *err = "repack: unsupported element size"; return ACCB_ERR_ARG;
    }
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) { *err = cudaGetErrorString(e); return ACCB_ERR_CUDA; }
    return 1;
}

}  // namespace accb
