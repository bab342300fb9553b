// Internal interfaces between the C-ABI layer (abi.cu) and the kernel files.
// Everything here takes DEVICE pointers and a stream; host staging, argument
// validation and error reporting live in abi.cu.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stddef.h>

#include "../../include/accera_b200.h"

namespace accb {

// Words of the per-device status buffer that kernels write to (never trap):
//   [0] gather: number of indices found outside [0, dim)
//   [1] tcgen05 GEMM: first bounded wait that ran out, encoded as
//       (site << 24) | (blockIdx.x & 0xffffff), 0 if none
//   [2] tcgen05 GEMM: k-block / tile the wait was at
//   [3] reserved
constexpr int kStatusWords = 4;
// The status buffer is followed by kPaceSlots counters: one per in-flight tensor-core GEMM launch,
// used to keep its persistent CTAs roughly in step (see gemm_umma.cu).
constexpr int kPaceSlots = 64;

struct GemmLaunch {
    accb_gemm_desc d;
    const void* a;
    const void* b;
    void* c;
    const float* bias;
    // additional destinations that receive the same result with the same layout (may be peer memory);
    // only the tensor-core path with a TMA-storable C supports them
    void* extra_c[7];
    int n_extra_c;
    // batched GEMM: `batch` independent problems of the same shape; operand i of problem b starts
    // b * *_batch_stride elements after the base (a stride of 0 shares that operand between all problems)
    int64_t batch = 1;
    int64_t a_batch_stride = 0, b_batch_stride = 0, c_batch_stride = 0;
    cudaStream_t stream;
    int* status;       // device pointer to kStatusWords ints
    int device;
    int num_sms;
};

// gemm_simt.cu: any supported type combination, any strides. Returns launches made (<0: ACCB_ERR_*).
int launch_gemm_simt(const GemmLaunch& g, const char** err);

// gemm_umma.cu: tcgen05/TMEM path. `supported` explains in *why when it returns false.
bool gemm_umma_supported(const GemmLaunch& g, const char** why);
// want_two_sm: 1 = CTA pairs (cta_group::2), 0 = single CTAs, -1 = whichever tile shape suits the problem.
int launch_gemm_umma(const GemmLaunch& g, int want_two_sm, const char** err);
// host only: the tile shape launch_gemm_umma would pick (from d, batch, num_sms, max_ctas) and the rounds of tiles it gives
void gemm_umma_tile_plan(const GemmLaunch& g, int want_two_sm, int* two_sm, int* tile_cols, int64_t* tiles, int64_t* rounds);

// reduce_mean.cu
// Scratch (fp32 partial sums) a launch needs for these dims, in bytes; 0 when the
// single-pass kernels are used.
size_t reduce_mean_scratch_bytes(int64_t d0, int64_t d1, int64_t d2, int axes_mask, int num_sms);
int launch_reduce_mean(const float* data, int64_t d0, int64_t d1, int64_t d2, float* reduced, int axes_mask,
                       float* scratch, size_t scratch_bytes, int num_sms, cudaStream_t stream, const char** err);

// gather.cu
int launch_gather(const void* data, int64_t d0, int64_t d1, const int64_t* indices, int64_t i0, int64_t i1,
                  void* output, int axis, int elem_bytes, int* status, cudaStream_t stream, const char** err);

// range.cu: output[i] = start + i rounded additions of delta (bit-identical to the serial recurrence); writes the
// value after n additions to *final_value (host memory).  range_count_f32 is host-only.
int64_t range_count_f32(float start, float limit, float delta);
int64_t range_plan_f32(float start, float delta, int64_t n, int64_t* first, uint32_t* bits, int32_t* step, int64_t capacity,
                       float* final_value);
int launch_range_f32(int64_t n, float* output, float start, float delta, float* final_value, cudaStream_t stream,
                     const char** err);

// counts kernels launched (reported by accb_launch_count)
void note_launches(int n);

// records `msg` as the calling thread's last error (what accb_last_error returns) and returns `code`
int set_error(int code, const char* msg);

}  // namespace accb
