// Internal interfaces between the C-ABI layer (abi.cu) and the kernel files.
// Everything here takes DEVICE pointers and a stream; host staging, argument
// validation and error reporting live in abi.cu.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stddef.h>

#include "../../include/accera_b200.h"

namespace accb {

// Words of the per-device status buffer that kernels write to (never trap).  Every launch that can fail on the
// device carries a launch id (next_launch_id), so that a failure is attributed to the launch that had it and a
// stale, not yet collected failure of an earlier launch neither aborts nor mislabels a later one.
//   [0] gather: number of indices found outside [0, dim) since the last collection
//   [1] tcgen05 GEMM: first bounded wait that ran out, (site << 24) | (blockIdx.x & 0xffffff)
//   [2] tcgen05 GEMM: k-block / tile that wait was at
//   [3] tcgen05 GEMM: launch id of the launch that recorded [1] and [2]; 0 = no failure recorded
//   [4] tcgen05 GEMM: number of waits that ran out since the last collection (all launches)
//   [5] gather: launch id of the last launch that met a bad index
constexpr int kStatusWords = 8;
enum { ST_GATHER_COUNT = 0, ST_GEMM_SITE = 1, ST_GEMM_STEP = 2, ST_GEMM_ID = 3, ST_GEMM_COUNT = 4, ST_GATHER_ID = 5 };
// The status buffer is followed by kPaceSlots counters: one per in-flight tensor-core GEMM launch,
// used to keep its persistent CTAs roughly in step (see gemm_umma.cu).
constexpr int kPaceSlots = 64;

// a fresh non-zero launch id (process-wide, 31 bits, wraps past zero)
int next_launch_id();

// Per-thread overrides of what the launch code would choose by itself (accb_set_option): used by the tests to
// reach every code path on small problems, by tuning runs, and by the time-out self-test.  Zero-initialised =
// "choose as usual".
struct Options {
    int gemm_tile_cols = 0;          // 128 | 256: accumulator columns per tile
    int gemm_staged_store = -1;      // epilogue: 0 stores straight from registers, 1 shared-memory staging + TMA stores,
                                     // 2 staging boxes moved by the epilogue warps themselves
    int gemm_pace_pct = -1;          // tile-by-tile pacing of the persistent CTAs: 0 off, 1..100 on
    int gemm_group_m = 0;            // tile rows visited together
    int gemm_hint_a = 0, gemm_hint_b = 0;   // L2 eviction priority of the operand loads (1 evict-first, 2 evict-last)
    int gemm_c_stream = 0;           // streaming (evict-first) accesses to C
    int gemm_peer_store = -1;        // replicated GEMM: 0 = TMA stores to every replica, 1 = register stores to the peers
    int gemm_copy_ctas = -1;         // replicated GEMM: CTAs that forward finished tiles to the replicas (0 = none: the
                                     // computing CTAs' epilogues store to every replica themselves)
    int gemm_wait_limit_us = 0;      // limit of every bounded device-side wait (default: one second)
    int gemm_test_drop_commit = 0;   // self-test: the MMA issuer leaves out the commit that completes the last accumulator
    int gemm_pdl = -1;               // programmatic dependent launch of the tensor-core GEMM: 0 off, 1 on
    int gemm_epi_warps = 0;          // epilogue with warp-moved boxes: 0 / 8 = eight epilogue warps, 4 = four
    int gemm_split_k = -1;           // K slices of few-tile problems: -1 cost model, 0 never, n >= 2 exactly n when possible
    int gemm_c_in = -1;              // beta != 0 with warp-moved boxes: old C copied into the boxes ahead of use (1) or read row by row (0)
    int gemm_verbose = 0;            // print the launch plan to stderr
    int host_stage_chunks = 0;       // row chunks of the staged host-pointer GEMM (default 16)
    int reduce_rows_tpr = 0;         // reduce_mean over contiguous segments: threads per output (32, 64, 128 or 256)
    int stream_pdl = -1;             // programmatic dependent launch of the reduce / gather / range kernels: 0 off, 1 on
};
Options& options();

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
    // per-tile completion counters for a replicated launch with forwarding CTAs (device memory, this launch's own
    // region; the launch code zeroes what it uses), null = not available
    int* tile_flags = nullptr;
    int64_t tile_flags_capacity = 0;
    // batched GEMM: `batch` independent problems of the same shape; operand i of problem b starts
    // b * *_batch_stride elements after the base (a stride of 0 shares that operand between all problems)
    int64_t batch = 1;
    int64_t a_batch_stride = 0, b_batch_stride = 0, c_batch_stride = 0;
    int force_tile_cols = 0;   // tensor-core path: 128 or 256 accumulator columns per tile instead of the cost model's choice
    bool no_split_k = false;   // row chunks of one staged host-pointer GEMM: every chunk must round like a single launch would
    cudaStream_t stream;
    int* status;       // device pointer to kStatusWords ints
    int launch_id;     // attribution of device-side failures (next_launch_id)
    int device;
    int num_sms;
};

// Launch with programmatic stream serialization: the kernel may be scheduled while the kernel before it in the
// stream is still draining, which hides the launch and block-scheduling latency of back-to-back launches.  The
// kernel must execute pdl_enter() before it touches global memory: that returns once everything earlier in the
// stream has completed (at once for an ordinary predecessor).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, cudaStream_t stream, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = 0; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = options().stream_pdl == 0 ? 0 : 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_enter()
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
#endif

// gemm_simt.cu: any supported type combination, any strides. Returns launches made (<0: ACCB_ERR_*).
int launch_gemm_simt(const GemmLaunch& g, const char** err);

// gemm_umma.cu: tcgen05/TMEM path. `supported` explains in *why when it returns false.
bool gemm_umma_supported(const GemmLaunch& g, const char** why);
bool gemm_umma_types_supported(const accb_gemm_desc& d);   // element types only, whatever the layout
// want_two_sm: 1 = CTA pairs (cta_group::2), 0 = single CTAs, -1 = whichever tile shape suits the problem.
int launch_gemm_umma(const GemmLaunch& g, int want_two_sm, const char** err);
// host only: the tile shape launch_gemm_umma would pick (from d, batch, num_sms, max_ctas) and the rounds of tiles it gives
void gemm_umma_tile_plan(const GemmLaunch& g, int want_two_sm, int* two_sm, int* tile_cols, int64_t* tiles, int64_t* rounds);
// host only: grid, block and dynamic shared memory of the launch launch_gemm_umma would make (out[0..2] grid,
// out[3..5] block, out[6] dynamic shared-memory bytes, out[7] pipeline stages)
void gemm_umma_launch_geometry(const GemmLaunch& g, int want_two_sm, int32_t out[8]);

// gemm_splitk.cu: C <- epi(alpha * sum of `slices` dense row-major M x N partials (fp32, or int32 for an int32 C) + beta * C + bias)
int launch_splitk_reduce(const void* partial, int slices, const accb_gemm_desc& d, void* c, const float* bias,
                         cudaStream_t stream, const char** err);

// repack.cu: copy of an operand into rows with a 16-byte aligned pitch, zero-padded (see the file)
int launch_repack_rows(const void* src, int64_t src_pitch, int64_t rows, int64_t width, int elem_bytes, void* dst,
                       int64_t dst_pitch, int64_t dst_rows, cudaStream_t stream, const char** err);

// reduce_mean.cu
// Scratch (fp32 partial sums) a launch needs for these dims, in bytes; 0 when the
// single-pass kernels are used.
// `cols_blocks_per_sm`: how many blocks per SM a strided (column) reduction is split into.  More blocks need more
// partial sums and a longer second pass: 8 per SM was measured slower than 2 on every shape tried (4096 x 8192 over
// the rows: 32.8 us against 30.3; 64 x 512 x 1024 over the middle axis: 30.7 against 22.8, because it starts to
// split at all).  The entry point with the fixed built-in scratch depends on this number: keep the two in step.
constexpr int kColsBlocksPerSm = 2;
constexpr int kNoAllocColsBlocksPerSm = 2;
size_t reduce_mean_scratch_bytes(int64_t d0, int64_t d1, int64_t d2, int axes_mask, int num_sms,
                                 int cols_blocks_per_sm = kColsBlocksPerSm);
int launch_reduce_mean(const float* data, int64_t d0, int64_t d1, int64_t d2, float* reduced, int axes_mask,
                       float* scratch, size_t scratch_bytes, int num_sms, cudaStream_t stream, const char** err,
                       int cols_blocks_per_sm = kColsBlocksPerSm);

// gather.cu
int launch_gather(const void* data, int64_t d0, int64_t d1, const int64_t* indices, int64_t i0, int64_t i1,
                  void* output, int axis, int elem_bytes, int* status, int launch_id, cudaStream_t stream, const char** err);

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
// forgets the calling thread's last error (every entry point starts with this)
void clear_error();
// the device this thread's calls run on: the one chosen with accb_set_device (made current here), else the current
// CUDA device.  Returns ACCB_OK or an error code (with the error text recorded).
int selected_device(int* dev);

}  // namespace accb
