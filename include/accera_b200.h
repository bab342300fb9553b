/*
 * accera_b200 - C ABI of the B200 (sm_100a) launch layer behind HAT packages.
 *
 * A HAT package built by accera_b200.Package exports, per function, exactly the
 * prototype the reference compiler would have exported
 *     void <base_name>_<16 hex>(T_in* A, T_in* B, T_out* C);            (GEMM family)
 *     void <name>(int64_t dims..., float* out, float* data, int64_t* indices);   (gather)
 * and each of those thin stubs forwards into one of the entry points declared
 * here.  Everything is extern "C", plain pointers and sizes, no C++ or torch types.
 *
 * Pointers may be host or device addresses.  Host buffers are staged through a
 * cached device workspace and the call returns after the result is back in host
 * memory; device buffers are used in place, the kernel is enqueued on the stream
 * selected with accb_set_stream() and the call returns without synchronising
 * (like the launcher the reference generates, which only launches).
 *
 * Every entry point returns 0 on success or a negative ACCB_ERR_* code; the text
 * of the last error on the calling thread is available from accb_last_error().
 * There is no CPU fallback: without a usable CUDA device every compute entry
 * point fails with ACCB_ERR_CUDA.
 */
#ifndef ACCERA_B200_H
#define ACCERA_B200_H

#if defined(__cplusplus)
#include <cstdint>
extern "C" {
#else
#include <stdint.h>
#endif

/* element types (storage) */
enum {
    ACCB_F32 = 0,
    ACCB_F16 = 1,
    ACCB_BF16 = 2,
    ACCB_S8 = 3,
    ACCB_S32 = 4,
    ACCB_U8 = 5,
    ACCB_S16 = 6   /* int16 inputs accumulate exactly into int32 on the CUDA cores (no tensor-core path) */
};

/* how a GEMM is computed */
enum {
    ACCB_COMPUTE_AUTO = 0,   /* tensor cores for f16/bf16/s8/u8 inputs, fp32 SIMT for f32 inputs */
    ACCB_COMPUTE_SIMT = 1,   /* CUDA-core FMA in fp32 / int32: bit-faithful fp32; the only path for int16 inputs */
    ACCB_COMPUTE_TENSOR = 2, /* tcgen05: f16/bf16 -> f32, s8/u8 -> s32, f32 inputs as TF32 */
    ACCB_COMPUTE_TENSOR_2SM = 3, /* tcgen05 with CTA pairs (cta_group::2); same numerics as TENSOR */
    ACCB_COMPUTE_TENSOR_PREFERRED = 4 /* tcgen05 when the operand layout allows it (K-contiguous A and B,
                                         16-byte row pitch), otherwise the SIMT kernel: what a tensorized
                                         plan asks for, whatever the array layouts are */
};

/* fused epilogue applied to the accumulator before it is stored
 * (reference: MMAFragmentOp, accera/ir/include/value/ValueMMAOp.h:64-71) */
enum {
    ACCB_EPI_NONE = 0,
    ACCB_EPI_RELU = 1
};

enum {
    ACCB_OK = 0,
    ACCB_ERR_ARG = -1,       /* bad descriptor, null pointer, unsupported combination */
    ACCB_ERR_CUDA = -2,      /* a CUDA call failed (no device, out of memory, launch error) */
    ACCB_ERR_INDEX = -3,     /* gather met an index outside [0, dim): that row was zero-filled */
    ACCB_ERR_TIMEOUT = -4,   /* a bounded device-side wait ran out; results are invalid */
    ACCB_ERR_LIMIT = -5      /* a fixed-capacity resource is too small for the request */
};

/*
 * GEMM with fused epilogue:   C <- epi(alpha * (A @ B) + beta * C + bias[j])
 *
 * Replaces the reference's generated GEMM kernels and their launchers
 * (accera/transforms/src/exec/ExecutionPlanToAffineLoweringPass.cpp:5986-6533,
 *  accera/acc-translate/src/Target/Cpp/GpuDialectCppPrinter.cpp:426-561); the
 * nest it implements is README.md:61-76 (C is INPUT_OUTPUT, i.e. beta = 1).
 * A is M x K, B is K x N, C is M x N; strides are in elements and are the
 * affine_map of the .hat argument (row-major {ld,1}, column-major {1,ld}).
 */
typedef struct accb_gemm_desc {
    int64_t m, n, k;
    int32_t a_type, b_type, c_type; /* ACCB_F32 ... */
    int32_t compute;                /* ACCB_COMPUTE_* */
    int64_t a_stride[2];
    int64_t b_stride[2];
    int64_t c_stride[2];
    float alpha;
    float beta;
    int32_t epilogue;               /* ACCB_EPI_* */
    int32_t max_ctas;               /* tensor-core path: upper bound on the persistent grid (0 = one CTA per SM).
                                       Leaving a few SMs free lets a collective running on another stream
                                       make progress while the GEMM computes. */
} accb_gemm_desc;

/* bias may be NULL; when given it is n fp32 values added to every row before the ReLU.
 * Memory: host-pointer calls stage through a cached per-device workspace.  A device-pointer call allocates only in two
 * cases, both from the stream-ordered allocator on the launch stream (freed on it right after the launch): 16-bit or
 * 8-bit operands whose rows are not 16-byte aligned are repacked into aligned rows for the tensor cores, and few-tile
 * long-K problems that are split along K keep their fp32 partial sums there. */
int accb_gemm(const accb_gemm_desc* desc, const void* a, const void* b, void* c, const float* bias);

/*
 * Batched GEMM: `batch` independent problems of the shape, types, strides and epilogue in `desc`,
 *     C[b] <- epi(alpha * (A[b] @ B[b]) + beta * C[b] + bias[j]),   b = 0 .. batch-1,
 * in one call (on the tensor cores: one persistent launch that walks all problems' tiles).
 *
 * Replaces the kernels the reference generates for the rank-3 nest
 *     C[b, i, j] += A[b, i, k] * B[b, k, j]
 * (accera/python/accera/test/mfma_tests.py:435-466; tensorised at :486-499).
 * X[b] starts b * x_batch_stride elements after the base pointer; for the nest above with dense
 * first-major arrays these are M*K, K*N and M*N.  a_batch_stride or b_batch_stride may be 0: that
 * operand is then shared by all problems.  c_batch_stride must be at least the extent of one C.
 * bias (n values, may be NULL) is shared by all problems.  The tensor-core path additionally needs
 * batch strides of A and B that are multiples of 16 bytes; ACCB_COMPUTE_TENSOR_PREFERRED and
 * ACCB_COMPUTE_AUTO fall back to the SIMT kernels otherwise.  Host or device pointers as for accb_gemm.
 */
int accb_gemm_batched(const accb_gemm_desc* desc, int64_t batch, int64_t a_batch_stride, int64_t b_batch_stride,
                      int64_t c_batch_stride, const void* a, const void* b, void* c, const float* bias);

/*
 * Host-only helper (no counterpart in the reference; touches no CUDA state, works without a GPU): the tile shape
 * the tensor-core path picks for `desc` x `batch` on a device with `num_sms` SMs - *cta_pairs = 1 for 256-row tiles
 * computed by two CTAs (cta_group::2), 0 for 128-row single-CTA tiles; *tile_cols = 256 or 128 - with the number of
 * tiles and of rounds the persistent grid needs for them.  desc->compute fixes the CTA mode for ACCB_COMPUTE_TENSOR
 * (single) and ACCB_COMPUTE_TENSOR_2SM (pairs) and leaves it to the cost model otherwise.  Returns ACCB_ERR_ARG for a
 * null pointer or non-positive sizes.
 */
int accb_gemm_tile_plan(const accb_gemm_desc* desc, int64_t batch, int32_t num_sms, int32_t* cta_pairs, int32_t* tile_cols,
                        int64_t* tiles, int64_t* rounds);

/*
 * Host-only helper (no GPU needed): the launch the tensor-core path makes for `desc` x `batch` on a device with
 * `num_sms` SMs - grid[3], block[3] and the dynamic shared memory of the kernel.  This is the information the
 * reference records per GPU function as launch_parameters / dynamic_shared_mem_bytes
 * (accera/python/accera/Package.py:714-743, derived there from accera/python/accera/lang/Plan.py:879-956); here the
 * kernel is persistent, so the grid follows from the SM count and the tile plan, not from the problem alone.
 */
int accb_gemm_launch_geometry(const accb_gemm_desc* desc, int64_t batch, int32_t num_sms, int32_t* grid, int32_t* block,
                              int32_t* dynamic_shared_mem_bytes);

/*
 * The same GEMM on the tensor cores, with the result stored to several replicas of C at once.
 * (No counterpart in the reference, which has no multi-GPU path.)  c_replicas[0] is the local C: it is
 * read when beta != 0 and written; c_replicas[1..n_replicas-1] receive the same values with the same
 * layout and are only written.  They may be another GPU's memory mapped into this process (peer /
 * symmetric memory): every output tile is then pushed over NVLink from inside the GEMM kernel, so an
 * M-row sharded GEMM reassembles C on all GPUs without a separate all-gather.  With 1 or 2 extra
 * replicas the computing CTAs' epilogues TMA-store each staged box to every replica; with 3 or more,
 * a few CTAs of the same launch (18, or 32 from 6 extra replicas on) do no math and forward finished
 * tiles instead: they wait for a tile's completion counter, TMA-load the tile from the local C (L2)
 * into a shared-memory ring and write it to every other replica with 16-byte stores - stores that
 * wait for NVLink credit then never stall an SM that feeds the tensor cores.  Peer memory is only
 * ever stored to, never loaded from.  "gemm.copy_ctas" overrides the number of forwarding CTAs.
 * Device pointers only; C must be row-major with a 16-byte aligned pitch and base; 1 <= n_replicas <= 8.
 * The kernel's stores have completed when the launch has completed on its stream; making them visible
 * to the other GPUs' later work (a barrier between the ranks) is the caller's job.
 */
int accb_gemm_replicated(const accb_gemm_desc* desc, const void* a, const void* b, void* const* c_replicas,
                         int32_t n_replicas, const float* bias);

/*
 * ReduceMean over a dense first-major rank-3 fp32 array.
 * Replaces the nests of kernels/reduce_mean/naive_runtime_sized.py:66-148.
 * axes_mask bit d set = dimension d is averaged away.  `reduced` holds the kept
 * dimensions densely, first-major (keepdims only changes the shape reported by
 * accb_reduce_mean_rank3_dims, not the element order).
 */
int accb_reduce_mean_rank3(const float* data, int64_t d0, int64_t d1, int64_t d2, float* reduced, int32_t axes_mask);

/*
 * ReduceMean for callers that must not see a device allocation happen inside the call.
 * (No counterpart in the reference: it has no GPU reduce_mean and no allocation contract.)
 *
 * accb_reduce_mean_rank3 may grow a cached scratch buffer with cudaMalloc when a reduction has
 * too few outputs to fill the GPU and is split over blocks.  That is wrong for a host that owns
 * all of device memory itself - an inference server or framework that wraps a HAT function as a
 * custom operator and hands it buffers from its own arena (a hidden cudaMalloc escapes the arena's
 * accounting, can fail when the arena already holds nearly all of HBM, and synchronises the whole
 * device in the middle of a serving loop) - and for code that runs after such a host has frozen
 * allocation.  This variant computes the same result with the same kernels but keeps the partial
 * sums in a 256 KiB array compiled into the library, and calls no cudaMalloc, cudaFree or any
 * other allocating routine.
 *
 *  - data and reduced must be DEVICE pointers (there is no staging here); the work is enqueued on
 *    cuda_stream (a cudaStream_t, NULL = default stream) of the current device and not synchronised.
 *  - A shape whose split reduction needs more than 256 KiB of partial sums is rejected with
 *    ACCB_ERR_LIMIT (nothing is launched).  On a 148-SM part the planner asks for at most about
 *    300 KiB, and only for very wide, short column reductions (tens of thousands of outputs, each
 *    split in two); everything else fits.  Use accb_reduce_mean_rank3 for the rejected shapes.
 *  - The first call on each device resolves the array's device address (cudaGetSymbolAddress), so
 *    make that first call during set-up, before any stream capture begins.
 *  - Every call on a device shares the one array, and it keeps whatever the previous call left:
 *    each call overwrites every partial sum it later reads, so nothing needs clearing, but two
 *    calls that overlap on the GPU (different streams, no ordering) race on it - serialise them.
 *  - Every GPU that loads the library holds the 256 KiB until the process exits.
 */
int accb_reduce_mean_rank3_noalloc(const float* data, int64_t d0, int64_t d1, int64_t d2, float* reduced,
                                   int32_t axes_mask, void* cuda_stream);

/* host-only helper: writes the output dims, returns the output rank (1..3) */
int accb_reduce_mean_rank3_dims(int64_t d0, int64_t d1, int64_t d2, int32_t axes_mask, int32_t keepdims,
                                int64_t* out_dims);

/*
 * Gather with rank-2 data and rank-2 int64 indices, dense first-major.
 * Replaces the nests of kernels/gather/naive_runtime_sized.py:26-49 and
 * accera/python/accera/test/dsl_tests.py:1596-1601, 1642-1647.
 *   axis 0: output[i,j,k] = data[indices[i,j], k]     output is (i0, i1, d1)
 *   axis 1: output[i,j,k] = data[i, indices[j,k]]     output is (d0, i0, i1)
 * elem_bytes is 1, 2, 4 or 8; elements are copied bit for bit.  Like the
 * reference, negative indices are not supported; unlike it, an index outside
 * [0, dim) is not dereferenced: the element is zero-filled and the call reports
 * ACCB_ERR_INDEX (host buffers: from this call; device buffers: from the next
 * accb_synchronize()).
 */
int accb_gather_rank2(const void* data, int64_t d0, int64_t d1, const int64_t* indices, int64_t i0, int64_t i1,
                      void* output, int32_t axis, int32_t elem_bytes);

/* host-only helper: output dims of the gather above */
int accb_gather_rank2_dims(int64_t d0, int64_t d1, int64_t i0, int64_t i1, int32_t axis, int64_t* out_dims);

/*
 * Range (the ONNX operator), fp32.  Replaces the two functions of the reference's range-node test
 * (accera/python/accera/test/dsl_tests.py:1436-1506; prototype kernels/range/naive_runtime_sized.py:11-41):
 *   get_size:    *size = (int64) floor((limit - start) / delta), evaluated in fp32
 *   get_result:  for i in [0, n): output[i] = *start; *start = *start + delta   (one rounded fp32 addition per
 *                element, in index order; the scalar is an in/out argument and ends as the value after n additions)
 * accb_range_f32 produces exactly the values of that serial loop, bit for bit, for any start, delta and n.
 * `output` is a host or device pointer to n floats; `start_inout` is always a HOST pointer (it is the by-pointer
 * scalar argument of the HAT prototype) and is updated before the call returns, also for device output.
 * accb_range_count_f32 is host-only; a quotient that is negative, NaN or beyond int64 gives 0.
 */
int64_t accb_range_count_f32(float start, float limit, float delta);
int accb_range_f32(int64_t n, float* output, float* start_inout, float delta);

/*
 * Host-only helper (no counterpart in the reference): the plan accb_range_f32 executes.  The n values of the serial
 * loop fall into segments inside which consecutive fp32 BIT PATTERNS differ by a constant: element i of segment j
 * (first[j] <= i < first[j+1], the last segment runs to n) has the bit pattern bits[j] + (i - first[j]) * step[j]
 * (32-bit wrap-around arithmetic).  Writes at most `capacity` segments (any of the arrays may be NULL), returns the
 * number of segments of the full plan, and stores the running value after n additions to *final_value if non-NULL.
 */
int64_t accb_range_plan_f32(float start, float delta, int64_t n, int64_t* first, uint32_t* bits, int32_t* step,
                            int64_t capacity, float* final_value);

/*
 * Runtime control.  These replace what the reference leaves to its loader
 * (device selection and synchronisation, tools/benchmarkers/accera_gemm.py:612-626)
 * and accera/runtime; none of them appears in a HAT prototype.
 */
int accb_set_device(int32_t device);      /* device used by this thread's following calls (made current); -1 = no
                                             selection, follow the current CUDA device again */
int accb_get_device(void);                /* this thread's selection, -1 if none */
int accb_current_device(void);            /* the CUDA runtime's current device of this thread, or ACCB_ERR_CUDA */
int accb_set_stream(void* cuda_stream);   /* cudaStream_t used for device-pointer calls; NULL = default stream */
int accb_synchronize(void);               /* wait for the selected stream; reports deferred device-side errors */
const char* accb_last_error(void);        /* text of the last error on this thread ("" if none) */
int64_t accb_launch_count(void);          /* kernels launched by this library so far (all threads) */
int accb_release_workspace(void);         /* free the cached staging buffers of the current device */
int accb_device_count(void);              /* number of visible CUDA devices, 0 if none / no driver */
const char* accb_version(void);

/*
 * Errors that happen ON the device - a bounded wait of the tensor-core GEMM that ran out (ACCB_ERR_TIMEOUT), a
 * gather index outside the data (ACCB_ERR_INDEX) - are written by the kernel into a per-device status record
 * together with the id of the launch that had them.  A call on HOST pointers is synchronous and returns its own
 * launches' errors.  A call on DEVICE pointers only enqueues work: its device-side errors are DEFERRED and are
 * returned (and cleared) by the next accb_synchronize() on that device; they are never attributed to a later call,
 * and a failure that has not been collected yet does not disturb later launches.
 *
 * Per-thread overrides of choices the launch code otherwise makes by itself.  They exist so that tests reach every
 * code path on small problems, for tuning runs, and for the self-test of the time-out path; none is needed in
 * normal use and none has a counterpart in the reference.  accb_set_option("reset", 0) restores all defaults.
 *   "gemm.tile_cols"         0 (choose) | 128 | 256   accumulator columns per tile of the tensor-core GEMM
 *   "gemm.staged_store"      -1 (choose) | 0 | 1 | 2  epilogue from registers (0), through shared-memory boxes stored by TMA (1),
 *                                                     or through boxes that the epilogue warps move themselves (2)
 *   "gemm.pace_pct"          -1 (choose) | 0..100     tile-by-tile pacing of the persistent CTAs
 *   "gemm.group_m"           0 (choose) | rows        tile rows visited together
 *   "gemm.hint_a" / "gemm.hint_b"   0 | 1 | 2         L2 eviction priority of the operand loads
 *   "gemm.c_stream"          0 | 1                    streaming accesses to C
 *   "gemm.peer_store"        -1 (choose) | 0 | 1      accb_gemm_replicated: TMA stores (0) or register stores (1) to peers
 *   "gemm.copy_ctas"         -1 (choose) | 0..128     accb_gemm_replicated: CTAs set aside to forward finished tiles to the
 *                                                     replicas (0: the computing CTAs store to every replica themselves)
 *   "gemm.wait_limit_us"     0 (one second) | us      limit of every bounded device-side wait
 *   "gemm.test_drop_commit"  0 | 1                    self-test: each CTA's last accumulator is never signalled complete,
 *                                                     so the epilogue's bounded wait runs out and the launch reports
 *                                                     ACCB_ERR_TIMEOUT (no fault, no trap; the context stays usable)
 *   "gemm.pdl"               -1 (on) | 0 | 1          programmatic dependent launch: the next GEMM of a stream is scheduled
 *                                                     and sets itself up while the previous kernel still runs
 *   "gemm.epi_warps"         0 (choose) | 4 | 8       epilogue warps of a launch with warp-moved boxes
 *   "gemm.split_k"           -1 (choose) | 0 | n      K slices of a few-tile problem: cost model, never, or exactly n when n divides K
 *   "gemm.c_in"              -1 (choose) | 0 | 1      beta != 0 with warp-moved boxes: the old C is copied into the boxes ahead
 *                                                     of its use (1) or read row by row when needed (0)
 *   "gemm.verbose"           0 | 1                    print the launch plan to stderr
 *   "stream_kernels.pdl"     -1 (on) | 0 | 1          programmatic dependent launch of the reduce_mean, gather and range kernels
 *   "host_gemm.stage_chunks" 0 (16) | 1..256          row chunks of the staged host-pointer GEMM
 *   "reduce.rows_threads_per_output"  0 (choose) | 32 | 64 | 128 | 256   reduce_mean over contiguous segments
 */
int accb_set_option(const char* name, int64_t value);

/* Test hook: decodes eight status words as the library would (what: 0 everything, 1 the GEMM launch `launch_id`,
 * 2 the gather launch `launch_id`); returns the ACCB_* code and writes the message.  Host only. */
int accb_debug_decode_status(const int32_t* words, int32_t what, int32_t launch_id, char* message, int32_t capacity);

#if defined(__cplusplus)
} /* extern "C" */
#endif

#endif /* ACCERA_B200_H */
