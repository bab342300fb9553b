// C-ABI layer: argument validation, host<->device staging, kernel selection and
// error reporting for the entry points declared in include/accera_b200.h.
//
// The reference leaves all of this to its loader: a generated GPU host function
// only launches (docs/Tutorials/GPU/Hello_MatMul_GPU.md:143-158) and hatlib copies
// numpy buffers to and from the device around it.  Here one call does both jobs:
// host pointers are staged through a cached per-device workspace (and the call
// is synchronous), device pointers are used in place on the selected stream.
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>

#include "accb_internal.h"

namespace accb {

static std::atomic<int64_t> g_launches{0};
void note_launches(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

int next_launch_id()
{
    static std::atomic<uint32_t> next{1};
    for (;;) {
        const int id = (int)(next.fetch_add(1, std::memory_order_relaxed) & 0x7fffffffu);
        if (id != 0) return id;
    }
}

Options& options()
{
    thread_local Options o;
    return o;
}

namespace {

constexpr int kMaxDevices = 64;
constexpr int64_t kTileFlagInts = 1 << 18;   // 1 MiB of per-tile counters per device, shared by the replicated launches in flight

thread_local std::string t_error;
thread_local int t_device = -1;             // -1: use the current CUDA device
thread_local cudaStream_t t_stream = nullptr;

int fail(int code, const std::string& msg)
{
    t_error = msg;
    return code;
}

int fail_cuda(const char* what, cudaError_t e)
{
    (void)cudaGetLastError();
    return fail(ACCB_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
}

// Per-device state: status words written by kernels, a cached staging workspace
// for host-pointer calls and a scratch buffer for multi-pass kernels.
struct DeviceState {
    std::mutex mu;
    bool ready = false;
    int num_sms = 0;
    int* status = nullptr;          // device, kStatusWords ints
    int* status_host = nullptr;     // pinned mirror
    void* slot[4] = { nullptr, nullptr, nullptr, nullptr };   // staging: A/data, B/indices, C/output, bias
    size_t slot_bytes[4] = { 0, 0, 0, 0 };
    void* scratch = nullptr;
    size_t scratch_bytes = 0;
    // the scratch buffer is shared by all streams of the device: a launch that uses it on another stream than
    // the previous user first waits (on the device) for that user's kernels
    cudaEvent_t scratch_done = nullptr;
    cudaStream_t scratch_stream = nullptr;
    bool scratch_used = false;
    // per-tile completion counters of replicated GEMM launches: a ring that launches take regions from
    int* tile_flags = nullptr;
    int64_t tile_flags_cursor = 0;
    cudaStream_t pipe[2] = { nullptr, nullptr };   // staging pipeline of large host-pointer GEMMs
    cudaEvent_t pipe_ready = nullptr;              // B (and bias) have arrived
};
DeviceState g_dev[kMaxDevices];

int current_device(int* dev)
{
    if (t_device >= 0) {
        cudaError_t e = cudaSetDevice(t_device);
        if (e != cudaSuccess) return fail_cuda("cudaSetDevice", e);
        *dev = t_device;
        return ACCB_OK;
    }
    cudaError_t e = cudaGetDevice(dev);
    if (e != cudaSuccess) return fail_cuda("no usable CUDA device (cudaGetDevice)", e);
    return ACCB_OK;
}

int device_state(DeviceState** out, int* dev_out)
{
    int dev = 0;
    int rc = current_device(&dev);
    if (rc != ACCB_OK) return rc;
    if (dev < 0 || dev >= kMaxDevices) return fail(ACCB_ERR_ARG, "device index out of range");
    DeviceState& s = g_dev[dev];
    std::lock_guard<std::mutex> lock(s.mu);
    if (!s.ready) {
        cudaDeviceProp prop;
        cudaError_t e = cudaGetDeviceProperties(&prop, dev);
        if (e != cudaSuccess) return fail_cuda("cudaGetDeviceProperties", e);
        if (prop.major != 10) {
            char buf[160];
            snprintf(buf, sizeof buf, "device %d is sm_%d%d; this library contains sm_100a code only", dev, prop.major, prop.minor);
            return fail(ACCB_ERR_CUDA, buf);
        }
        s.num_sms = prop.multiProcessorCount;
        e = cudaMalloc(&s.status, (kStatusWords + kPaceSlots) * sizeof(int));
        if (e != cudaSuccess) return fail_cuda("cudaMalloc(status)", e);
        e = cudaMemset(s.status, 0, (kStatusWords + kPaceSlots) * sizeof(int));
        if (e != cudaSuccess) return fail_cuda("cudaMemset(status)", e);
        e = cudaMallocHost(&s.status_host, kStatusWords * sizeof(int));
        if (e != cudaSuccess) return fail_cuda("cudaMallocHost(status)", e);
        s.ready = true;
    }
    *out = &s;
    if (dev_out) *dev_out = dev;
    return ACCB_OK;
}

bool is_device_pointer(const void* p)
{
    if (!p) return false;
    cudaPointerAttributes a;
    cudaError_t e = cudaPointerGetAttributes(&a, p);
    if (e != cudaSuccess) { (void)cudaGetLastError(); return false; }
    return a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged;
}

int ensure(void** buf, size_t* have, size_t need)
{
    if (need <= *have) return ACCB_OK;
    if (*buf) { cudaFree(*buf); *buf = nullptr; *have = 0; }
    size_t want = need + need / 8;   // a little slack so that slowly growing sizes do not reallocate every call
    cudaError_t e = cudaMalloc(buf, want);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        e = cudaMalloc(buf, need);
        want = need;
    }
    if (e != cudaSuccess) return fail_cuda("cudaMalloc(staging workspace)", e);
    *have = want;
    return ACCB_OK;
}

// Reads the status words back (synchronises `stream`) and turns them into an error code.
//   what = COLLECT_GEMM / COLLECT_GATHER: a synchronous host-pointer call asks about its own launches only
//          (launch id `id`); a failure an earlier device-pointer launch left behind stays recorded for
//          accb_synchronize and does not become this call's result.
//   what = COLLECT_ALL: accb_synchronize reports whatever is recorded.
// What is reported is cleared.
enum { COLLECT_ALL = 0, COLLECT_GEMM = 1, COLLECT_GATHER = 2 };

int decode_status(const int* w, int what, int id, bool* clear_gemm, bool* clear_gather, std::string* msg)
{
    *clear_gemm = *clear_gather = false;
    const bool gemm_failed = w[ST_GEMM_ID] != 0 || w[ST_GEMM_COUNT] != 0;
    const bool gemm_mine = what == COLLECT_ALL || (what == COLLECT_GEMM && w[ST_GEMM_ID] == id);
    if (gemm_failed && gemm_mine) {
        static const char* sites[] = { "?", "producer waiting for a free stage", "MMA waiting for operands",
                                       "MMA waiting for a free accumulator", "epilogue waiting for the accumulator",
                                       "forwarding CTA waiting for a tile" };
        const int site = (w[ST_GEMM_SITE] >> 24) & 0xff;
        char buf[256];
        snprintf(buf, sizeof buf, "tcgen05 GEMM (launch %d): bounded wait ran out (%s, block %d, step %d; %d wait(s) in all); "
                 "results are invalid", w[ST_GEMM_ID], site >= 1 && site <= 5 ? sites[site] : sites[0],
                 w[ST_GEMM_SITE] & 0xffffff, w[ST_GEMM_STEP], w[ST_GEMM_COUNT]);
        *msg = buf;
        *clear_gemm = true;
        return ACCB_ERR_TIMEOUT;
    }
    const bool gather_mine = what == COLLECT_ALL || (what == COLLECT_GATHER && w[ST_GATHER_ID] == id);
    if (w[ST_GATHER_COUNT] != 0 && gather_mine) {
        char buf[200];
        snprintf(buf, sizeof buf, "gather: %d index value(s) outside the data dimension; those elements were zero-filled",
                 w[ST_GATHER_COUNT]);
        *msg = buf;
        *clear_gather = true;
        return ACCB_ERR_INDEX;
    }
    return ACCB_OK;
}

int collect_status(DeviceState& s, cudaStream_t stream, int what = COLLECT_ALL, int id = 0)
{
    cudaError_t e = cudaMemcpyAsync(s.status_host, s.status, kStatusWords * sizeof(int), cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return fail_cuda("kernel execution", e);
    int w[kStatusWords];
    memcpy(w, s.status_host, sizeof w);
    bool clear_gemm = false, clear_gather = false;
    std::string msg;
    const int rc = decode_status(w, what, id, &clear_gemm, &clear_gather, &msg);
    if (rc == ACCB_OK) return ACCB_OK;
    if (clear_gemm) e = cudaMemsetAsync(s.status + ST_GEMM_SITE, 0, 4 * sizeof(int), stream);      // words 1..4
    if (clear_gather && e == cudaSuccess) {
        e = cudaMemsetAsync(s.status + ST_GATHER_COUNT, 0, sizeof(int), stream);
        if (e == cudaSuccess) e = cudaMemsetAsync(s.status + ST_GATHER_ID, 0, sizeof(int), stream);
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return fail_cuda("cudaMemsetAsync(status)", e);
    return fail(rc, msg);
}

size_t type_bytes(int t)
{
    switch (t) {
    case ACCB_F32: case ACCB_S32: return 4;
    case ACCB_F16: case ACCB_BF16: case ACCB_S16: return 2;
    case ACCB_S8: case ACCB_U8: return 1;
    default: return 0;
    }
}

// Number of elements spanned by a 2-D array with the given strides (0 if empty).
int64_t span_elems(int64_t d0, int64_t d1, const int64_t* st)
{
    if (d0 <= 0 || d1 <= 0) return 0;
    return (d0 - 1) * st[0] + (d1 - 1) * st[1] + 1;
}

}  // namespace

int set_error(int code, const char* msg) { return fail(code, msg ? msg : ""); }
void clear_error() { t_error.clear(); }
int selected_device(int* dev) { return current_device(dev); }

namespace {

int tensor_gemm_split_k(const GemmLaunch& g, const char** err);

// An operand the tensor-core path cannot take only because its rows (or its base) are not 16-byte aligned - a
// K of 30522 bf16 elements, say - is copied into a temporary with an aligned pitch (one kernel, repack.cu,
// which also writes the zero padding of K; rows past the matrix edge need none, TMA zero-fills them) and the GEMM runs on that.  The temporary comes
// from the stream-ordered allocator (cudaMallocAsync on the launch stream, freed on it right after the launch), so
// nothing synchronises and concurrent streams do not share it.  Returns launches made, 0 when this does not apply
// (the caller then uses the CUDA-core kernel), or a negative ACCB_ERR_*.
int tensor_gemm_with_repacked_operands(const GemmLaunch& g0, const char** err)
{
    const accb_gemm_desc& d0 = g0.d;
    if (g0.batch > 1 || g0.n_extra_c > 0 || d0.k <= 0 || !gemm_umma_types_supported(d0)) return 0;
    if ((double)d0.m * (double)d0.n * (double)d0.k < (double)(1 << 24)) return 0;      // too small to pay for two more operations
    GemmLaunch g = g0;
    accb_gemm_desc& d = g.d;
    const size_t es = type_bytes(d.a_type);
    if (es == 0 || type_bytes(d.b_type) != es) return 0;
    // how each operand lies in memory: `rows` runs of `width` contiguous elements, `pitch` elements apart;
    // k_is_width: the contiguous direction is K
    struct Op { const void** base; int64_t* pitch; int64_t rows, width; bool k_is_width, aligned; };
    Op ops[2];
    auto describe = [&](Op& o, const void** base, int64_t* stride, int64_t dim0, int64_t dim1, bool k_is_dim1) {
        // the array is dim0 x dim1 with element strides stride[0], stride[1]; one of them must be 1
        if (stride[1] == 1) { o.rows = dim0; o.width = dim1; o.pitch = &stride[0]; o.k_is_width = k_is_dim1; }
        else if (stride[0] == 1) { o.rows = dim1; o.width = dim0; o.pitch = &stride[1]; o.k_is_width = !k_is_dim1; }
        else return false;
        o.base = base;
        o.aligned = ((*o.pitch * (int64_t)es) % 16 == 0) && ((reinterpret_cast<uintptr_t>(*base) & 15) == 0);
        return true;
    };
    if (!describe(ops[0], &g.a, d.a_stride, d.m, d.k, true) || !describe(ops[1], &g.b, d.b_stride, d.k, d.n, false)) return 0;
    if (ops[0].aligned && ops[1].aligned) return 0;             // alignment is not what keeps it off the tensor cores
    // A long K is padded with zeros to a multiple of 512 while the operands are copied anyway, so that it divides
    // into equal, aligned slices for the K-split below (30522 has no such divisor, 30720 has plenty).
    const int64_t k_new = (d.k >= 4096 && d.k % 512 != 0) ? (d.k + 511) / 512 * 512 : d.k;
    void* tmp[2] = { nullptr, nullptr };
    auto release = [&]() { for (void* t : tmp) if (t) cudaFreeAsync(t, g.stream); };
    for (int i = 0; i < 2; ++i) {
        Op& o = ops[i];
        if (o.aligned && k_new == d.k) continue;
        const int64_t new_rows = o.k_is_width ? o.rows : k_new;              // K-rows operands get zero rows appended
        const int64_t new_width = o.k_is_width ? k_new : o.width;            // K-contiguous ones get zero columns
        const int64_t old_rows = o.k_is_width ? o.rows : d.k;
        const int64_t old_width = o.k_is_width ? d.k : o.width;
        const size_t new_pitch = ((size_t)new_width * es + 15) & ~(size_t)15;
        cudaError_t e = cudaMallocAsync(&tmp[i], new_pitch * (size_t)new_rows, g.stream);
        if (e != cudaSuccess) { (void)cudaGetLastError(); tmp[i] = nullptr; release(); return 0; }   // no memory to spare: CUDA-core kernel
        // one kernel copies the rows and writes the zero columns / rows of the padding
        const int rc = launch_repack_rows(*o.base, *o.pitch * (int64_t)es, old_rows, old_width, (int)es, tmp[i], (int64_t)new_pitch,
                                          new_rows, g.stream, err);
        if (rc < 0) { release(); return rc; }
        *o.base = tmp[i];
        *o.pitch = (int64_t)(new_pitch / es);
    }
    d.k = k_new;
    const char* why = nullptr;
    int n = 0;
    if (gemm_umma_supported(g, &why)) {
        n = tensor_gemm_split_k(g, err);
        if (n == 0) n = launch_gemm_umma(g, d.m > 128 ? -1 : 0, err);
    }
    release();
    if (n > 0) note_launches(2);
    return n;
}

// A problem with few output tiles and a long K (1024 x 2048 x 30528: 32 tiles for 74 CTA pairs, 477 K steps each)
// is cut along K into `slices` equal parts that run as ONE batched launch - slice s is "problem" s, reading
// A[:, s*k/S ...] and B[s*k/S ..., :] in place through the batched kernel's rank-3 tensor maps and writing an fp32
// (int32) partial result - followed by one streaming pass that adds the partials in slice order and applies the
// epilogue (deterministic: no atomics, the same bits on every run).  The partials live in a stream-ordered temporary.
// Returns launches made, 0 when splitting does not apply, or a negative ACCB_ERR_*.
int tensor_gemm_split_k(const GemmLaunch& g, const char** err)
{
    const accb_gemm_desc& d = g.d;
    const int forced = options().gemm_split_k;
    if (g.batch > 1 || g.n_extra_c > 0 || g.no_split_k || forced == 0 || (forced < 0 && d.k < 2048)) return 0;
    const size_t es = type_bytes(d.a_type);
    const double slab = 128.0 / (double)es;                 // K elements per pipeline stage
    // Two tilings are candidates: the one the launch code would pick for the unsplit problem, and the widest tile
    // (256 columns; a CTA pair when M spans more than one tile row).  For each, the largest slice count that fills
    // the machine, divides K exactly (a slice must not run into the next row of a K-contiguous operand), keeps
    // every slice's start 16-byte aligned and leaves each slice at least 512 long.  Costs in microseconds from
    // measured launches of few-tile problems (64 x 320 x 2880, 512 x 512 x 8192, 1024 x 2048 x 4096): 0.33 us per stage
    // of a 256-column tile, 0.27 us of a 128-column one (a lone tile per SM is bound by the latency of its loads, not
    // by the tensor pipe); the split adds the reduction pass (about 3.5 us, launched so that it overlaps the tail of
    // the GEMM) and the partials' round trip through memory (bytes at 4 TB/s).
    int plan_two = 0, plan_cols = 0;
    int64_t plan_tiles = 0, plan_rounds = 0;
    gemm_umma_tile_plan(g, d.m > 128 ? -1 : 0, &plan_two, &plan_cols, &plan_tiles, &plan_rounds);
    struct Cand { int two_sm, cols; };
    const Cand cands[2] = { { plan_two, plan_cols }, { d.m > 128 ? 1 : 0, 256 } };
    const double unsplit_us = (double)plan_rounds * ((double)d.k / slab) * (plan_cols == 256 ? 0.33 : 0.27);
    double best_us = unsplit_us;
    int best_slices = 1;
    Cand best = cands[0];
    for (const Cand& c : cands) {
        const int64_t rows = c.two_sm ? 256 : 128;
        const int64_t tiles = ((d.m + rows - 1) / rows) * ((d.n + c.cols - 1) / c.cols);
        const int64_t units = c.two_sm ? g.num_sms / 2 : g.num_sms;
        for (int64_t sl = forced >= 2 ? forced : (units / tiles < 16 ? units / tiles : 16); sl >= 2; --sl) {
            if (d.k % sl != 0) { if (forced >= 2) break; continue; }
            const int64_t ks = d.k / sl;
            if ((ks < 512 && forced < 2) || (ks * (int64_t)es) % 16 != 0) { if (forced >= 2) break; continue; }
            const double rounds = (double)((tiles * sl + units - 1) / units);
            const double us = rounds * ((double)ks / slab) * (c.cols == 256 ? 0.33 : 0.27) + 3.5 +
                              (double)(sl + 1) * (double)d.m * (double)d.n * 4.0 / 4.0e6;
            if (us < best_us * 0.9 || (forced >= 2 && best_slices < 2)) { best_us = us; best_slices = (int)sl; best = c; }
            break;                                          // fewer slices of this tiling only cost more
        }
    }
    if (best_slices < 2) return 0;
    const int slices = best_slices;
    const int64_t ks = d.k / slices;
    const bool integer = d.c_type == ACCB_S32;
    void* ws = nullptr;
    cudaError_t e = cudaMallocAsync(&ws, (size_t)slices * (size_t)d.m * (size_t)d.n * 4, g.stream);
    if (e != cudaSuccess) { (void)cudaGetLastError(); return 0; }     // no memory to spare: unsplit launch
    GemmLaunch part = g;
    part.d.k = ks;
    part.d.c_type = integer ? ACCB_S32 : ACCB_F32;
    part.d.c_stride[0] = d.n; part.d.c_stride[1] = 1;
    part.d.alpha = 1.0f; part.d.beta = 0.0f;
    part.d.epilogue = ACCB_EPI_NONE;
    part.bias = nullptr;
    part.c = ws;
    part.batch = slices;
    part.a_batch_stride = ks * d.a_stride[1];
    part.b_batch_stride = ks * d.b_stride[0];
    part.c_batch_stride = d.m * d.n;
    part.force_tile_cols = best.cols;
    const char* why = nullptr;
    int n = 0;
    if (gemm_umma_supported(part, &why)) n = launch_gemm_umma(part, best.two_sm, err);
    if (n > 0) {
        const int r = launch_splitk_reduce(ws, slices, d, g.c, g.bias, g.stream, err);
        n = r < 0 ? r : n + r;
    }
    cudaFreeAsync(ws, g.stream);
    return n;
}

// Picks the kernel for one GEMM on device pointers.  Returns launches made or a negative ACCB_ERR_*.
int dispatch_gemm(const GemmLaunch& g, const char** err)
{
    const accb_gemm_desc& d = g.d;
    if (d.k == 0) return launch_gemm_simt(g, err);          // nothing to accumulate: epilogue of beta * C
    if (d.compute == ACCB_COMPUTE_SIMT) return launch_gemm_simt(g, err);
    if (d.compute == ACCB_COMPUTE_TENSOR) return launch_gemm_umma(g, 0, err);
    if (d.compute == ACCB_COMPUTE_TENSOR_2SM) return launch_gemm_umma(g, 1, err);
    // TENSOR_PREFERRED: the tensor cores whenever the element types have a tensor-core form - directly when the
    // layout allows it, through an aligned copy of an operand whose rows are not 16-byte aligned, and the CUDA-core
    // kernel for what is left (general strides, M / N-contiguous fp32).
    // AUTO: the same, except that fp32 inputs stay on the bit-faithful fp32 path.
    if (d.compute == ACCB_COMPUTE_TENSOR_PREFERRED || d.a_type != ACCB_F32) {
        const char* why = nullptr;
        if (gemm_umma_supported(g, &why)) {
            const int n = tensor_gemm_split_k(g, err);
            return n != 0 ? n : launch_gemm_umma(g, d.m > 128 ? -1 : 0, err);
        }
        const int n = tensor_gemm_with_repacked_operands(g, err);
        if (n != 0) return n;
    }
    return launch_gemm_simt(g, err);
}

// Large host-pointer GEMM: rows of A / C are staged in row chunks on two streams so that the host->device
// copy of chunk i+1, the GEMM of chunk i and the device->host copy of chunk i-1 overlap (PCIe is full
// duplex and the copies dwarf the GEMM).  Needs row-major A and C so that a row range is one byte range.
int pipelined_host_gemm(DeviceState& s, GemmLaunch g, const void* a, const void* b, void* c, const float* bias,
                        size_t ea, size_t ec, size_t bytes_b)
{
    const accb_gemm_desc d = g.d;
    cudaError_t e = cudaSuccess;
    for (int i = 0; i < 2 && e == cudaSuccess; ++i)
        if (!s.pipe[i]) e = cudaStreamCreateWithFlags(&s.pipe[i], cudaStreamNonBlocking);
    if (e == cudaSuccess && !s.pipe_ready) e = cudaEventCreateWithFlags(&s.pipe_ready, cudaEventDisableTiming);
    if (e != cudaSuccess) return fail_cuda("creating the staging pipeline", e);

    // 16 row chunks by default (the host_stage_chunks option overrides): the copy in of the first chunk and
    // the copy out of the last one are the part of the pipeline that nothing overlaps.  Measured on
    // 65536 x 8192 x 8192 bf16: 47.7 ms with 8 chunks, 46.0 with 12 or 16, 46.4 with 32.
    int64_t parts = 16;
    if (const int v = options().host_stage_chunks; v >= 1 && v <= 256) parts = v;
    int64_t chunk = (d.m + parts - 1) / parts;
    chunk = (chunk + 255) / 256 * 256;
    if (chunk < 1024) chunk = 1024;

    e = cudaMemcpyAsync(s.slot[1], b, bytes_b, cudaMemcpyHostToDevice, s.pipe[0]);
    if (e == cudaSuccess && bias) e = cudaMemcpyAsync(s.slot[3], bias, (size_t)d.n * 4, cudaMemcpyHostToDevice, s.pipe[0]);
    if (e == cudaSuccess) e = cudaEventRecord(s.pipe_ready, s.pipe[0]);
    if (e != cudaSuccess) return fail_cuda("host to device copy", e);
    g.b = s.slot[1];
    g.bias = bias ? (const float*)s.slot[3] : nullptr;

    int idx = 0;
    for (int64_t r0 = 0; r0 < d.m; r0 += chunk, ++idx) {
        const int64_t rows = (d.m - r0 < chunk) ? d.m - r0 : chunk;
        cudaStream_t st = s.pipe[idx & 1];
        const size_t off_a = (size_t)r0 * d.a_stride[0] * ea, len_a = ((size_t)(rows - 1) * d.a_stride[0] + d.k) * ea;
        const size_t off_c = (size_t)r0 * d.c_stride[0] * ec, len_c = ((size_t)(rows - 1) * d.c_stride[0] + d.n) * ec;
        if (idx & 1) e = cudaStreamWaitEvent(st, s.pipe_ready, 0);
        if (e == cudaSuccess) e = cudaMemcpyAsync((char*)s.slot[0] + off_a, (const char*)a + off_a, len_a, cudaMemcpyHostToDevice, st);
        if (e == cudaSuccess && (d.beta != 0.0f || d.c_stride[0] != d.n))     // padded rows: keep the caller's bytes in the gaps
            e = cudaMemcpyAsync((char*)s.slot[2] + off_c, (const char*)c + off_c, len_c, cudaMemcpyHostToDevice, st);
        if (e != cudaSuccess) return fail_cuda("host to device copy", e);
        GemmLaunch part = g;
        part.d.m = rows;
        part.a = (const char*)s.slot[0] + off_a;
        part.c = (char*)s.slot[2] + off_c;
        part.stream = st;
        part.no_split_k = true;          // the chunks are a way of moving the data: the result must not depend on them
        const char* err = "";
        const int n = dispatch_gemm(part, &err);
        if (n < 0) {
            cudaStreamSynchronize(s.pipe[0]);
            cudaStreamSynchronize(s.pipe[1]);
            return fail(n, std::string("accb_gemm: ") + err);
        }
        e = cudaMemcpyAsync((char*)c + off_c, (char*)s.slot[2] + off_c, len_c, cudaMemcpyDeviceToHost, st);
        if (e != cudaSuccess) return fail_cuda("device to host copy", e);
    }
    e = cudaStreamSynchronize(s.pipe[0]);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s.pipe[1]);
    if (e != cudaSuccess) return fail_cuda("kernel execution", e);
    return collect_status(s, s.pipe[0], COLLECT_GEMM, g.launch_id);
}

}  // namespace

}  // namespace accb

using namespace accb;

extern "C" {

// One entry for accb_gemm (batch = 1, `fn` names the caller in error texts) and accb_gemm_batched.
static int gemm_entry(const char* fn, const accb_gemm_desc* desc, int64_t batch, int64_t a_bs, int64_t b_bs, int64_t c_bs,
                      const void* a, const void* b, void* c, const float* bias)
{
    t_error.clear();
    const std::string who = std::string(fn) + ": ";
    if (!desc) return fail(ACCB_ERR_ARG, who + "null descriptor");
    const accb_gemm_desc& d = *desc;
    if (d.m < 0 || d.n < 0 || d.k < 0) return fail(ACCB_ERR_ARG, who + "negative dimension");
    const size_t ea = type_bytes(d.a_type), eb = type_bytes(d.b_type), ec = type_bytes(d.c_type);
    if (!ea || !eb || !ec) return fail(ACCB_ERR_ARG, who + "unknown element type");
    for (int i = 0; i < 2; ++i)
        if (d.a_stride[i] < 1 || d.b_stride[i] < 1 || d.c_stride[i] < 1)
            return fail(ACCB_ERR_ARG, who + "strides must be positive");
    if (d.epilogue != ACCB_EPI_NONE && d.epilogue != ACCB_EPI_RELU) return fail(ACCB_ERR_ARG, who + "unknown epilogue");
    if (d.compute < ACCB_COMPUTE_AUTO || d.compute > ACCB_COMPUTE_TENSOR_PREFERRED) return fail(ACCB_ERR_ARG, who + "unknown compute mode");
    if (d.max_ctas < 0) return fail(ACCB_ERR_ARG, who + "max_ctas must be >= 0");
    if (batch < 0 || a_bs < 0 || b_bs < 0 || c_bs < 0) return fail(ACCB_ERR_ARG, who + "negative batch count or batch stride");
    if (d.m == 0 || d.n == 0 || batch == 0) return ACCB_OK;
    if (batch > 1 && c_bs < span_elems(d.m, d.n, d.c_stride))
        return fail(ACCB_ERR_ARG, who + "c_batch_stride is smaller than one C: the problems' results would overlap");
    if (!a || !b || !c) return fail(ACCB_ERR_ARG, who + "null array pointer");

    DeviceState* sp = nullptr;
    int dev = 0;
    int rc = device_state(&sp, &dev);
    if (rc != ACCB_OK) return rc;
    DeviceState& s = *sp;

    const bool dev_a = is_device_pointer(a), dev_b = is_device_pointer(b), dev_c = is_device_pointer(c);
    const bool dev_bias = bias ? is_device_pointer(bias) : dev_c;
    const bool all_dev = dev_a && dev_b && dev_c && dev_bias;
    const bool all_host = !dev_a && !dev_b && !dev_c && (bias ? !dev_bias : true);
    if (!all_dev && !all_host) return fail(ACCB_ERR_ARG, who + "mix of host and device pointers");

    GemmLaunch g;
    g.d = d;
    g.n_extra_c = 0;
    g.batch = batch;
    g.a_batch_stride = batch > 1 ? a_bs : 0;
    g.b_batch_stride = batch > 1 ? b_bs : 0;
    g.c_batch_stride = batch > 1 ? c_bs : 0;
    g.stream = t_stream;
    g.status = s.status;
    g.launch_id = next_launch_id();
    g.device = dev;
    g.num_sms = s.num_sms;

    // bytes from the base pointer to the end of the last problem's array
    auto span_bytes = [&](int64_t d0, int64_t d1, const int64_t* st, int64_t bs, size_t es) -> size_t {
        const int64_t one = span_elems(d0, d1, st);
        return one ? (size_t)((batch - 1) * (batch > 1 ? bs : 0) + one) * es : 0;
    };
    const size_t bytes_a = span_bytes(d.m, d.k, d.a_stride, a_bs, ea);
    const size_t bytes_b = span_bytes(d.k, d.n, d.b_stride, b_bs, eb);
    const size_t bytes_c = span_bytes(d.m, d.n, d.c_stride, c_bs, ec);

    std::unique_lock<std::mutex> lock(s.mu, std::defer_lock);
    if (all_host) {
        lock.lock();   // the staging workspace is shared by all host-pointer calls on this device
        if ((rc = ensure(&s.slot[0], &s.slot_bytes[0], bytes_a)) != ACCB_OK) return rc;
        if ((rc = ensure(&s.slot[1], &s.slot_bytes[1], bytes_b)) != ACCB_OK) return rc;
        if ((rc = ensure(&s.slot[2], &s.slot_bytes[2], bytes_c)) != ACCB_OK) return rc;
        if (bias && (rc = ensure(&s.slot[3], &s.slot_bytes[3], (size_t)d.n * 4)) != ACCB_OK) return rc;
        const bool row_major_ac = d.a_stride[1] == 1 && d.c_stride[1] == 1 && d.a_stride[0] >= d.k && d.c_stride[0] >= d.n;
        if (batch == 1 && row_major_ac && d.m >= 4096 && d.k > 0 && bytes_a + bytes_c >= ((size_t)64 << 20))
            return pipelined_host_gemm(s, g, a, b, c, bias, ea, ec, bytes_b);
        cudaError_t e = cudaSuccess;
        if (bytes_a) e = cudaMemcpyAsync(s.slot[0], a, bytes_a, cudaMemcpyHostToDevice, g.stream);
        if (e == cudaSuccess && bytes_b) e = cudaMemcpyAsync(s.slot[1], b, bytes_b, cudaMemcpyHostToDevice, g.stream);
        // C goes to the device when it is read (beta != 0) and also when it has gaps (padded rows or problems):
        // the copy back covers the whole extent, so the gaps must carry the caller's bytes
        const bool c_dense = bytes_c == (size_t)batch * (size_t)d.m * (size_t)d.n * ec;
        if (e == cudaSuccess && (d.beta != 0.0f || !c_dense)) e = cudaMemcpyAsync(s.slot[2], c, bytes_c, cudaMemcpyHostToDevice, g.stream);
        if (e == cudaSuccess && bias) e = cudaMemcpyAsync(s.slot[3], bias, (size_t)d.n * 4, cudaMemcpyHostToDevice, g.stream);
        if (e != cudaSuccess) return fail_cuda("host to device copy", e);
        g.a = s.slot[0]; g.b = s.slot[1]; g.c = s.slot[2]; g.bias = bias ? (const float*)s.slot[3] : nullptr;
    } else {
        g.a = a; g.b = b; g.c = c; g.bias = bias;
    }

    const char* err = "";
    const int n = dispatch_gemm(g, &err);
    if (n < 0) return fail(n, who + err);

    if (all_host) {
        cudaError_t e = cudaMemcpyAsync(c, s.slot[2], bytes_c, cudaMemcpyDeviceToHost, g.stream);
        if (e != cudaSuccess) return fail_cuda("device to host copy", e);
        return collect_status(s, g.stream, COLLECT_GEMM, g.launch_id);
    }
    return ACCB_OK;
}

int accb_gemm(const accb_gemm_desc* desc, const void* a, const void* b, void* c, const float* bias)
{
    return gemm_entry("accb_gemm", desc, 1, 0, 0, 0, a, b, c, bias);
}

int accb_gemm_batched(const accb_gemm_desc* desc, int64_t batch, int64_t a_batch_stride, int64_t b_batch_stride,
                      int64_t c_batch_stride, const void* a, const void* b, void* c, const float* bias)
{
    return gemm_entry("accb_gemm_batched", desc, batch, a_batch_stride, b_batch_stride, c_batch_stride, a, b, c, bias);
}

int accb_gemm_tile_plan(const accb_gemm_desc* desc, int64_t batch, int32_t num_sms, int32_t* cta_pairs, int32_t* tile_cols,
                        int64_t* tiles, int64_t* rounds)
{
    t_error.clear();
    if (!desc || !cta_pairs || !tile_cols || !tiles || !rounds) return fail(ACCB_ERR_ARG, "accb_gemm_tile_plan: null pointer");
    if (desc->m < 1 || desc->n < 1 || desc->k < 1 || batch < 1 || num_sms < 2)
        return fail(ACCB_ERR_ARG, "accb_gemm_tile_plan: sizes must be positive (num_sms >= 2)");
    GemmLaunch g;
    g.d = *desc;
    g.a = g.b = nullptr; g.c = nullptr; g.bias = nullptr;
    g.n_extra_c = 0;
    g.batch = batch;
    g.stream = nullptr; g.status = nullptr; g.device = -1; g.launch_id = 0;
    g.num_sms = num_sms;
    const int want = desc->compute == ACCB_COMPUTE_TENSOR ? 0 : desc->compute == ACCB_COMPUTE_TENSOR_2SM ? 1 : (desc->m > 128 ? -1 : 0);
    int pairs = 0, cols = 0;
    gemm_umma_tile_plan(g, want, &pairs, &cols, tiles, rounds);
    *cta_pairs = pairs;
    *tile_cols = cols;
    return ACCB_OK;
}

int accb_gemm_launch_geometry(const accb_gemm_desc* desc, int64_t batch, int32_t num_sms, int32_t* grid, int32_t* block,
                              int32_t* dynamic_shared_mem_bytes)
{
    t_error.clear();
    if (!desc || !grid || !block || !dynamic_shared_mem_bytes) return fail(ACCB_ERR_ARG, "accb_gemm_launch_geometry: null pointer");
    if (desc->m < 1 || desc->n < 1 || desc->k < 1 || batch < 1 || num_sms < 2)
        return fail(ACCB_ERR_ARG, "accb_gemm_launch_geometry: sizes must be positive (num_sms >= 2)");
    GemmLaunch g;
    g.d = *desc;
    g.a = g.b = nullptr; g.c = nullptr; g.bias = nullptr;
    g.n_extra_c = 0;
    g.batch = batch;
    g.stream = nullptr; g.status = nullptr; g.device = -1; g.launch_id = 0;
    g.num_sms = num_sms;
    const int want = desc->compute == ACCB_COMPUTE_TENSOR ? 0 : desc->compute == ACCB_COMPUTE_TENSOR_2SM ? 1 : (desc->m > 128 ? -1 : 0);
    int32_t out[8];
    gemm_umma_launch_geometry(g, want, out);
    for (int i = 0; i < 3; ++i) { grid[i] = out[i]; block[i] = out[3 + i]; }
    *dynamic_shared_mem_bytes = out[6];
    return ACCB_OK;
}

int accb_set_option(const char* name, int64_t value)
{
    t_error.clear();
    if (!name) return fail(ACCB_ERR_ARG, "accb_set_option: null name");
    Options& o = options();
    const std::string n(name);
    const int v = (int)value;
    if (n == "reset") { o = Options(); return ACCB_OK; }
    if (n == "gemm.tile_cols") { if (v != 0 && v != 128 && v != 256) return fail(ACCB_ERR_ARG, "accb_set_option: gemm.tile_cols is 0, 128 or 256"); o.gemm_tile_cols = v; }
    else if (n == "gemm.staged_store") o.gemm_staged_store = v < 0 ? -1 : (v > 2 ? 1 : (int)v);
    else if (n == "gemm.pace_pct") { if (v > 100) return fail(ACCB_ERR_ARG, "accb_set_option: gemm.pace_pct is -1 or 0..100"); o.gemm_pace_pct = v < 0 ? -1 : v; }
    else if (n == "gemm.group_m") { if (v < 0 || v > 4096) return fail(ACCB_ERR_ARG, "accb_set_option: gemm.group_m is 0..4096"); o.gemm_group_m = v; }
    else if (n == "gemm.hint_a") o.gemm_hint_a = (v >= 0 && v <= 2) ? v : 0;
    else if (n == "gemm.hint_b") o.gemm_hint_b = (v >= 0 && v <= 2) ? v : 0;
    else if (n == "gemm.c_stream") o.gemm_c_stream = v ? 1 : 0;
    else if (n == "gemm.peer_store") o.gemm_peer_store = v < 0 ? -1 : (v ? 1 : 0);
    else if (n == "gemm.copy_ctas") { if (v > 128) return fail(ACCB_ERR_ARG, "accb_set_option: gemm.copy_ctas is -1 (choose) or 0..128"); o.gemm_copy_ctas = v < 0 ? -1 : v; }
    else if (n == "gemm.wait_limit_us") { if (value < 0 || value > 10000000) return fail(ACCB_ERR_ARG, "accb_set_option: gemm.wait_limit_us is 0 (default) .. 10000000"); o.gemm_wait_limit_us = v; }
    else if (n == "gemm.test_drop_commit") o.gemm_test_drop_commit = v ? 1 : 0;
    else if (n == "gemm.pdl") o.gemm_pdl = v < 0 ? -1 : (v ? 1 : 0);
    else if (n == "gemm.epi_warps") o.gemm_epi_warps = (v == 4) ? 4 : (v == 8 ? 8 : 0);
    else if (n == "gemm.split_k") o.gemm_split_k = v < 0 ? -1 : (int)v;
    else if (n == "stream_kernels.pdl") o.stream_pdl = v < 0 ? -1 : (v ? 1 : 0);
    else if (n == "gemm.c_in") o.gemm_c_in = v < 0 ? -1 : (v ? 1 : 0);
    else if (n == "gemm.verbose") o.gemm_verbose = v ? 1 : 0;
    else if (n == "host_gemm.stage_chunks") { if (v < 0 || v > 256) return fail(ACCB_ERR_ARG, "accb_set_option: host_gemm.stage_chunks is 0 (default) .. 256"); o.host_stage_chunks = v; }
    else if (n == "reduce.rows_threads_per_output") { if (v != 0 && v != 32 && v != 64 && v != 128 && v != 256) return fail(ACCB_ERR_ARG, "accb_set_option: reduce.rows_threads_per_output is 0, 32, 64, 128 or 256"); o.reduce_rows_tpr = v; }
    else return fail(ACCB_ERR_ARG, "accb_set_option: unknown option " + n);
    return ACCB_OK;
}

int accb_gemm_replicated(const accb_gemm_desc* desc, const void* a, const void* b, void* const* c_replicas,
                         int32_t n_replicas, const float* bias)
{
    t_error.clear();
    if (!desc) return fail(ACCB_ERR_ARG, "accb_gemm_replicated: null descriptor");
    if (!c_replicas || n_replicas < 1 || n_replicas > 8) return fail(ACCB_ERR_ARG, "accb_gemm_replicated: 1 to 8 replicas");
    const accb_gemm_desc& d = *desc;
    if (d.m <= 0 || d.n <= 0 || d.k <= 0) return fail(ACCB_ERR_ARG, "accb_gemm_replicated: dimensions must be positive");
    if (!type_bytes(d.a_type) || !type_bytes(d.b_type) || !type_bytes(d.c_type)) return fail(ACCB_ERR_ARG, "accb_gemm_replicated: unknown element type");
    for (int i = 0; i < 2; ++i)
        if (d.a_stride[i] < 1 || d.b_stride[i] < 1 || d.c_stride[i] < 1)
            return fail(ACCB_ERR_ARG, "accb_gemm_replicated: strides must be positive");
    if (d.epilogue != ACCB_EPI_NONE && d.epilogue != ACCB_EPI_RELU) return fail(ACCB_ERR_ARG, "accb_gemm_replicated: unknown epilogue");
    if (d.max_ctas < 0) return fail(ACCB_ERR_ARG, "accb_gemm_replicated: max_ctas must be >= 0");
    if (!a || !b || !c_replicas[0]) return fail(ACCB_ERR_ARG, "accb_gemm_replicated: null array pointer");
    DeviceState* sp = nullptr;
    int dev = 0;
    int rc = device_state(&sp, &dev);
    if (rc != ACCB_OK) return rc;
    if (!is_device_pointer(a) || !is_device_pointer(b) || !is_device_pointer(c_replicas[0]) || (bias && !is_device_pointer(bias)))
        return fail(ACCB_ERR_ARG, "accb_gemm_replicated: device pointers only");
    GemmLaunch g;
    g.d = d;
    g.a = a; g.b = b; g.c = c_replicas[0]; g.bias = bias;
    g.n_extra_c = n_replicas - 1;
    for (int r = 1; r < n_replicas; ++r) g.extra_c[r - 1] = c_replicas[r];
    g.stream = t_stream;
    g.status = sp->status;
    g.launch_id = next_launch_id();
    g.device = dev;
    g.num_sms = sp->num_sms;
    if (n_replicas > 1) {
        // a region of the counter ring, large enough for any tiling of this problem (128 x 128 tiles at the least)
        const int64_t need = ((d.m + 127) / 128) * ((d.n + 127) / 128);
        std::lock_guard<std::mutex> lock(sp->mu);
        if (!sp->tile_flags) {
            cudaError_t e = cudaMalloc(&sp->tile_flags, kTileFlagInts * sizeof(int));
            if (e != cudaSuccess) return fail_cuda("cudaMalloc(tile counters)", e);
        }
        if (need <= kTileFlagInts) {
            if (sp->tile_flags_cursor + need > kTileFlagInts) sp->tile_flags_cursor = 0;
            g.tile_flags = sp->tile_flags + sp->tile_flags_cursor;
            g.tile_flags_capacity = need;
            sp->tile_flags_cursor += need;
        }
    }
    const char* err = "";
    const int n = launch_gemm_umma(g, d.compute != ACCB_COMPUTE_TENSOR ? 1 : 0, &err);
    if (n < 0) return fail(n, std::string("accb_gemm_replicated: ") + err);
    return ACCB_OK;
}

int accb_reduce_mean_rank3_dims(int64_t d0, int64_t d1, int64_t d2, int32_t axes_mask, int32_t keepdims, int64_t* out_dims)
{
    if (!out_dims) return fail(ACCB_ERR_ARG, "accb_reduce_mean_rank3_dims: null out_dims");
    axes_mask &= 7;
    if (axes_mask == 0) axes_mask = 7;
    const int64_t dims[3] = { d0, d1, d2 };
    int n = 0;
    for (int d = 0; d < 3; ++d) {
        if (axes_mask & (1 << d)) { if (keepdims) out_dims[n++] = 1; }
        else out_dims[n++] = dims[d];
    }
    if (n == 0) out_dims[n++] = 1;
    return n;
}

int accb_reduce_mean_rank3(const float* data, int64_t d0, int64_t d1, int64_t d2, float* reduced, int32_t axes_mask)
{
    t_error.clear();
    if (d0 < 0 || d1 < 0 || d2 < 0) return fail(ACCB_ERR_ARG, "accb_reduce_mean_rank3: negative dimension");
    if (axes_mask < 0 || axes_mask > 7) return fail(ACCB_ERR_ARG, "accb_reduce_mean_rank3: axes_mask must be in [0, 7]");
    if (axes_mask == 0) axes_mask = 7;
    const int64_t dims[3] = { d0, d1, d2 };
    int64_t n_out = 1, n_in = d0 * d1 * d2;
    for (int d = 0; d < 3; ++d) if (!(axes_mask & (1 << d))) n_out *= dims[d];
    if (n_out == 0) return ACCB_OK;
    if (n_in == 0) return fail(ACCB_ERR_ARG, "accb_reduce_mean_rank3: mean over zero elements");
    if (!data || !reduced) return fail(ACCB_ERR_ARG, "accb_reduce_mean_rank3: null array pointer");

    DeviceState* sp = nullptr;
    int rc = device_state(&sp, nullptr);
    if (rc != ACCB_OK) return rc;
    DeviceState& s = *sp;
    const bool dev_in = is_device_pointer(data), dev_out = is_device_pointer(reduced);
    if (dev_in != dev_out) return fail(ACCB_ERR_ARG, "accb_reduce_mean_rank3: mix of host and device pointers");
    cudaStream_t stream = t_stream;

    std::lock_guard<std::mutex> lock(s.mu);   // staging and scratch buffers are shared per device
    const float* din = data;
    float* dout = reduced;
    if (!dev_in) {
        if ((rc = ensure(&s.slot[0], &s.slot_bytes[0], (size_t)n_in * 4)) != ACCB_OK) return rc;
        if ((rc = ensure(&s.slot[2], &s.slot_bytes[2], (size_t)n_out * 4)) != ACCB_OK) return rc;
        cudaError_t e = cudaMemcpyAsync(s.slot[0], data, (size_t)n_in * 4, cudaMemcpyHostToDevice, stream);
        if (e != cudaSuccess) return fail_cuda("host to device copy", e);
        din = (const float*)s.slot[0];
        dout = (float*)s.slot[2];
    }
    const size_t need = reduce_mean_scratch_bytes(d0, d1, d2, axes_mask, s.num_sms);
    if (need && (rc = ensure(&s.scratch, &s.scratch_bytes, need)) != ACCB_OK) return rc;
    if (need) {
        // order this launch after the previous user of the shared scratch buffer if that ran on another stream
        cudaError_t e = cudaSuccess;
        if (!s.scratch_done) e = cudaEventCreateWithFlags(&s.scratch_done, cudaEventDisableTiming);
        if (e == cudaSuccess && s.scratch_used && s.scratch_stream != stream) e = cudaStreamWaitEvent(stream, s.scratch_done, 0);
        if (e != cudaSuccess) return fail_cuda("ordering the scratch buffer between streams", e);
    }
    const char* err = "";
    int n = launch_reduce_mean(din, d0, d1, d2, dout, axes_mask, (float*)s.scratch, s.scratch_bytes, s.num_sms, stream, &err);
    if (n < 0) return fail(n, std::string("accb_reduce_mean_rank3: ") + err);
    if (need) {
        cudaError_t e = cudaEventRecord(s.scratch_done, stream);
        if (e != cudaSuccess) return fail_cuda("cudaEventRecord", e);
        s.scratch_stream = stream;
        s.scratch_used = true;
    }
    if (!dev_in) {
        cudaError_t e = cudaMemcpyAsync(reduced, dout, (size_t)n_out * 4, cudaMemcpyDeviceToHost, stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
        if (e != cudaSuccess) return fail_cuda("device to host copy", e);
    }
    return ACCB_OK;
}

int accb_gather_rank2_dims(int64_t d0, int64_t d1, int64_t i0, int64_t i1, int32_t axis, int64_t* out_dims)
{
    if (!out_dims) return fail(ACCB_ERR_ARG, "accb_gather_rank2_dims: null out_dims");
    if (axis == 0) { out_dims[0] = i0; out_dims[1] = i1; out_dims[2] = d1; }
    else if (axis == 1) { out_dims[0] = d0; out_dims[1] = i0; out_dims[2] = i1; }
    else return fail(ACCB_ERR_ARG, "accb_gather_rank2_dims: axis must be 0 or 1");
    return ACCB_OK;
}

int accb_gather_rank2(const void* data, int64_t d0, int64_t d1, const int64_t* indices, int64_t i0, int64_t i1,
                      void* output, int32_t axis, int32_t elem_bytes)
{
    t_error.clear();
    if (d0 < 0 || d1 < 0 || i0 < 0 || i1 < 0) return fail(ACCB_ERR_ARG, "accb_gather_rank2: negative dimension");
    if (axis != 0 && axis != 1) return fail(ACCB_ERR_ARG, "accb_gather_rank2: axis must be 0 or 1");
    if (elem_bytes != 1 && elem_bytes != 2 && elem_bytes != 4 && elem_bytes != 8)
        return fail(ACCB_ERR_ARG, "accb_gather_rank2: elem_bytes must be 1, 2, 4 or 8");
    const int64_t n_idx = i0 * i1;
    const int64_t n_out = (axis == 0) ? n_idx * d1 : d0 * n_idx;
    if (n_out == 0) return ACCB_OK;
    if (!data || !indices || !output) return fail(ACCB_ERR_ARG, "accb_gather_rank2: null array pointer");

    DeviceState* sp = nullptr;
    int rc = device_state(&sp, nullptr);
    if (rc != ACCB_OK) return rc;
    DeviceState& s = *sp;
    const bool dd = is_device_pointer(data), di = is_device_pointer(indices), dout = is_device_pointer(output);
    if (dd != di || dd != dout) return fail(ACCB_ERR_ARG, "accb_gather_rank2: mix of host and device pointers");
    cudaStream_t stream = t_stream;
    const char* err = "";
    const int launch_id = next_launch_id();
    if (dd) {
        int n = launch_gather(data, d0, d1, indices, i0, i1, output, axis, elem_bytes, s.status, launch_id, stream, &err);
        if (n < 0) return fail(n, std::string("accb_gather_rank2: ") + err);
        return ACCB_OK;
    }
    std::lock_guard<std::mutex> lock(s.mu);
    const size_t bytes_data = (size_t)(d0 * d1) * elem_bytes, bytes_idx = (size_t)n_idx * 8, bytes_out = (size_t)n_out * elem_bytes;
    if ((rc = ensure(&s.slot[0], &s.slot_bytes[0], bytes_data)) != ACCB_OK) return rc;
    if ((rc = ensure(&s.slot[1], &s.slot_bytes[1], bytes_idx)) != ACCB_OK) return rc;
    if ((rc = ensure(&s.slot[2], &s.slot_bytes[2], bytes_out)) != ACCB_OK) return rc;
    cudaError_t e = cudaMemcpyAsync(s.slot[0], data, bytes_data, cudaMemcpyHostToDevice, stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(s.slot[1], indices, bytes_idx, cudaMemcpyHostToDevice, stream);
    if (e != cudaSuccess) return fail_cuda("host to device copy", e);
    int n = launch_gather(s.slot[0], d0, d1, (const int64_t*)s.slot[1], i0, i1, s.slot[2], axis, elem_bytes, s.status, launch_id, stream, &err);
    if (n < 0) return fail(n, std::string("accb_gather_rank2: ") + err);
    e = cudaMemcpyAsync(output, s.slot[2], bytes_out, cudaMemcpyDeviceToHost, stream);
    if (e != cudaSuccess) return fail_cuda("device to host copy", e);
    return collect_status(s, stream, COLLECT_GATHER, launch_id);
}

int64_t accb_range_count_f32(float start, float limit, float delta)
{
    return range_count_f32(start, limit, delta);
}

int64_t accb_range_plan_f32(float start, float delta, int64_t n, int64_t* first, uint32_t* bits, int32_t* step,
                            int64_t capacity, float* final_value)
{
    if (n < 0 || capacity < 0) return 0;
    return range_plan_f32(start, delta, n, first, bits, step, capacity, final_value);
}

int accb_range_f32(int64_t n, float* output, float* start_inout, float delta)
{
    t_error.clear();
    if (n < 0) return fail(ACCB_ERR_ARG, "accb_range_f32: negative length");
    if (!start_inout) return fail(ACCB_ERR_ARG, "accb_range_f32: null start pointer");
    if (n == 0) return ACCB_OK;
    if (!output) return fail(ACCB_ERR_ARG, "accb_range_f32: null output pointer");
    DeviceState* sp = nullptr;
    int rc = device_state(&sp, nullptr);
    if (rc != ACCB_OK) return rc;
    DeviceState& s = *sp;
    if (is_device_pointer(start_inout)) return fail(ACCB_ERR_ARG, "accb_range_f32: start_inout must be a host pointer");
    const bool dev_out = is_device_pointer(output);
    cudaStream_t stream = t_stream;
    std::unique_lock<std::mutex> lock(s.mu, std::defer_lock);
    float* dout = output;
    if (!dev_out) {
        lock.lock();
        if ((rc = ensure(&s.slot[2], &s.slot_bytes[2], (size_t)n * 4)) != ACCB_OK) return rc;
        dout = (float*)s.slot[2];
    }
    const char* err = "";
    float last = *start_inout;
    const int launched = launch_range_f32(n, dout, *start_inout, delta, &last, stream, &err);
    if (launched < 0) return fail(launched, std::string("accb_range_f32: ") + err);
    *start_inout = last;
    if (!dev_out) {
        cudaError_t e = cudaMemcpyAsync(output, dout, (size_t)n * 4, cudaMemcpyDeviceToHost, stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
        if (e != cudaSuccess) return fail_cuda("device to host copy", e);
    }
    return ACCB_OK;
}

int accb_set_device(int32_t device)
{
    t_error.clear();
    if (device == -1) { t_device = -1; return ACCB_OK; }     // back to "whatever CUDA device is current"
    if (device < 0 || device >= kMaxDevices) return fail(ACCB_ERR_ARG, "accb_set_device: device index out of range");
    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) return fail_cuda("cudaSetDevice", e);
    t_device = device;
    return ACCB_OK;
}

int accb_get_device(void) { return t_device; }

int accb_current_device(void)
{
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) { (void)cudaGetLastError(); return ACCB_ERR_CUDA; }
    return dev;
}

int accb_debug_decode_status(const int32_t* words, int32_t what, int32_t launch_id, char* message, int32_t capacity)
{
    if (!words) return ACCB_ERR_ARG;
    int w[kStatusWords];
    for (int i = 0; i < kStatusWords; ++i) w[i] = words[i];
    bool cg = false, ca = false;
    std::string msg;
    const int rc = decode_status(w, what, launch_id, &cg, &ca, &msg);
    if (message && capacity > 0) { strncpy(message, msg.c_str(), (size_t)capacity - 1); message[capacity - 1] = 0; }
    return rc;
}

int accb_set_stream(void* cuda_stream)
{
    t_stream = (cudaStream_t)cuda_stream;
    return ACCB_OK;
}

int accb_synchronize(void)
{
    t_error.clear();
    DeviceState* sp = nullptr;
    int rc = device_state(&sp, nullptr);
    if (rc != ACCB_OK) return rc;
    std::lock_guard<std::mutex> lock(sp->mu);
    return collect_status(*sp, t_stream);
}

const char* accb_last_error(void) { return t_error.c_str(); }

int64_t accb_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int accb_release_workspace(void)
{
    t_error.clear();
    int dev = 0;
    int rc = current_device(&dev);
    if (rc != ACCB_OK) return rc;
    DeviceState& s = g_dev[dev];
    std::lock_guard<std::mutex> lock(s.mu);
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return fail_cuda("cudaDeviceSynchronize", e);
    for (int i = 0; i < 4; ++i) {
        if (s.slot[i]) cudaFree(s.slot[i]);
        s.slot[i] = nullptr;
        s.slot_bytes[i] = 0;
    }
    if (s.scratch) cudaFree(s.scratch);
    s.scratch = nullptr;
    s.scratch_bytes = 0;
    return ACCB_OK;
}

int accb_device_count(void)
{
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) { (void)cudaGetLastError(); return 0; }
    return n;
}

const char* accb_version(void) { return "accera_b200 0.1 (sm_100a)"; }

}  // extern "C"
