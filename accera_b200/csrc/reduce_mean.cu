// ReduceMean over a dense first-major rank-3 fp32 array, for sm_100a.
//
// The reference defines the op as three fused nests (zero-init, accumulate in
// index order, divide by the count; kernels/reduce_mean/naive_runtime_sized.py:
// 66-148) and has no GPU kernel for it.  Here every reduction is HBM-bound
// streaming: 128-bit loads, several of them in flight per thread before the
// first add, fp32 partial sums per thread, a warp-shuffle tree and one shared-
// memory hop per block.  Sums are therefore pairwise rather than sequential,
// which is at least as accurate as the reference order.
//
// Two data-access shapes cover all 7 axis subsets of a rank-3 array:
//   "rows":  every output owns `nseg` contiguous segments of `len` elements
//            (axes {2}, {1,2}, {0,1,2}, {0,2})
//   "cols":  the innermost kept dimension is contiguous and the reduced
//            dimension strides over it: out[o,i] = mean_r x[o,r,i]
//            (axes {1}, {0}, {0,1})
// When there are too few outputs to fill the GPU, each output's reduction is
// split over several blocks that write fp32 partial sums to a scratch buffer and
// a second small kernel folds them in a fixed order (deterministic, no atomics).
#include <mutex>
#include <string>

#include "accb_internal.h"

// Scratch for accb_reduce_mean_rank3_noalloc: lives in the library image, so every GPU that loads the
// library carries these 256 KiB until the process exits.  In host code this name is only a handle for
// cudaGetSymbolAddress; kernels are always given the device address obtained from it.
constexpr size_t kStaticScratchFloats = 64 * 1024;
static __device__ __align__(256) float g_static_scratch[kStaticScratchFloats];

namespace accb {
namespace {

constexpr int kBlock = 256;

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Sum over all threads of the block; valid in thread 0.
__device__ __forceinline__ float block_sum(float v, float* smem)
{
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    float r = 0.0f;
    if (warp == 0) {
        r = (lane < (int)(blockDim.x >> 5)) ? smem[lane] : 0.0f;
        r = warp_sum(r);
    }
    return r;
}

// Streams [begin, end) of one contiguous segment, 4 independent 128-bit loads in
// flight per thread.  `vec_ok` = segment start and length are 16-byte aligned.
template <int TPR>
__device__ __forceinline__ float segment_sum(const float* __restrict__ seg, int64_t begin, int64_t end, int t, bool vec_ok)
{
    float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
    if (vec_ok) {
        const float4* v = reinterpret_cast<const float4*>(seg);
        const int64_t vb = begin >> 2, ve = end >> 2;
        int64_t i = vb + t;
        for (; i + 3 * TPR < ve; i += 4 * TPR) {
            float4 a = __ldcs(v + i);
            float4 b = __ldcs(v + i + TPR);
            float4 c = __ldcs(v + i + 2 * TPR);
            float4 d = __ldcs(v + i + 3 * TPR);
            s0 += (a.x + a.y) + (a.z + a.w);
            s1 += (b.x + b.y) + (b.z + b.w);
            s2 += (c.x + c.y) + (c.z + c.w);
            s3 += (d.x + d.y) + (d.z + d.w);
        }
        for (; i < ve; i += TPR) {
            float4 a = __ldcs(v + i);
            s0 += (a.x + a.y) + (a.z + a.w);
        }
    } else {
        for (int64_t i = begin + t; i < end; i += TPR) s0 += __ldcs(seg + i);
    }
    return (s0 + s1) + (s2 + s3);
}

struct RowsParams {
    int64_t n_out;        // number of outputs
    int64_t row_stride;   // elements between the first segments of consecutive outputs
    int64_t nseg;         // segments per output
    int64_t seg_stride;   // elements between consecutive segments of one output
    int64_t len;          // contiguous elements per segment
    int64_t nsplit;       // blocks per output (1 = single pass)
    float count;          // number of reduced elements, as the reference divides by it in fp32
    int vec_ok;
};

// TPR threads cooperate on one output; kBlock / TPR outputs per block.
// nsplit > 1: blockIdx.y selects a slice of the (segment, chunk) space and the
// block writes a raw partial sum to `out[o * nsplit + split]` (the scratch buffer).
template <int TPR>
__global__ void __launch_bounds__(kBlock)
reduce_rows_kernel(const float* __restrict__ data, float* __restrict__ out, RowsParams p)
{
    __shared__ float smem[kBlock / 32];
    constexpr int RPB = kBlock / TPR;
    const int t = threadIdx.x % TPR;
    const int64_t o = (int64_t)blockIdx.x * RPB + threadIdx.x / TPR;
    const bool live = o < p.n_out;
    float s = 0.0f;
    if (live) {
        const float* row = data + o * p.row_stride;
        if (p.nsplit == 1) {
            for (int64_t g = 0; g < p.nseg; ++g)
                s += segment_sum<TPR>(row + g * p.seg_stride, 0, p.len, t, p.vec_ok);
        } else {
            // split the len axis of every segment into nsplit aligned slices
            int64_t chunk = (p.len + p.nsplit - 1) / p.nsplit;
            chunk = (chunk + 3) & ~int64_t(3);
            const int64_t b = (int64_t)blockIdx.y * chunk;
            const int64_t e = (b + chunk < p.len) ? b + chunk : p.len;
            if (b < e)
                for (int64_t g = 0; g < p.nseg; ++g)
                    s += segment_sum<TPR>(row + g * p.seg_stride, b, e, t, p.vec_ok);
        }
    }
    if (TPR == 32) {
        s = warp_sum(s);
        if (live && t == 0) {
            if (p.nsplit == 1) out[o] = s / p.count;
            else out[o * p.nsplit + blockIdx.y] = s;
        }
    } else {
        s = block_sum(s, smem);
        if (live && threadIdx.x == 0) {
            if (p.nsplit == 1) out[o] = s / p.count;
            else out[o * p.nsplit + blockIdx.y] = s;
        }
    }
}

struct ColsParams {
    int64_t outer, r, inner;
    int64_t col_blocks;   // blocks along the inner dimension; gridDim.x = col_blocks * outer
    int64_t nsplit;       // slices of r (gridDim.y)
    float count;          // number of reduced elements, as the reference divides by it in fp32
    int vec_ok;
};

// out[o, i] = mean_r x[o, r, i].  blockDim = (32, 8): 32 column groups (of 4 when
// vectorised) by 8 interleaved slices of r, folded through shared memory.
__global__ void __launch_bounds__(kBlock)
reduce_cols_kernel(const float* __restrict__ data, float* __restrict__ out, ColsParams p)
{
    __shared__ float4 smem[8][32];
    const int tx = threadIdx.x, ty = threadIdx.y;
    const int64_t o = blockIdx.x / p.col_blocks;
    const int vec = p.vec_ok ? 4 : 1;
    const int64_t col = ((int64_t)(blockIdx.x % p.col_blocks) * 32 + tx) * vec;
    int64_t r_chunk = (p.r + p.nsplit - 1) / p.nsplit;
    const int64_t rb = (int64_t)blockIdx.y * r_chunk;
    const int64_t re = (rb + r_chunk < p.r) ? rb + r_chunk : p.r;
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    if (col < p.inner) {
        const float* base = data + o * p.r * p.inner + col;
        if (p.vec_ok) {
            int64_t r = rb + ty;
            for (; r + 24 < re; r += 32) {
                float4 a = __ldcs(reinterpret_cast<const float4*>(base + r * p.inner));
                float4 b = __ldcs(reinterpret_cast<const float4*>(base + (r + 8) * p.inner));
                float4 c = __ldcs(reinterpret_cast<const float4*>(base + (r + 16) * p.inner));
                float4 d = __ldcs(reinterpret_cast<const float4*>(base + (r + 24) * p.inner));
                s.x += (a.x + b.x) + (c.x + d.x);
                s.y += (a.y + b.y) + (c.y + d.y);
                s.z += (a.z + b.z) + (c.z + d.z);
                s.w += (a.w + b.w) + (c.w + d.w);
            }
            for (; r < re; r += 8) {
                float4 a = __ldcs(reinterpret_cast<const float4*>(base + r * p.inner));
                s.x += a.x; s.y += a.y; s.z += a.z; s.w += a.w;
            }
        } else {
            for (int64_t r = rb + ty; r < re; r += 8) s.x += __ldcs(base + r * p.inner);
        }
    }
    smem[ty][tx] = s;
    __syncthreads();
    if (ty == 0 && col < p.inner) {
#pragma unroll
        for (int y = 1; y < 8; ++y) {
            float4 q = smem[y][tx];
            s.x += q.x; s.y += q.y; s.z += q.z; s.w += q.w;
        }
        if (p.nsplit == 1) {
            float* dst = out + o * p.inner + col;
            if (p.vec_ok) {
                *reinterpret_cast<float4*>(dst) =
                    make_float4(s.x / p.count, s.y / p.count, s.z / p.count, s.w / p.count);
            } else {
                dst[0] = s.x / p.count;
            }
        } else {
            // partials laid out [split][outer * inner] so that the fold below is coalesced
            float* dst = out + ((int64_t)blockIdx.y * p.outer + o) * p.inner + col;
            if (p.vec_ok) *reinterpret_cast<float4*>(dst) = s;
            else dst[0] = s.x;
        }
    }
}

// Second pass of a split reduction: out[i] = (sum_s partial[...]) / count in a fixed order.
// rows layout:  partial[i * nsplit + s];  cols layout: partial[s * n + i].
__global__ void __launch_bounds__(kBlock)
reduce_fold_kernel(const float* __restrict__ partial, float* __restrict__ out, int64_t n, int64_t nsplit,
                   int cols_layout, float count)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float s = 0.0f;
    if (cols_layout) {
        for (int64_t k = 0; k < nsplit; ++k) s += partial[k * n + i];
    } else {
        for (int64_t k = 0; k < nsplit; ++k) s += partial[i * nsplit + k];
    }
    out[i] = s / count;
}

struct Plan {
    bool rows;            // rows or cols shape
    RowsParams rp;
    ColsParams cp;
    int tpr;              // threads per output for the rows kernel (32 or 256)
    int64_t nsplit;
    int64_t n_out;
};

Plan make_plan(int64_t d0, int64_t d1, int64_t d2, int mask, int num_sms)
{
    Plan pl{};
    mask &= 7;
    if (mask == 0) mask = 7;  // ONNX: no axes = reduce everything
    const int64_t total = d0 * d1 * d2;
    const int64_t target_blocks = 2 * (int64_t)num_sms;
    pl.nsplit = 1;
    if (mask & 4) {
        pl.rows = true;
        RowsParams& r = pl.rp;
        r.nseg = 1; r.seg_stride = 0;
        if (mask == 4) { r.n_out = d0 * d1; r.row_stride = d2; r.len = d2; }
        else if (mask == 6) { r.n_out = d0; r.row_stride = d1 * d2; r.len = d1 * d2; }
        else if (mask == 7) { r.n_out = 1; r.row_stride = 0; r.len = total; }
        else /* mask == 5 */ { r.n_out = d1; r.row_stride = d2; r.nseg = d0; r.seg_stride = d1 * d2; r.len = d2; }
        const int64_t count = r.nseg * r.len;
        r.count = (float)count;
        pl.tpr = (r.len >= 1024) ? kBlock : 32;
        // too few outputs to fill the machine and long segments: split each output
        const int64_t blocks = (pl.tpr == kBlock) ? r.n_out : (r.n_out + 7) / 8;
        if (blocks < target_blocks && r.len >= 16384) {
            int64_t want = (target_blocks + blocks - 1) / blocks;
            int64_t max_split = r.len / 4096;      // keep at least 16 KB per slice
            pl.nsplit = want < max_split ? want : max_split;
            if (pl.nsplit < 1) pl.nsplit = 1;
            if (pl.nsplit > 1) pl.tpr = kBlock;
        }
        r.nsplit = pl.nsplit;
        pl.n_out = r.n_out;
    } else {
        pl.rows = false;
        ColsParams& c = pl.cp;
        if (mask == 2) { c.outer = d0; c.r = d1; c.inner = d2; }
        else if (mask == 1) { c.outer = 1; c.r = d0; c.inner = d1 * d2; }
        else /* mask == 3 */ { c.outer = 1; c.r = d0 * d1; c.inner = d2; }
        c.count = (float)c.r;
        const int64_t col_blocks = ((c.inner + 127) / 128) * c.outer;
        if (col_blocks < target_blocks && c.r >= 256) {
            int64_t want = (target_blocks + col_blocks - 1) / col_blocks;
            int64_t max_split = c.r / 64;          // at least 64 rows per slice
            pl.nsplit = want < max_split ? want : max_split;
            if (pl.nsplit < 1) pl.nsplit = 1;
            if (pl.nsplit > 65535) pl.nsplit = 65535;
        }
        c.nsplit = pl.nsplit;
        pl.n_out = c.outer * c.inner;
    }
    return pl;
}

}  // namespace

size_t reduce_mean_scratch_bytes(int64_t d0, int64_t d1, int64_t d2, int axes_mask, int num_sms)
{
    if (d0 <= 0 || d1 <= 0 || d2 <= 0) return 0;
    Plan pl = make_plan(d0, d1, d2, axes_mask, num_sms);
    return pl.nsplit > 1 ? (size_t)(pl.n_out * pl.nsplit) * sizeof(float) : 0;
}

int launch_reduce_mean(const float* data, int64_t d0, int64_t d1, int64_t d2, float* reduced, int axes_mask,
                       float* scratch, size_t scratch_bytes, int num_sms, cudaStream_t stream, const char** err)
{
    Plan pl = make_plan(d0, d1, d2, axes_mask, num_sms);
    if (pl.n_out == 0) return 0;
    const bool split = pl.nsplit > 1;
    if (split && (scratch == nullptr || scratch_bytes < (size_t)(pl.n_out * pl.nsplit) * sizeof(float))) {
        *err = "reduce_mean: scratch buffer too small for the split reduction";
        return ACCB_ERR_LIMIT;
    }
    int launches = 0;
    float* dst = split ? scratch : reduced;
    const bool base_ok = (reinterpret_cast<uintptr_t>(data) & 15) == 0;
    if (pl.rows) {
        RowsParams& r = pl.rp;
        r.vec_ok = base_ok && (r.len % 4 == 0) && (r.row_stride % 4 == 0) && (r.seg_stride % 4 == 0);
        if (pl.tpr == kBlock) {
            if (r.n_out > 0x7fffffff) { *err = "reduce_mean: too many outputs"; return ACCB_ERR_ARG; }
            dim3 grid((unsigned)r.n_out, (unsigned)pl.nsplit);
            reduce_rows_kernel<kBlock><<<grid, kBlock, 0, stream>>>(data, dst, r);
        } else {
            const int64_t blocks = (r.n_out + 7) / 8;
            if (blocks > 0x7fffffff) { *err = "reduce_mean: too many outputs"; return ACCB_ERR_ARG; }
            dim3 grid((unsigned)blocks, 1);
            reduce_rows_kernel<32><<<grid, kBlock, 0, stream>>>(data, dst, r);
        }
        ++launches;
    } else {
        ColsParams& c = pl.cp;
        c.vec_ok = base_ok && (c.inner % 4 == 0) && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0);
        const int vec = c.vec_ok ? 4 : 1;
        const int64_t gx = (c.inner + 32 * vec - 1) / (32 * vec);
        if (gx * c.outer > 0x7fffffff) { *err = "reduce_mean: too many outputs"; return ACCB_ERR_ARG; }
        c.col_blocks = gx;
        dim3 grid((unsigned)(gx * c.outer), (unsigned)pl.nsplit);
        reduce_cols_kernel<<<grid, dim3(32, 8), 0, stream>>>(data, dst, c);
        ++launches;
    }
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess && split) {
        const float inv = pl.rows ? pl.rp.count : pl.cp.count;
        const int64_t blocks = (pl.n_out + kBlock - 1) / kBlock;
        reduce_fold_kernel<<<(unsigned)blocks, kBlock, 0, stream>>>(scratch, reduced, pl.n_out, pl.nsplit,
                                                                   pl.rows ? 0 : 1, inv);
        ++launches;
        e = cudaGetLastError();
    }
    if (e != cudaSuccess) { *err = cudaGetErrorString(e); return ACCB_ERR_CUDA; }
    note_launches(launches);
    return launches;
}

}  // namespace accb

// ---------------------------------------------------------------------------------
// accb_reduce_mean_rank3_noalloc
// ---------------------------------------------------------------------------------

namespace {

constexpr int kMaxDevicesNoAlloc = 64;
std::mutex g_noalloc_mu;
float* g_noalloc_scratch[kMaxDevicesNoAlloc];   // device address of g_static_scratch, per device
int g_noalloc_sms[kMaxDevicesNoAlloc];

bool on_device(const void* p)
{
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) { (void)cudaGetLastError(); return false; }
    return a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged;
}

}  // namespace

extern "C" int accb_reduce_mean_rank3_noalloc(const float* data, int64_t d0, int64_t d1, int64_t d2, float* reduced,
                                              int32_t axes_mask, void* cuda_stream)
{
    using accb::set_error;
    accb::clear_error();
    if (d0 < 0 || d1 < 0 || d2 < 0) return set_error(ACCB_ERR_ARG, "accb_reduce_mean_rank3_noalloc: negative dimension");
    if (axes_mask < 0 || axes_mask > 7) return set_error(ACCB_ERR_ARG, "accb_reduce_mean_rank3_noalloc: axes_mask must be in [0, 7]");
    if (axes_mask == 0) axes_mask = 7;
    const int64_t dims[3] = { d0, d1, d2 };
    int64_t n_out = 1;
    for (int d = 0; d < 3; ++d) if (!(axes_mask & (1 << d))) n_out *= dims[d];
    if (n_out == 0) return ACCB_OK;
    if (d0 * d1 * d2 == 0) return set_error(ACCB_ERR_ARG, "accb_reduce_mean_rank3_noalloc: mean over zero elements");
    if (!data || !reduced) return set_error(ACCB_ERR_ARG, "accb_reduce_mean_rank3_noalloc: null array pointer");

    // the device this thread selected with accb_set_device (made current), else the current one: the same
    // choice every other entry point makes
    int dev = -1;
    int rc = accb::selected_device(&dev);
    if (rc != ACCB_OK) return rc;
    cudaError_t e = cudaSuccess;
    if (dev < 0 || dev >= kMaxDevicesNoAlloc) return set_error(ACCB_ERR_ARG, "accb_reduce_mean_rank3_noalloc: device index out of range");
    if (!on_device(data) || !on_device(reduced))
        return set_error(ACCB_ERR_ARG, "accb_reduce_mean_rank3_noalloc: data and reduced must be device memory "
                                       "(this entry point cannot stage host buffers, it allocates nothing)");
    float* scratch = nullptr;
    int sms = 0;
    {
        // one-time set-up per device, with that device current: resolve the device address of the array
        std::lock_guard<std::mutex> lock(g_noalloc_mu);
        if (g_noalloc_scratch[dev] == nullptr) {
            float* p = nullptr;
            e = cudaGetSymbolAddress((void**)&p, g_static_scratch);
            if (e != cudaSuccess || p == nullptr) {
                (void)cudaGetLastError();
                return set_error(ACCB_ERR_CUDA, (std::string("cudaGetSymbolAddress(static scratch): ") + cudaGetErrorString(e)).c_str());
            }
            int major = 0;
            e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
            if (e != cudaSuccess) { (void)cudaGetLastError(); return set_error(ACCB_ERR_CUDA, "cudaDeviceGetAttribute(computeCapabilityMajor) failed"); }
            if (major != 10) return set_error(ACCB_ERR_CUDA, "accb_reduce_mean_rank3_noalloc: this library contains sm_100a code only");
            int n = 0;
            e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
            if (e != cudaSuccess || n <= 0) { (void)cudaGetLastError(); return set_error(ACCB_ERR_CUDA, "cudaDeviceGetAttribute(multiProcessorCount) failed"); }
            g_noalloc_sms[dev] = n;
            g_noalloc_scratch[dev] = p;
        }
        scratch = g_noalloc_scratch[dev];
        sms = g_noalloc_sms[dev];
    }
    const size_t capacity = kStaticScratchFloats * sizeof(float);
    const size_t need = accb::reduce_mean_scratch_bytes(d0, d1, d2, axes_mask, sms);
    if (need > capacity) {
        const std::string msg = "accb_reduce_mean_rank3_noalloc: this shape needs " + std::to_string(need) +
                                " bytes of partial sums but the built-in scratch holds " + std::to_string(capacity) +
                                "; use accb_reduce_mean_rank3";
        return set_error(ACCB_ERR_LIMIT, msg.c_str());
    }
    const char* err = "";
    const int n = accb::launch_reduce_mean(data, d0, d1, d2, reduced, axes_mask, scratch, capacity, sms,
                                           (cudaStream_t)cuda_stream, &err);
    if (n < 0) return set_error(n, (std::string("accb_reduce_mean_rank3_noalloc: ") + err).c_str());
    return ACCB_OK;
}

