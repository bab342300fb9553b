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

// Streams [begin, end) of one contiguous segment, 8 independent 128-bit loads in
// flight per thread (then 4, then 1 for the tail).  `vec_ok` = segment start and length are 16-byte aligned.
template <int TPR>
__device__ __forceinline__ float segment_sum(const float* __restrict__ seg, int64_t begin, int64_t end, int t, bool vec_ok)
{
    float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
    if (vec_ok) {
        const float4* v = reinterpret_cast<const float4*>(seg);
        const int64_t vb = begin >> 2, ve = end >> 2;
        int64_t i = vb + t;
        for (; i + 7 * TPR < ve; i += 8 * TPR) {
            float4 a = __ldcs(v + i);
            float4 b = __ldcs(v + i + TPR);
            float4 c = __ldcs(v + i + 2 * TPR);
            float4 d = __ldcs(v + i + 3 * TPR);
            float4 e = __ldcs(v + i + 4 * TPR);
            float4 f = __ldcs(v + i + 5 * TPR);
            float4 g = __ldcs(v + i + 6 * TPR);
            float4 h = __ldcs(v + i + 7 * TPR);
            s0 += ((a.x + a.y) + (a.z + a.w)) + ((e.x + e.y) + (e.z + e.w));
            s1 += ((b.x + b.y) + (b.z + b.w)) + ((f.x + f.y) + (f.z + f.w));
            s2 += ((c.x + c.y) + (c.z + c.w)) + ((g.x + g.y) + (g.z + g.w));
            s3 += ((d.x + d.y) + (d.z + d.w)) + ((h.x + h.y) + (h.z + h.w));
        }
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
    pdl_enter();
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
    // fold: shuffles inside each warp, then the first thread of every group adds its warps' sums in a fixed order
    s = warp_sum(s);
    if (TPR == 32) {
        if (live && t == 0) {
            if (p.nsplit == 1) out[o] = s / p.count;
            else out[o * p.nsplit + blockIdx.y] = s;
        }
    } else {
        constexpr int WPG = TPR / 32;                       // warps per group
        const int warp = threadIdx.x >> 5;
        if ((threadIdx.x & 31) == 0) smem[warp] = s;
        __syncthreads();
        if (live && t == 0) {
            float r = 0.0f;
#pragma unroll
            for (int w = 0; w < WPG; ++w) r += smem[(threadIdx.x / TPR) * WPG + w];
            if (p.nsplit == 1) out[o] = r / p.count;
            else out[o * p.nsplit + blockIdx.y] = r;
        }
    }
}

// Rows of up to VPT * 1024 elements, one block per row at a time, persistent: a block walks rows blockIdx.x,
// blockIdx.x + gridDim.x, ... and issues the loads of its next row before it folds the current one, so that the
// fold (shuffles, one shared-memory hop, one barrier) never leaves the memory pipe idle.  Used for row lengths that
// do not divide into whole rounds of 4 vectors per thread, where the block-per-row kernel ends every row with a
// partly filled round (8192 rows of 6144: 30.8 us against 34.8); on exact multiples the two are equal.
template <int VPT>
__global__ void __launch_bounds__(kBlock)
reduce_rows_stream_kernel(const float* __restrict__ data, float* __restrict__ out, int64_t n_out, int64_t row_stride,
                          int nv, float count)
{
    __shared__ float smem[2][kBlock / 32];
    pdl_enter();
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    float4 cur[VPT], nxt[VPT];
    auto load_row = [&](float4 (&v)[VPT], int64_t o) {
        const float4* row = reinterpret_cast<const float4*>(data + o * row_stride);
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int idx = t + i * kBlock;
            v[i] = idx < nv ? __ldcs(row + idx) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    };
    int64_t o = blockIdx.x;
    if (o < n_out) load_row(cur, o);
    int buf = 0;
    for (; o < n_out; o += gridDim.x) {
        const int64_t on = o + gridDim.x;
        if (on < n_out) load_row(nxt, on);
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < VPT; ++i) s += (cur[i].x + cur[i].y) + (cur[i].z + cur[i].w);
        s = warp_sum(s);
        if (lane == 0) smem[buf][warp] = s;
        __syncthreads();
        if (t == 0) {
            float r = 0.0f;
#pragma unroll
            for (int w = 0; w < kBlock / 32; ++w) r += smem[buf][w];
            out[o] = r / count;
        }
        buf ^= 1;       // the other half is rewritten only after the next barrier, which thread 0 reaches after this read
#pragma unroll
        for (int i = 0; i < VPT; ++i) cur[i] = nxt[i];
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
    pdl_enter();
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
    pdl_enter();
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

// Dimensions of size 1 carry no data movement and neighbours that are both reduced (or both kept) are one run of
// elements: squeeze and merge, so that e.g. a mean over axis 1 of (8192, 4096, 1) is recognised as the contiguous
// row reduction it is instead of a strided one with an inner extent of 1.  The order of the kept dimensions, and
// with it the order of the outputs, does not change.
void canonical_shape(int64_t& d0, int64_t& d1, int64_t& d2, int& mask)
{
    int64_t dims[3] = { d0, d1, d2 };
    int64_t ext[3];
    bool red[3];
    int n = 0;
    for (int d = 0; d < 3; ++d) {
        if (dims[d] == 1) continue;
        const bool r = (mask >> d) & 1;
        if (n > 0 && red[n - 1] == r) ext[n - 1] *= dims[d];
        else { ext[n] = dims[d]; red[n] = r; ++n; }
    }
    if (n == 0) { d0 = d1 = d2 = 1; mask = 4; return; }                                  // a single element
    if (n == 1) { d0 = 1; d1 = red[0] ? 1 : ext[0]; d2 = red[0] ? ext[0] : 1; mask = 4; return; }   // all reduced / all kept (copy)
    if (n == 2) {
        d0 = 1; d1 = ext[0]; d2 = ext[1];
        mask = red[0] ? 2 : 4;                                                           // [R, K] strided, [K, R] contiguous
        return;
    }
    d0 = ext[0]; d1 = ext[1]; d2 = ext[2];
    mask = red[0] ? 5 : 2;                                                               // [R, K, R] or [K, R, K]
}

Plan make_plan(int64_t d0, int64_t d1, int64_t d2, int mask, int num_sms, int cols_blocks_per_sm)
{
    Plan pl{};
    mask &= 7;
    if (mask == 0) mask = 7;  // ONNX: no axes = reduce everything
    canonical_shape(d0, d1, d2, mask);
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
        // A warp per output for short segments when that still gives the machine enough blocks (8192 x 4096 and
        // longer rows: a block per row wins; 32768 x 1024 and 65536 x 512: a warp per row, 24.3 us against 61.5 and
        // 112.8); a block per output otherwise, also for short segments when outputs are few.
        pl.tpr = (r.len >= 4096 || (r.len * r.nseg >= 1024 && (r.n_out + 7) / 8 < target_blocks)) ? kBlock : 32;
        if (const int forced = options().reduce_rows_tpr; forced == 32 || forced == 64 || forced == 128 || forced == 256) pl.tpr = forced;
        // too few outputs to fill the machine and long segments: split each output
        const int64_t rpb = kBlock / pl.tpr;
        const int64_t blocks = (r.n_out + rpb - 1) / rpb;
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
        const int64_t cols_target = (int64_t)cols_blocks_per_sm * num_sms;
        if (col_blocks < cols_target && c.r >= 256) {
            int64_t want = (cols_target + col_blocks - 1) / col_blocks;
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

size_t reduce_mean_scratch_bytes(int64_t d0, int64_t d1, int64_t d2, int axes_mask, int num_sms, int cols_blocks_per_sm)
{
    if (d0 <= 0 || d1 <= 0 || d2 <= 0) return 0;
    Plan pl = make_plan(d0, d1, d2, axes_mask, num_sms, cols_blocks_per_sm);
    return pl.nsplit > 1 ? (size_t)(pl.n_out * pl.nsplit) * sizeof(float) : 0;
}

int launch_reduce_mean(const float* data, int64_t d0, int64_t d1, int64_t d2, float* reduced, int axes_mask,
                       float* scratch, size_t scratch_bytes, int num_sms, cudaStream_t stream, const char** err,
                       int cols_blocks_per_sm)
{
    Plan pl = make_plan(d0, d1, d2, axes_mask, num_sms, cols_blocks_per_sm);
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
        const int64_t rpb = kBlock / pl.tpr;
        const int64_t blocks = (r.n_out + rpb - 1) / rpb;
        if (blocks > 0x7fffffff) { *err = "reduce_mean: too many outputs"; return ACCB_ERR_ARG; }
        dim3 grid((unsigned)blocks, (unsigned)pl.nsplit);
        const int64_t nv = r.len / 4;
        const bool streaming = options().reduce_rows_tpr == 0 && pl.tpr == kBlock && !split && r.nseg == 1 && r.vec_ok &&
                            nv <= 8 * kBlock && nv % (4 * kBlock) != 0 && r.n_out >= 2 * (int64_t)num_sms;
        if (streaming) {
            const unsigned g = (unsigned)(r.n_out < 8 * (int64_t)num_sms ? r.n_out : 8 * (int64_t)num_sms);
            if (nv <= 4 * kBlock) (void)launch_pdl(reduce_rows_stream_kernel<4>, dim3(g), dim3(kBlock), stream, data, dst, r.n_out, r.row_stride, (int)nv, r.count);
            else (void)launch_pdl(reduce_rows_stream_kernel<8>, dim3(g), dim3(kBlock), stream, data, dst, r.n_out, r.row_stride, (int)nv, r.count);
        } else
        switch (pl.tpr) {
        case 32: (void)launch_pdl(reduce_rows_kernel<32>, grid, dim3(kBlock), stream, data, dst, r); break;
        case 64: (void)launch_pdl(reduce_rows_kernel<64>, grid, dim3(kBlock), stream, data, dst, r); break;
        case 128: (void)launch_pdl(reduce_rows_kernel<128>, grid, dim3(kBlock), stream, data, dst, r); break;
        default: (void)launch_pdl(reduce_rows_kernel<kBlock>, grid, dim3(kBlock), stream, data, dst, r); break;
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
        (void)launch_pdl(reduce_cols_kernel, grid, dim3(32, 8), stream, data, dst, c);
        ++launches;
    }
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess && split) {
        const float inv = pl.rows ? pl.rp.count : pl.cp.count;
        const int64_t blocks = (pl.n_out + kBlock - 1) / kBlock;
        (void)launch_pdl(reduce_fold_kernel, dim3((unsigned)blocks), dim3(kBlock), stream, scratch, reduced, pl.n_out, pl.nsplit,
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
    const size_t need = accb::reduce_mean_scratch_bytes(d0, d1, d2, axes_mask, sms, accb::kNoAllocColsBlocksPerSm);
    if (need > capacity) {
        const std::string msg = "accb_reduce_mean_rank3_noalloc: this shape needs " + std::to_string(need) +
                                " bytes of partial sums but the built-in scratch holds " + std::to_string(capacity) +
                                "; use accb_reduce_mean_rank3";
        return set_error(ACCB_ERR_LIMIT, msg.c_str());
    }
    const char* err = "";
    const int n = accb::launch_reduce_mean(data, d0, d1, d2, reduced, axes_mask, scratch, capacity, sms,
                                           (cudaStream_t)cuda_stream, &err, accb::kNoAllocColsBlocksPerSm);
    if (n < 0) return set_error(n, (std::string("accb_reduce_mean_rank3_noalloc: ") + err).c_str());
    return ACCB_OK;
}

