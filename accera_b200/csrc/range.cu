// Range (ONNX) for sm_100a: output[i] = start; start = start + delta, one rounded fp32 addition per element.
//
// Reference nests: accera/python/accera/test/dsl_tests.py:1459-1462 (get_result) and
// kernels/range/naive_runtime_sized.py:25-28.  As written it is a serial recurrence - element i needs i
// rounded additions - and the reference has no GPU kernel for it.  It parallelises exactly all the same:
//
//   While the running value x stays inside one binade (same sign and exponent, so one fixed ulp u), x is a
//   multiple of u and the exact sum x + delta is rounded on that same grid.  Writing delta = q*u + r
//   (0 <= r < u), the rounded step is q or q+1 grid points depending only on r - not on x - unless r is exactly
//   u/2, where round-to-nearest-even makes the first step depend on the parity of x/u and every later step equal.
//   So inside a binade, after at most one irregular step, consecutive values differ by a constant number of
//   ulps, i.e. their BIT PATTERNS form an arithmetic progression.
//
// The host walks the recurrence binade by binade (a few steps each, O(number of binades crossed) in total)
// and emits segments (first index, first bit pattern, bit-pattern step); the kernel fills every element as
//   bits(i) = first_bits + (i - first_index) * step
// with 128-bit streaming stores.  The result is bit-identical to the serial loop for any start, delta and
// length, including denormals, sign changes, stalls (|delta| below half an ulp) and infinities.
// The kernel is a pure HBM write: 4 bytes per element.
#include <cmath>
#include <cstring>
#include <vector>

#include "accb_internal.h"

namespace accb {
namespace {

struct RangeSegment {
    int64_t first;      // index of the segment's first element
    uint32_t bits;      // bit pattern of that element
    int32_t step;       // difference of consecutive bit patterns inside the segment
};

// Segments per launch (the table travels as a kernel parameter); longer tables are issued as several launches.
// A range that keeps its sign needs about two segments per binade it crosses, so 32 covers a factor of 2^16
// between its smallest and largest magnitude in one launch.
constexpr int kMaxSegments = 32;
struct RangeTable {
    RangeSegment seg[kMaxSegments];
    int count;
};

constexpr int kBlock = 256;
constexpr int kVecPerThread = 4;                              // 128-bit stores per thread
constexpr int kPerBlock = kBlock * kVecPerThread * 4;         // 4096 elements (16 KiB) per block

__device__ __forceinline__ int find_segment(const RangeTable& t, int64_t i)
{
    int lo = 0, hi = t.count - 1;
    while (lo < hi) {                                         // segments are sorted by `first`
        const int mid = (lo + hi + 1) >> 1;
        if (t.seg[mid].first <= i) lo = mid; else hi = mid - 1;
    }
    return lo;
}

// Elements [begin, end) of the output; `table` covers exactly that index range.  Blocks own kPerBlock elements
// aligned to kPerBlock in the whole output (so a launch that starts at an odd index - a later part of a long
// table - still writes aligned vectors).  A block that lies inside one segment - all but a few dozen blocks of
// a launch - takes the branch-free path: lane-contiguous 128-bit streaming stores, one multiply and four
// additions per store.  Everything in it is 32-bit wrap-around arithmetic: only the low 32 bits of
// (i - first) * step matter.
__global__ void __launch_bounds__(kBlock)
range_fill_kernel(uint32_t* __restrict__ out, int64_t begin, int64_t end, const __grid_constant__ RangeTable table)
{
    pdl_enter();
    const int64_t block_base = (begin / kPerBlock + (int64_t)blockIdx.x) * kPerBlock;
    if (block_base >= end) return;
    const int s0 = find_segment(table, block_base < begin ? begin : block_base);
    const int64_t seg_end = (s0 + 1 < table.count) ? table.seg[s0 + 1].first : end;
    const bool whole = block_base >= begin && block_base + kPerBlock <= end && block_base + kPerBlock <= seg_end &&
                       (reinterpret_cast<uintptr_t>(out + block_base) & 15) == 0;
    if (whole) {
        const uint32_t step = (uint32_t)table.seg[s0].step;
        const uint32_t bits0 = table.seg[s0].bits + step * (uint32_t)(block_base - table.seg[s0].first);
        uint4* dst = reinterpret_cast<uint4*>(out + block_base);
#pragma unroll
        for (int q = 0; q < kVecPerThread; ++q) {
            const uint32_t e = (uint32_t)((q * kBlock + (int)threadIdx.x) * 4);
            const uint32_t v = bits0 + step * e;
            __stcs(dst + q * kBlock + threadIdx.x, make_uint4(v, v + step, v + 2 * step, v + 3 * step));
        }
        return;
    }
    // a block that straddles a segment boundary, the ragged ends of the launch, or an unaligned output
    for (int q = 0; q < kVecPerThread; ++q) {
        const int64_t i0 = block_base + (int64_t)(q * kBlock + (int)threadIdx.x) * 4;
        if (i0 >= end || i0 + 4 <= begin) continue;
        int s = find_segment(table, i0 < begin ? begin : i0);
        for (int j = 0; j < 4; ++j) {
            const int64_t i = i0 + j;
            if (i < begin || i >= end) continue;
            while (s + 1 < table.count && i >= table.seg[s + 1].first) ++s;
            out[i] = table.seg[s].bits + (uint32_t)table.seg[s].step * (uint32_t)(i - table.seg[s].first);
        }
    }
}

inline uint32_t bits_of(float x) { uint32_t b; memcpy(&b, &x, 4); return b; }
inline float float_of(uint32_t b) { float x; memcpy(&x, &b, 4); return x; }
inline bool same_binade(uint32_t a, uint32_t b) { return ((a ^ b) & 0xFF800000u) == 0; }   // sign and exponent equal

// One rounded fp32 addition, kept out of any wider-precision or fused evaluation.
inline float add_f32(float x, float d)
{
    volatile float r = x + d;
    return r;
}

// Walks v_0 = start, v_{i+1} = fl(v_i + delta) for n elements; returns v_n.
float build_segments(float start, float delta, int64_t n, std::vector<RangeSegment>& segs)
{
    float x = start;
    int64_t i = 0;
    while (i < n) {
        const uint32_t bx = bits_of(x);
        const float x1 = add_f32(x, delta);
        const uint32_t b1 = bits_of(x1);
        if (b1 == bx) {
            // fixed point (delta below half an ulp, +-inf, NaN that reproduces itself, delta == 0): constant from here on
            segs.push_back({i, bx, 0});
            return x;
        }
        const float x2 = add_f32(x1, delta);
        const uint32_t b2 = bits_of(x2);
        const int64_t d1 = (int64_t)b1 - (int64_t)bx, d2 = (int64_t)b2 - (int64_t)b1;
        if (same_binade(bx, b1) && same_binade(b1, b2) && d1 == d2) {
            // steady inside this binade: bit patterns advance by d1 until the binade ends
            const uint32_t lo = bx & 0xFF800000u, hi = bx | 0x007FFFFFu;
            // Away from zero (d1 > 0) every pattern up to the binade's last one is reached by a sum rounded on this
            // binade's grid.  Towards zero the last predicted pattern can belong to a sum whose exact value already
            // lies below the binade (it is then rounded on the finer grid underneath): stop one step earlier and
            // let the single-step branch below walk across the boundary.
            int64_t room = d1 > 0 ? ((int64_t)hi - (int64_t)bx) / d1 : ((int64_t)bx - (int64_t)lo) / (-d1) - 1;
            if (room < 0) room = 0;
            const int64_t len = (n - i < room + 1) ? n - i : room + 1;     // elements with pattern bx + j * d1, j < len
            segs.push_back({i, bx, (int32_t)d1});
            const float last = float_of((uint32_t)((int64_t)bx + (len - 1) * d1));
            x = add_f32(last, delta);                                      // first value after the segment
            i += len;
        } else {
            // a step that changes binade, or the one irregular step of a tie: a segment of a single element
            segs.push_back({i, bx, 0});
            x = x1;
            i += 1;
        }
    }
    return x;
}

}  // namespace

int64_t range_count_f32(float start, float limit, float delta)
{
    // floor((limit - start) / delta) in fp32 (dsl_tests.py:1452-1454, 1482); negative, NaN or huge -> 0
    const float span = add_f32(limit, -start);
    volatile float q = span / delta;
    const float f = std::floor(q);
    if (!(f >= 0.0f) || f >= 9.2e18f) return 0;
    return (int64_t)f;
}

int64_t range_plan_f32(float start, float delta, int64_t n, int64_t* first, uint32_t* bits, int32_t* step, int64_t capacity,
                       float* final_value)
{
    std::vector<RangeSegment> segs;
    const float last = build_segments(start, delta, n, segs);
    if (final_value) *final_value = last;
    for (size_t j = 0; j < segs.size() && (int64_t)j < capacity; ++j) {
        if (first) first[j] = segs[j].first;
        if (bits) bits[j] = segs[j].bits;
        if (step) step[j] = segs[j].step;
    }
    return (int64_t)segs.size();
}

int launch_range_f32(int64_t n, float* output, float start, float delta, float* final_value, cudaStream_t stream,
                     const char** err)
{
    std::vector<RangeSegment> segs;
    const float last = build_segments(start, delta, n, segs);
    if (final_value) *final_value = last;
    int launches = 0;
    for (size_t s0 = 0; s0 < segs.size(); s0 += kMaxSegments) {
        RangeTable table;
        table.count = (int)((segs.size() - s0 < (size_t)kMaxSegments) ? segs.size() - s0 : (size_t)kMaxSegments);
        for (int j = 0; j < table.count; ++j) table.seg[j] = segs[s0 + j];
        const int64_t begin = table.seg[0].first;
        const int64_t end = (s0 + kMaxSegments < segs.size()) ? segs[s0 + kMaxSegments].first : n;
        const int64_t blocks = (end - (begin / kPerBlock) * kPerBlock + kPerBlock - 1) / kPerBlock;
        if (blocks > 0x7fffffff) { *err = "range: too many elements for this kernel's grid"; return ACCB_ERR_ARG; }
        if (blocks == 0) continue;
        cudaError_t e = launch_pdl(range_fill_kernel, dim3((unsigned)blocks), dim3(kBlock), stream, reinterpret_cast<uint32_t*>(output),
                                   begin, end, table);
        if (e == cudaSuccess) e = cudaGetLastError();
        if (e != cudaSuccess) { *err = cudaGetErrorString(e); return ACCB_ERR_CUDA; }
        ++launches;
    }
    note_launches(launches);
    return launches;
}

}  // namespace accb
