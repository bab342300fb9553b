// CUDA-core (SIMT) GEMM with the fused epilogue, for sm_100a.
//
//   C <- epi(alpha * (A @ B) + beta * C + bias)
//
// This is the bit-faithful fp32 path (true fp32 FMA, no TF32) and the general
// path for every element-type / layout combination the tensor-core kernel does
// not take: f32, f16, bf16 inputs with an fp32 accumulator, s8/u8 inputs with an
// int32 accumulator, arbitrary element strides (row- or column-major operands).
//
// It replaces the generated per-thread kernel of the reference
// (docs/Tutorials/GPU/Hello_MatMul_GPU.md:161-191: one thread per C element, C
// read-modify-written in global memory every k) by a shared-memory tiled kernel:
// BM x BN output tile per block, BK-deep k tiles double buffered in shared
// memory with the next tile prefetched into registers, TM x TN register tile per
// thread, the epilogue applied once to the register tile before the only store.
#include <cuda_fp16.h>
#include <cuda_bf16.h>

#include <cstdlib>
#include <type_traits>

#include "accb_internal.h"

namespace accb {
namespace {

struct SimtParams {
    int64_t m, n, k;
    int64_t as0, as1, bs0, bs1, cs0, cs1;
    float alpha, beta;
    int relu;
    int64_t a_bs, b_bs, c_bs;   // batched GEMM: element offsets between consecutive problems (blockIdx.z walks them)
};

template <typename ACC, typename T>
__device__ __forceinline__ ACC widen(T v);
template <> __device__ __forceinline__ float widen<float, float>(float v) { return v; }
template <> __device__ __forceinline__ float widen<float, __half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float widen<float, __nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ int widen<int, int8_t>(int8_t v) { return (int)v; }
template <> __device__ __forceinline__ int widen<int, uint8_t>(uint8_t v) { return (int)v; }
template <> __device__ __forceinline__ int widen<int, int16_t>(int16_t v) { return (int)v; }

template <typename T>
__device__ __forceinline__ T narrow(float v);
template <> __device__ __forceinline__ float narrow<float>(float v) { return v; }
template <> __device__ __forceinline__ __half narrow<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 narrow<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <typename T>
__device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename TA, typename TB, typename TC, typename ACC, int BM, int BN, int BK, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
gemm_simt_kernel(const TA* __restrict__ A, const TB* __restrict__ B, TC* __restrict__ C,
                 const float* __restrict__ bias, SimtParams p)
{
    constexpr int NT = (BM / TM) * (BN / TN);
    constexpr int LA = (BM * BK) / NT;
    constexpr int LB = (BN * BK) / NT;
    static_assert((BM * BK) % NT == 0 && (BN * BK) % NT == 0, "tile must divide evenly over the threads");
    constexpr int PAD = 4;

    __shared__ ACC As[2][BK][BM + PAD];
    __shared__ ACC Bs[2][BK][BN + PAD];

    const int tid = threadIdx.x;
    const int tx = tid % (BN / TN);
    const int ty = tid / (BN / TN);
    const int64_t m0 = (int64_t)blockIdx.y * BM;
    const int64_t n0 = (int64_t)blockIdx.x * BN;
    A += (int64_t)blockIdx.z * p.a_bs;
    B += (int64_t)blockIdx.z * p.b_bs;
    C += (int64_t)blockIdx.z * p.c_bs;

    // Walk the tile along whichever dimension is contiguous in global memory so
    // that consecutive threads read consecutive addresses.
    const bool a_kfast = (p.as1 == 1);
    const bool b_kfast = (p.bs0 == 1);

    ACC ra[LA], rb[LB];

    auto fetch = [&](int64_t k0) {
#pragma unroll
        for (int l = 0; l < LA; ++l) {
            int e = tid + l * NT;
            int mm = a_kfast ? e / BK : e % BM;
            int kk = a_kfast ? e % BK : e / BM;
            int64_t gm = m0 + mm, gk = k0 + kk;
            ra[l] = (gm < p.m && gk < p.k) ? widen<ACC, TA>(A[gm * p.as0 + gk * p.as1]) : ACC(0);
        }
#pragma unroll
        for (int l = 0; l < LB; ++l) {
            int e = tid + l * NT;
            int nn = b_kfast ? e / BK : e % BN;
            int kk = b_kfast ? e % BK : e / BN;
            int64_t gn = n0 + nn, gk = k0 + kk;
            rb[l] = (gn < p.n && gk < p.k) ? widen<ACC, TB>(B[gk * p.bs0 + gn * p.bs1]) : ACC(0);
        }
    };
    auto stash = [&](int buf) {
#pragma unroll
        for (int l = 0; l < LA; ++l) {
            int e = tid + l * NT;
            int mm = a_kfast ? e / BK : e % BM;
            int kk = a_kfast ? e % BK : e / BM;
            As[buf][kk][mm] = ra[l];
        }
#pragma unroll
        for (int l = 0; l < LB; ++l) {
            int e = tid + l * NT;
            int nn = b_kfast ? e / BK : e % BN;
            int kk = b_kfast ? e % BK : e / BN;
            Bs[buf][kk][nn] = rb[l];
        }
    };

    // alpha = beta = 1 with a floating-point accumulator: start from C (see gemm_simt_f32_rr_kernel); integer
    // accumulation is exact in any order
    const bool from_c = !std::is_same<ACC, int>::value && p.alpha == 1.0f && p.beta == 1.0f;
    ACC acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i) {
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            acc[i][j] = ACC(0);
            if constexpr (!std::is_same<ACC, int>::value) {
                const int64_t gm = m0 + ty * TM + i, gn = n0 + tx * TN + j;
                if (from_c && gm < p.m && gn < p.n) acc[i][j] = (ACC)to_float<TC>(C[gm * p.cs0 + gn * p.cs1]);
            }
        }
    }

    const int64_t kt_count = (p.k + BK - 1) / BK;
    if (kt_count > 0) {
        fetch(0);
        stash(0);
    }
    __syncthreads();

    for (int64_t kt = 0; kt < kt_count; ++kt) {
        const int buf = (int)(kt & 1);
        const bool more = (kt + 1 < kt_count);
        if (more) fetch((kt + 1) * BK);
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            ACC av[TM], bv[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) av[i] = As[buf][kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) bv[j] = Bs[buf][kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] += av[i] * bv[j];
        }
        if (more) stash(buf ^ 1);
        __syncthreads();
    }

    // fused epilogue: one read of C (if beta != 0), one write
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int64_t gm = m0 + ty * TM + i;
        if (gm >= p.m) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int64_t gn = n0 + tx * TN + j;
            if (gn >= p.n) continue;
            TC* dst = C + gm * p.cs0 + gn * p.cs1;
            if constexpr (std::is_same<ACC, int>::value) {
                int v = acc[i][j];
                if (p.beta != 0.0f) v += (int)(*dst);
                if (p.relu && v < 0) v = 0;
                *dst = (TC)v;
            } else {
                float v = (float)acc[i][j];
                if (from_c) {
                    // C is already inside the accumulator
                } else if (p.alpha == 1.0f) {
                    if (p.beta == 1.0f) v += to_float<TC>(*dst);
                    else if (p.beta != 0.0f) v += p.beta * to_float<TC>(*dst);
                } else {
                    v *= p.alpha;
                    if (p.beta != 0.0f) v += p.beta * to_float<TC>(*dst);
                }
                if (bias) v += bias[gn];
                if (p.relu) v = fmaxf(v, 0.0f);
                *dst = narrow<TC>(v);
            }
        }
    }
}

// ---------------------------------------------------------------------------------
// fp32, row-major A / B / C: the quickstart layout.  Same arithmetic (fp32 FMA, k in
// order inside a thread) but operands reach shared memory through a multi-stage
// cp.async pipeline (16-byte copies, zero-filled at the ragged edges), so global-
// memory latency is paid once in the prologue instead of once per k tile - at
// 512^3 the kernel is otherwise bound by exactly that latency.
// ---------------------------------------------------------------------------------

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src, int src_bytes)
{
    const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gmem_src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int BM, int BN, int BK, int TM, int TN, int STAGES>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
gemm_simt_f32_rr_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C,
                        const float* __restrict__ bias, SimtParams p)
{
    constexpr int NT = (BM / TM) * (BN / TN);
    constexpr int LDA_S = BK + 4;                  // floats per A row in shared memory (16-byte aligned, conflict-free)
    constexpr int LDB_S = BN + 4;
    constexpr int A_STAGE = BM * LDA_S, B_STAGE = BK * LDB_S;
    constexpr int A_CHUNKS = BM * BK / 4, B_CHUNKS = BK * BN / 4;
    static_assert(TN == 4 && BK % 4 == 0, "thread tile is 4 columns wide; k tiles are whole 16-byte chunks");
    static_assert(A_CHUNKS % NT == 0 || A_CHUNKS < NT, "A chunks must divide over the threads");
    static_assert(B_CHUNKS % NT == 0, "B chunks must divide over the threads");
    extern __shared__ __align__(16) float smem_f[];
    float* As = smem_f;
    float* Bs = smem_f + STAGES * A_STAGE;

    const int tid = threadIdx.x;
    const int tx = tid % (BN / TN);
    const int ty = tid / (BN / TN);
    const int64_t m0 = (int64_t)blockIdx.y * BM;
    const int64_t n0 = (int64_t)blockIdx.x * BN;
    const int64_t kt_count = (p.k + BK - 1) / BK;
    A += (int64_t)blockIdx.z * p.a_bs;
    B += (int64_t)blockIdx.z * p.b_bs;
    C += (int64_t)blockIdx.z * p.c_bs;

    auto load_stage = [&](int stage, int64_t kt) {
        const int64_t k0 = kt * BK;
#pragma unroll
        for (int c = tid; c < A_CHUNKS; c += NT) {
            const int r = c / (BK / 4), kc = (c % (BK / 4)) * 4;
            const int64_t gm = m0 + r, gk = k0 + kc;
            int bytes = 0;
            if (gm < p.m && gk < p.k) bytes = (int)((p.k - gk >= 4 ? 4 : p.k - gk) * 4);
            const float* src = bytes ? A + gm * p.as0 + gk : A;
            cp_async16(As + stage * A_STAGE + r * LDA_S + kc, src, bytes);
        }
#pragma unroll
        for (int c = tid; c < B_CHUNKS; c += NT) {
            const int r = c / (BN / 4), nc = (c % (BN / 4)) * 4;
            const int64_t gk = k0 + r, gn = n0 + nc;
            int bytes = 0;
            if (gk < p.k && gn < p.n) bytes = (int)((p.n - gn >= 4 ? 4 : p.n - gn) * 4);
            const float* src = bytes ? B + gk * p.bs0 + gn : B;
            cp_async16(Bs + stage * B_STAGE + r * LDB_S + nc, src, bytes);
        }
    };

    // C += A @ B (alpha = beta = 1, what a HAT matmul is): the accumulator starts from C and the products are added
    // to it in k order, the order of the reference's nest (its compiled packages print 1536.419922 for
    // 0.42 + 256 * 6, the value of this order; summing the products first and adding C last gives 1536.420044)
    const bool from_c = (p.alpha == 1.0f && p.beta == 1.0f);
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i) {
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;
        const int64_t gm = m0 + ty * TM + i, gn = n0 + tx * TN;
        if (from_c && gm < p.m) {
#pragma unroll
            for (int j = 0; j < TN; ++j) if (gn + j < p.n) acc[i][j] = C[gm * p.cs0 + gn + j];
        }
    }

#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (s < kt_count) load_stage(s, s);
        cp_async_commit();
    }
    for (int64_t kt = 0; kt < kt_count; ++kt) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();                       // tile kt has landed; tile kt-1's buffer is free again
        if (kt + STAGES - 1 < kt_count) load_stage((int)((kt + STAGES - 1) % STAGES), kt + STAGES - 1);
        cp_async_commit();
        const float* as = As + (kt % STAGES) * A_STAGE + (ty * TM) * LDA_S;
        const float* bs = Bs + (kt % STAGES) * B_STAGE + tx * TN;
        // register double buffering: the fragments of the next 4 k are loaded while the current 4 are used,
        // so that shared-memory latency is covered even with two warps per scheduler
        float4 a_cur[TM], b_cur[4], a_nxt[TM], b_nxt[4];
#pragma unroll
        for (int i = 0; i < TM; ++i) a_cur[i] = *reinterpret_cast<const float4*>(as + i * LDA_S);
#pragma unroll
        for (int q = 0; q < 4; ++q) b_cur[q] = *reinterpret_cast<const float4*>(bs + q * LDB_S);
#pragma unroll
        for (int kk = 0; kk < BK; kk += 4) {
            if (kk + 4 < BK) {
#pragma unroll
                for (int i = 0; i < TM; ++i) a_nxt[i] = *reinterpret_cast<const float4*>(as + i * LDA_S + kk + 4);
#pragma unroll
                for (int q = 0; q < 4; ++q) b_nxt[q] = *reinterpret_cast<const float4*>(bs + (kk + 4 + q) * LDB_S);
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float4 bv = b_cur[q];
#pragma unroll
                for (int i = 0; i < TM; ++i) {
                    const float a = q == 0 ? a_cur[i].x : q == 1 ? a_cur[i].y : q == 2 ? a_cur[i].z : a_cur[i].w;
                    acc[i][0] += a * bv.x; acc[i][1] += a * bv.y; acc[i][2] += a * bv.z; acc[i][3] += a * bv.w;
                }
            }
            if (kk + 4 < BK) {
#pragma unroll
                for (int i = 0; i < TM; ++i) a_cur[i] = a_nxt[i];
#pragma unroll
                for (int q = 0; q < 4; ++q) b_cur[q] = b_nxt[q];
            }
        }
    }
    cp_async_wait<0>();

    const bool c_vec = (p.cs0 % 4 == 0) && ((reinterpret_cast<uintptr_t>(C) & 15) == 0);
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int64_t gm = m0 + ty * TM + i;
        if (gm >= p.m) continue;
        const int64_t gn = n0 + tx * TN;
        if (gn >= p.n) continue;
        float* dst = C + gm * p.cs0 + gn;
        float v[4] = { acc[i][0], acc[i][1], acc[i][2], acc[i][3] };
        const int ncols = (int)(p.n - gn >= 4 ? 4 : p.n - gn);
        float old[4] = { 0.f, 0.f, 0.f, 0.f };
        if (p.beta != 0.0f && !from_c) {
            if (c_vec && ncols == 4) { const float4 o = *reinterpret_cast<const float4*>(dst); old[0] = o.x; old[1] = o.y; old[2] = o.z; old[3] = o.w; }
            else {
#pragma unroll
                for (int j = 0; j < 4; ++j) if (j < ncols) old[j] = dst[j];
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float x = v[j];
            if (from_c) {
                // C is already inside the accumulator
            } else if (p.alpha == 1.0f) {
                if (p.beta == 1.0f) x += old[j];
                else if (p.beta != 0.0f) x += p.beta * old[j];
            } else {
                x *= p.alpha;
                if (p.beta != 0.0f) x += p.beta * old[j];
            }
            if (bias && j < ncols) x += bias[gn + j];
            if (p.relu) x = fmaxf(x, 0.0f);
            v[j] = x;
        }
        if (c_vec && ncols == 4) *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
        else {
#pragma unroll
            for (int j = 0; j < 4; ++j) if (j < ncols) dst[j] = v[j];
        }
    }
}

template <int BM, int BN, int BK, int TM, int TN, int STAGES>
cudaError_t launch_f32_rr(const GemmLaunch& g, const SimtParams& p)
{
    constexpr int NT = (BM / TM) * (BN / TN);
    constexpr size_t smem = (size_t)STAGES * (BM * (BK + 4) + BK * (BN + 4)) * sizeof(float);
    auto kernel = gemm_simt_f32_rr_kernel<BM, BN, BK, TM, TN, STAGES>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    dim3 grid((unsigned)((p.n + BN - 1) / BN), (unsigned)((p.m + BM - 1) / BM), (unsigned)g.batch);
    kernel<<<grid, NT, smem, g.stream>>>((const float*)g.a, (const float*)g.b, (float*)g.c, g.bias, p);
    return cudaGetLastError();
}

// true when the cp.async kernel can take the problem: unit-stride rows, 16-byte aligned row starts
bool f32_rr_ok(const GemmLaunch& g, const SimtParams& p)
{
    return p.as1 == 1 && p.bs1 == 1 && p.cs1 == 1 && p.as0 % 4 == 0 && p.bs0 % 4 == 0 &&
           p.a_bs % 4 == 0 && p.b_bs % 4 == 0 &&
           (reinterpret_cast<uintptr_t>(g.a) & 15) == 0 && (reinterpret_cast<uintptr_t>(g.b) & 15) == 0 && p.k > 0;
}

// ---------------------------------------------------------------------------------
// fp32, row-major A / B / C, 128 x 128 tile with 8 x 8 register tiles, optional split along K.
//
// With 2 x 4 register tiles the kernel above spends more cycles on shared-memory wavefronts than on FMAs;
// 8 x 8 tiles balance the two, but a 512^3 problem then has only 16 tiles for 148 SMs.  So K is split over
// a thread-block CLUSTER: the `splits` (1, 2, 4 or 8) CTAs of a cluster work on one output tile, each over
// its own K range, park their partial tile in their own shared memory, and after a cluster barrier every
// CTA folds 1/splits of the tile's rows by reading all the partials through distributed shared memory - in
// split order, so the result does not depend on timing - applies the epilogue and writes C.  No global
// workspace, no atomics.
// ---------------------------------------------------------------------------------

struct SplitKParams {
    int splits;              // cluster size along z
    int64_t k_per_split;     // multiple of 16
};

__device__ __forceinline__ float4 ld_dsmem_f4(uint32_t local_addr, uint32_t cta)
{
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(cta));
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote));
    return v;
}

__global__ void __launch_bounds__(256, 2)
gemm_simt_f32_8x8_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C,
                         const float* __restrict__ bias, SimtParams p, SplitKParams sk)
{
    constexpr int BM = 128, BN = 128, BK = 16, LDS_ = BM + 4;
    pdl_enter();    // launched with programmatic stream serialization: wait for the stream's earlier work before any access
    // 64 KB: the k-tile buffers during the main loop (2 x 2 x 16 x 132 floats = 33 KB), the whole partial tile after it
    extern __shared__ __align__(16) float smem_f[];
    float (*As)[BK][LDS_] = reinterpret_cast<float (*)[BK][LDS_]>(smem_f);                       // As[2][k][m]
    float (*Bs)[BK][LDS_] = reinterpret_cast<float (*)[BK][LDS_]>(smem_f + 2 * BK * LDS_);       // Bs[2][k][n]
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int64_t m0 = (int64_t)blockIdx.y * BM, n0 = (int64_t)blockIdx.x * BN;
    // blockIdx.z = problem * splits + split; clusters are 1 x 1 x splits, so `split` is also the rank in the cluster
    const int split = (int)(blockIdx.z % (unsigned)sk.splits);
    const int64_t problem = (int64_t)(blockIdx.z / (unsigned)sk.splits);
    A += problem * p.a_bs;
    B += problem * p.b_bs;
    C += problem * p.c_bs;
    const int64_t k_begin = (int64_t)split * sk.k_per_split;
    const int64_t k_end = (k_begin + sk.k_per_split < p.k) ? k_begin + sk.k_per_split : p.k;
    const int64_t kt_count = (k_end > k_begin) ? (k_end - k_begin + BK - 1) / BK : 0;

    float4 ra[2], rb[2];
    auto fetch = [&](int64_t k0) {
#pragma unroll
        for (int l = 0; l < 2; ++l) {
            const int idx = tid + l * 256;
            const int mm = idx >> 2, kq = (idx & 3) * 4;                  // A: 128 rows x 4 float4 along k
            const int64_t gm = m0 + mm, gk = k0 + kq;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (gm < p.m && gk < k_end) {
                const float* src = A + gm * p.as0 + gk;
                if (gk + 4 <= k_end) v = *reinterpret_cast<const float4*>(src);
                else { v.x = src[0]; if (gk + 1 < k_end) v.y = src[1]; if (gk + 2 < k_end) v.z = src[2]; }
            }
            ra[l] = v;
            const int kk = idx >> 5, nq = (idx & 31) * 4;                 // B: 16 rows x 32 float4 along n
            const int64_t gk2 = k0 + kk, gn = n0 + nq;
            float4 w = make_float4(0.f, 0.f, 0.f, 0.f);
            if (gk2 < k_end && gn < p.n) {
                const float* src = B + gk2 * p.bs0 + gn;
                if (gn + 4 <= p.n) w = *reinterpret_cast<const float4*>(src);
                else { w.x = src[0]; if (gn + 1 < p.n) w.y = src[1]; if (gn + 2 < p.n) w.z = src[2]; }
            }
            rb[l] = w;
        }
    };
    auto stash = [&](int buf) {
#pragma unroll
        for (int l = 0; l < 2; ++l) {
            const int idx = tid + l * 256;
            const int mm = idx >> 2, kq = (idx & 3) * 4;
            As[buf][kq + 0][mm] = ra[l].x; As[buf][kq + 1][mm] = ra[l].y;
            As[buf][kq + 2][mm] = ra[l].z; As[buf][kq + 3][mm] = ra[l].w;
            const int kk = idx >> 5, nq = (idx & 31) * 4;
            *reinterpret_cast<float4*>(&Bs[buf][kk][nq]) = rb[l];
        }
    };

    // this thread's 8 rows are ty*4 .. +3 and 64 + ty*4 .. +3, its 8 columns tx*4 .. +3 and 64 + tx*4 .. +3:
    // the two 4-wide halves keep every 128-bit shared-memory load of a warp phase inside one 128-byte line
    // (This kernel adds C in the epilogue: starting the 64 accumulators from C, as the smaller-tile kernels do for
    // alpha = beta = 1, cost 19 % at 4096^3 under this kernel's 128-register budget.)
    constexpr bool from_c = false;
    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.0f;

    if (kt_count > 0) { fetch(k_begin); stash(0); }
    __syncthreads();
    for (int64_t kt = 0; kt < kt_count; ++kt) {
        const int buf = (int)(kt & 1);
        const bool more = kt + 1 < kt_count;
        if (more) fetch(k_begin + (kt + 1) * BK);
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            const float4 a0 = *reinterpret_cast<const float4*>(&As[buf][kk][ty * 4]);
            const float4 a1 = *reinterpret_cast<const float4*>(&As[buf][kk][64 + ty * 4]);
            const float4 b0 = *reinterpret_cast<const float4*>(&Bs[buf][kk][tx * 4]);
            const float4 b1 = *reinterpret_cast<const float4*>(&Bs[buf][kk][64 + tx * 4]);
            const float av[8] = { a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w };
            const float bv[8] = { b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w };
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] += av[i] * bv[j];
        }
        if (more) stash(buf ^ 1);
        __syncthreads();
    }

    const bool c_vec = (p.cs0 % 4 == 0) && ((reinterpret_cast<uintptr_t>(C) & 15) == 0);
    auto finish4 = [&](float4 v4, int64_t gm, int64_t gn) {          // epilogue + store of 4 consecutive columns
        if (gm >= p.m || gn >= p.n) return;
        float* dst = C + gm * p.cs0 + gn;
        const int ncols = (int)(p.n - gn >= 4 ? 4 : p.n - gn);
        float v[4] = { v4.x, v4.y, v4.z, v4.w };
        float old[4] = { 0.f, 0.f, 0.f, 0.f };
        if (p.beta != 0.0f && !from_c) {
            if (c_vec && ncols == 4) { const float4 o = *reinterpret_cast<const float4*>(dst); old[0] = o.x; old[1] = o.y; old[2] = o.z; old[3] = o.w; }
            else {
#pragma unroll
                for (int j = 0; j < 4; ++j) if (j < ncols) old[j] = dst[j];
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float x = v[j];
            if (from_c) {
                // C is already inside the accumulator
            } else if (p.alpha == 1.0f) {
                if (p.beta == 1.0f) x += old[j];
                else if (p.beta != 0.0f) x += p.beta * old[j];
            } else {
                x *= p.alpha;
                if (p.beta != 0.0f) x += p.beta * old[j];
            }
            if (bias && j < ncols) x += bias[gn + j];
            if (p.relu) x = fmaxf(x, 0.0f);
            v[j] = x;
        }
        if (c_vec && ncols == 4) *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
        else {
#pragma unroll
            for (int j = 0; j < 4; ++j) if (j < ncols) dst[j] = v[j];
        }
    };

    if (sk.splits == 1) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int64_t gm = m0 + ((i < 4) ? ty * 4 + i : 64 + ty * 4 + (i - 4));
            finish4(make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]), gm, n0 + tx * 4);
            finish4(make_float4(acc[i][4], acc[i][5], acc[i][6], acc[i][7]), gm, n0 + 64 + tx * 4);
        }
        return;
    }

    // park the partial tile in shared memory, row-major [128][128] (the k-tile buffers are no longer needed:
    // the loop above ended with a __syncthreads)
    float* part = smem_f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int r = (i < 4) ? ty * 4 + i : 64 + ty * 4 + (i - 4);
        *reinterpret_cast<float4*>(part + r * BN + tx * 4) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
        *reinterpret_cast<float4*>(part + r * BN + 64 + tx * 4) = make_float4(acc[i][4], acc[i][5], acc[i][6], acc[i][7]);
    }
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    // CTA `split` folds rows [split * 128 / splits, (split + 1) * 128 / splits) of the tile
    const int rows_per = BM / sk.splits;
    const int vec_count = rows_per * (BN / 4);
    const uint32_t part_addr = (uint32_t)__cvta_generic_to_shared(part);
    for (int v = tid; v < vec_count; v += 256) {
        const int r = split * rows_per + v / (BN / 4), c4 = v % (BN / 4);
        const uint32_t off = (uint32_t)((r * BN + c4 * 4) * sizeof(float));
        float4 q[8];
#pragma unroll
        for (int s = 0; s < 8; ++s) if (s < sk.splits) q[s] = ld_dsmem_f4(part_addr + off, (uint32_t)s);
        float4 sum = q[0];
#pragma unroll
        for (int s = 1; s < 8; ++s)
            if (s < sk.splits) { sum.x += q[s].x; sum.y += q[s].y; sum.z += q[s].z; sum.w += q[s].w; }   // fixed order
        finish4(sum, m0 + r, n0 + c4 * 4);
    }
    // no CTA may leave while another one is still reading its shared memory
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// How the 8 x 8 kernel would be launched for this problem: number of K splits (1 = no split)
struct SplitPlan { int splits; int64_t k_per_split; int64_t tiles; bool use; };

SplitPlan plan_8x8(const SimtParams& p, int num_sms, int64_t batch)
{
    SplitPlan sp{1, 0, 0, false};
    const int64_t tiles = ((p.m + 127) / 128) * ((p.n + 127) / 128) * batch;
    sp.tiles = tiles;
    if (p.k < 16 || (p.m + 127) / 128 > 65535) return sp;
    sp.k_per_split = (p.k + 15) / 16 * 16;
    if (tiles >= 2 * (int64_t)num_sms) { sp.use = true; return sp; }       // big: no split
    // small: the largest power-of-two split (<= 8, >= 64 of K each) that does not overfill two CTAs per SM
    int s = 1;
    while (s < 8 && tiles * (s * 2) <= 2 * (int64_t)num_sms && p.k / (s * 2) >= 64) s *= 2;
    sp.splits = s;
    sp.k_per_split = ((p.k + s - 1) / s + 15) / 16 * 16;
    // worth it only if the grid is then reasonably full; otherwise the smaller-tile kernel does better
    sp.use = tiles * s >= num_sms / 2;
    return sp;
}

template <typename TA, typename TB, typename TC, typename ACC>
cudaError_t launch_typed(const GemmLaunch& g, const SimtParams& p)
{
    const int64_t tiles64 = ((p.m + 63) / 64) * ((p.n + 63) / 64) * g.batch;
    if (tiles64 >= 2 * (int64_t)g.num_sms) {
        constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;
        dim3 grid((unsigned)((p.n + BN - 1) / BN), (unsigned)((p.m + BM - 1) / BM), (unsigned)g.batch);
        gemm_simt_kernel<TA, TB, TC, ACC, BM, BN, BK, TM, TN><<<grid, (BM / TM) * (BN / TN), 0, g.stream>>>(
            (const TA*)g.a, (const TB*)g.b, (TC*)g.c, g.bias, p);
    } else {
        // small problems: smaller tiles so that the grid still covers the SMs
        constexpr int BM = 32, BN = 64, BK = 16, TM = 2, TN = 4;
        dim3 grid((unsigned)((p.n + BN - 1) / BN), (unsigned)((p.m + BM - 1) / BM), (unsigned)g.batch);
        gemm_simt_kernel<TA, TB, TC, ACC, BM, BN, BK, TM, TN><<<grid, (BM / TM) * (BN / TN), 0, g.stream>>>(
            (const TA*)g.a, (const TB*)g.b, (TC*)g.c, g.bias, p);
    }
    return cudaGetLastError();
}

}  // namespace

int launch_gemm_simt(const GemmLaunch& g, const char** err)
{
    const accb_gemm_desc& d = g.d;
    SimtParams p;
    p.m = d.m; p.n = d.n; p.k = d.k;
    p.as0 = d.a_stride[0]; p.as1 = d.a_stride[1];
    p.bs0 = d.b_stride[0]; p.bs1 = d.b_stride[1];
    p.cs0 = d.c_stride[0]; p.cs1 = d.c_stride[1];
    p.alpha = d.alpha; p.beta = d.beta; p.relu = (d.epilogue == ACCB_EPI_RELU);
    p.a_bs = g.a_batch_stride; p.b_bs = g.b_batch_stride; p.c_bs = g.c_batch_stride;
    if (d.m == 0 || d.n == 0 || g.batch <= 0) return 0;
    constexpr int64_t kMaxProblems = 8191;      // blockIdx.z carries problem * splits + split, splits <= 8
    if (g.batch > kMaxProblems) {
        auto esize = [](int t) { return (t == ACCB_F32 || t == ACCB_S32) ? 4 : (t == ACCB_F16 || t == ACCB_BF16) ? 2 : 1; };
        int total = 0;
        for (int64_t b0 = 0; b0 < g.batch; b0 += kMaxProblems) {
            GemmLaunch part = g;
            part.batch = (g.batch - b0 < kMaxProblems) ? g.batch - b0 : kMaxProblems;
            part.a = (const char*)g.a + b0 * g.a_batch_stride * esize(d.a_type);
            part.b = (const char*)g.b + b0 * g.b_batch_stride * esize(d.b_type);
            part.c = (char*)g.c + b0 * g.c_batch_stride * esize(d.c_type);
            const int n = launch_gemm_simt(part, err);
            if (n < 0) return n;
            total += n;
        }
        return total;
    }
    if ((d.m + 31) / 32 > 65535) { *err = "SIMT GEMM: M too large for this kernel's grid"; return ACCB_ERR_ARG; }

    cudaError_t e;
    const int a = d.a_type, b = d.b_type, c = d.c_type;
    if (a == ACCB_F32 && b == ACCB_F32 && c == ACCB_F32) {
        const SplitPlan sp = f32_rr_ok(g, p) ? plan_8x8(p, g.num_sms, g.batch) : SplitPlan{1, 0, 0, false};
        if (sp.use) {
            SplitKParams sk;
            sk.splits = sp.splits;
            sk.k_per_split = sp.k_per_split;
            constexpr int kSmem = 128 * 128 * (int)sizeof(float);
            e = cudaFuncSetAttribute(gemm_simt_f32_8x8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
            if (e == cudaSuccess) {
                cudaLaunchConfig_t cfg = {};
                cfg.gridDim = dim3((unsigned)((p.n + 127) / 128), (unsigned)((p.m + 127) / 128), (unsigned)(sp.splits * g.batch));
                cfg.blockDim = dim3(256);
                cfg.dynamicSmemBytes = kSmem;
                cfg.stream = g.stream;
                cudaLaunchAttribute attr[2];
                attr[0].id = cudaLaunchAttributeClusterDimension;
                attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = (unsigned)sp.splits;
                // two of these CTAs fit an SM, so the next launch of a stream can be resident (and past its set-up)
                // before this one has finished
                attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
                attr[1].val.programmaticStreamSerializationAllowed = options().stream_pdl == 0 ? 0 : 1;
                cfg.attrs = attr; cfg.numAttrs = 2;
                e = cudaLaunchKernelEx(&cfg, gemm_simt_f32_8x8_kernel, (const float*)g.a, (const float*)g.b, (float*)g.c, g.bias, p, sk);
            }
        } else if (f32_rr_ok(g, p)) {
            const int64_t tiles64 = ((p.m + 63) / 64) * ((p.n + 63) / 64) * g.batch;
            if (tiles64 >= 2 * (int64_t)g.num_sms) e = launch_f32_rr<64, 64, 32, 4, 4, 3>(g, p);
            else e = launch_f32_rr<32, 64, 32, 2, 4, 4>(g, p);       // small problems: more, smaller tiles
        } else {
            e = launch_typed<float, float, float, float>(g, p);
        }
    }
    else if (a == ACCB_F16 && b == ACCB_F16 && c == ACCB_F32) e = launch_typed<__half, __half, float, float>(g, p);
    else if (a == ACCB_F16 && b == ACCB_F16 && c == ACCB_F16) e = launch_typed<__half, __half, __half, float>(g, p);
    else if (a == ACCB_BF16 && b == ACCB_BF16 && c == ACCB_F32) e = launch_typed<__nv_bfloat16, __nv_bfloat16, float, float>(g, p);
    else if (a == ACCB_BF16 && b == ACCB_BF16 && c == ACCB_BF16) e = launch_typed<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16, float>(g, p);
    else if (a == ACCB_S8 && b == ACCB_S8 && c == ACCB_S32) {
        if (d.alpha != 1.0f || (d.beta != 0.0f && d.beta != 1.0f) || g.bias) { *err = "integer GEMM supports alpha=1, beta in {0,1}, no bias"; return ACCB_ERR_ARG; }
        e = launch_typed<int8_t, int8_t, int32_t, int>(g, p);
    } else if (a == ACCB_U8 && b == ACCB_U8 && c == ACCB_S32) {
        if (d.alpha != 1.0f || (d.beta != 0.0f && d.beta != 1.0f) || g.bias) { *err = "integer GEMM supports alpha=1, beta in {0,1}, no bias"; return ACCB_ERR_ARG; }
        e = launch_typed<uint8_t, uint8_t, int32_t, int>(g, p);
    } else if (a == ACCB_S16 && b == ACCB_S16 && c == ACCB_S32) {
        // the reference's int16 matmul (accera/python/accera/test/int_matmul_tests.py:40-68): exact int32 accumulation
        if (d.alpha != 1.0f || (d.beta != 0.0f && d.beta != 1.0f) || g.bias) { *err = "integer GEMM supports alpha=1, beta in {0,1}, no bias"; return ACCB_ERR_ARG; }
        e = launch_typed<int16_t, int16_t, int32_t, int>(g, p);
    } else {
        *err = "unsupported GEMM element-type combination";
        return ACCB_ERR_ARG;
    }
    if (e != cudaSuccess) { *err = cudaGetErrorString(e); return ACCB_ERR_CUDA; }
    note_launches(1);
    return 1;
}

}  // namespace accb
