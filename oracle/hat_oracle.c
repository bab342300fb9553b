/*
 * CPU oracle for the HAT GEMM(+ReLU) / reduce_mean / gather / range path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is a plain-C restatement of the loop
 * nests the reference (microsoft/Accera) compiles for its HOST target.  It is
 * the checker the GPU kernels are compared with and the timed CPU baseline; the
 * product never links, loads or calls it.
 *
 * Reference files each function follows (paths inside the reference project):
 *   matmul nest          README.md:61-65  (C[i,j] += A[i,k] * B[k,j], C is INPUT_OUTPUT)
 *   relu nest + fuse     README.md:67-76, accera/python/accera/lang/Schedule.py:522-628
 *                        (for every (i,j): all k of the matmul, then the relu)
 *   float max            accera/transforms/src/value/ValueToStandardLoweringPass.cpp:1117-1118
 *   strides from layout  accera/python/accera/lang/Layout.py:35-55
 *   int widening         accera/python/accera/test/int_matmul_tests.py:55
 *   alpha/beta recipe    docs/Tutorials/GPU/Tensor_MatMul_ElementWiseOps_GPU.md:88-99
 *   fragment ops         accera/acc-translate/src/Target/Cpp/CppPrinterUtils.h:630-655
 *   reduce_mean nests    kernels/reduce_mean/naive_runtime_sized.py:66-148
 *   gather nests         kernels/gather/naive_runtime_sized.py:26-49,
 *                        accera/python/accera/test/dsl_tests.py:1596-1601, 1642-1647
 *   range nests          accera/python/accera/test/dsl_tests.py:1450-1462,
 *                        kernels/range/naive_runtime_sized.py:21-28
 *
 * Pinning: the reference stores no golden vectors for this path.  The gather
 * functions are pinned against vectors produced by the reference's own numpy
 * loop restatement (kernels/gather/naive_runtime_sized.py:72-103) and the
 * reduce_mean / matmul+relu functions against vectors produced by executing the
 * reference's nest definitions under a small loop-nest interpreter; both sets
 * live in tests/golden/ with the script that made them; range is pinned against
 * the reference's own numpy loop (kernels/range/naive_runtime_sized.py:44-56) the
 * same way.  The compiled HOST package itself could not be built (needs a patched
 * LLVM 15).  The only outputs of compiled reference packages in its tree are the
 * two values its matmul tutorials print (docs/Tutorials/Optimized_MatMul.md:277-280
 * and docs/Tutorials/GPU/Hello_MatMul_GPU.md:277-281); orc_gemm_float reproduces
 * both digit for digit, and the second one (1536.419922) fixes the accumulation
 * order restated here (start from C, add the products in k order).  Beyond those
 * two values parity with the *compiled* reference remains unpinned.
 *
 * Build: see oracle/Makefile.  The strict library is compiled without FMA
 * contraction so every fp32 sum is a sequence of separately rounded mul and add
 * in index order; the "fast" library is the same source with -ffast-math, which
 * mirrors the reference's default fast-math flags
 * (accera/value/src/MLIREmitterContext.cpp:1219-1227) and is what gets timed.
 */
#include <stdint.h>
#include <stddef.h>
#include <string.h>
#include <math.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* element kinds shared with the Python wrapper */
enum { ORC_F32 = 0, ORC_F16 = 1, ORC_BF16 = 2, ORC_S8 = 3, ORC_S32 = 4, ORC_U8 = 5, ORC_S16 = 6 };

/* epilogue flags */
enum { ORC_EPI_NONE = 0, ORC_EPI_RELU = 1 };

/* ---- half / bfloat16 conversions (bit-exact, round-to-nearest-even) ---- */

static inline float bf16_to_f32(uint16_t h)
{
    uint32_t u = ((uint32_t)h) << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

static inline uint16_t f32_to_bf16(float f)
{
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u); /* quiet NaN */
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    return (uint16_t)(u >> 16);
}

static inline float f16_to_f32(uint16_t h)
{
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    uint32_t u;
    if (exp == 0) {
        if (man == 0) {
            u = sign;
        } else { /* subnormal: normalise */
            int e = -1;
            do { man <<= 1; ++e; } while (!(man & 0x400u));
            man &= 0x3ffu;
            u = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        u = sign | 0x7f800000u | (man << 13);
    } else {
        u = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &u, 4);
    return f;
}

static inline uint16_t f32_to_f16(float f)
{
    uint32_t u;
    memcpy(&u, &f, 4);
    uint32_t sign = (u >> 16) & 0x8000u;
    uint32_t a = u & 0x7fffffffu;
    if (a > 0x7f800000u) return (uint16_t)(sign | 0x7e00u);          /* NaN */
    if (a >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);         /* overflow -> inf (65520 rounds up) */
    if (a < 0x33000001u) return (uint16_t)sign;                      /* underflow to zero (<= 2^-25) */
    int32_t e = (int32_t)(a >> 23) - 127;
    uint32_t m = (a & 0x7fffffu) | 0x800000u;
    uint32_t shift, half;
    if (e < -14) { /* subnormal half */
        shift = (uint32_t)(13 + (-14 - e));
        uint32_t q = m >> shift;
        uint32_t rem = m & ((1u << shift) - 1u);
        half = 1u << (shift - 1);
        if (rem > half || (rem == half && (q & 1u))) ++q;
        return (uint16_t)(sign | q);
    }
    shift = 13;
    uint32_t q = ((uint32_t)(e + 15) << 10) | ((m >> shift) & 0x3ffu);
    uint32_t rem = m & 0x1fffu;
    half = 0x1000u;
    if (rem > half || (rem == half && (q & 1u))) ++q; /* carry into exponent is correct */
    return (uint16_t)(sign | q);
}

static inline float load_as_f32(const void* p, int kind, int64_t off)
{
    switch (kind) {
    case ORC_F32: return ((const float*)p)[off];
    case ORC_F16: return f16_to_f32(((const uint16_t*)p)[off]);
    case ORC_BF16: return bf16_to_f32(((const uint16_t*)p)[off]);
    default: return 0.0f;
    }
}

static inline void store_from_f32(void* p, int kind, int64_t off, float v)
{
    switch (kind) {
    case ORC_F32: ((float*)p)[off] = v; break;
    case ORC_F16: ((uint16_t*)p)[off] = f32_to_f16(v); break;
    case ORC_BF16: ((uint16_t*)p)[off] = f32_to_bf16(v); break;
    default: break;
    }
}

/*
 * Floating-point GEMM with the fused epilogue.
 *
 *   for i, j:  acc = C[i,j]                       (beta == 1, the reference's "C +=")
 *              for k in order: acc += A[i,k]*B[k,j]   (fp32, separately rounded)
 *              C[i,j] = epilogue(acc)
 *
 * With alpha != 1 or beta != 1 the result is alpha*(sum) + beta*C as in the
 * reference's GEMM recipe table; bias (optional, length N, fp32) is added before
 * the ReLU.  Inputs of kind f16/bf16 are widened exactly; the accumulator is
 * fp32; the output is rounded once to c_kind.  Strides are in elements.
 * Rows [m_begin, m_end) only, so large cases can be sampled.
 */
void orc_gemm_float(const void* A, const void* B, void* C,
                    int a_kind, int b_kind, int c_kind,
                    int64_t M, int64_t N, int64_t K,
                    int64_t sa0, int64_t sa1, int64_t sb0, int64_t sb1, int64_t sc0, int64_t sc1,
                    float alpha, float beta, const float* bias, int epilogue,
                    int64_t m_begin, int64_t m_end)
{
    (void)M;
#pragma omp parallel for schedule(static)
    for (int64_t i = m_begin; i < m_end; ++i) {
        for (int64_t j = 0; j < N; ++j) {
            float c0 = load_as_f32(C, c_kind, i * sc0 + j * sc1);
            float acc = (alpha == 1.0f) ? (beta == 1.0f ? c0 : beta * c0) : 0.0f;
            if (a_kind == ORC_F32 && b_kind == ORC_F32) {
                const float* a = (const float*)A + i * sa0;
                const float* b = (const float*)B + j * sb1;
                if (sa1 == 1 && sb0 == 1) { /* both operands K-contiguous: same order, unit stride */
                    for (int64_t k = 0; k < K; ++k) acc += a[k] * b[k];
                } else {
                    for (int64_t k = 0; k < K; ++k) acc += a[k * sa1] * b[k * sb0];
                }
            } else {
                for (int64_t k = 0; k < K; ++k)
                    acc += load_as_f32(A, a_kind, i * sa0 + k * sa1) * load_as_f32(B, b_kind, k * sb0 + j * sb1);
            }
            if (alpha != 1.0f) acc = alpha * acc + beta * c0;
            if (bias) acc += bias[j];
            if (epilogue == ORC_EPI_RELU) acc = fmaxf(acc, 0.0f);
            store_from_f32(C, c_kind, i * sc0 + j * sc1, acc);
        }
    }
}

/*
 * Integer GEMM: int8 (or uint8) inputs widened to int32 before the multiply,
 * int32 accumulate starting from C, optional ReLU (max with 0).  Exact.
 */
void orc_gemm_int8(const void* A, const void* B, int32_t* C,
                   int a_kind, int b_kind,
                   int64_t M, int64_t N, int64_t K,
                   int64_t sa0, int64_t sa1, int64_t sb0, int64_t sb1, int64_t sc0, int64_t sc1,
                   int beta_is_zero, int epilogue, int64_t m_begin, int64_t m_end)
{
    (void)M;
#pragma omp parallel for schedule(static)
    for (int64_t i = m_begin; i < m_end; ++i) {
        for (int64_t j = 0; j < N; ++j) {
            int32_t acc = beta_is_zero ? 0 : C[i * sc0 + j * sc1];
            if (a_kind == ORC_S8 && b_kind == ORC_S8 && sa1 == 1 && sb0 == 1) {
                const int8_t* a = (const int8_t*)A + i * sa0;
                const int8_t* b = (const int8_t*)B + j * sb1;
                for (int64_t k = 0; k < K; ++k) acc += (int32_t)a[k] * (int32_t)b[k];
            } else
            for (int64_t k = 0; k < K; ++k) {
                /* int16 operands: cast(a, int32) * cast(b, int32), accera/python/accera/test/int_matmul_tests.py:55 */
                int32_t a = (a_kind == ORC_S16) ? (int32_t)((const int16_t*)A)[i * sa0 + k * sa1]
                          : (a_kind == ORC_U8) ? (int32_t)((const uint8_t*)A)[i * sa0 + k * sa1]
                                               : (int32_t)((const int8_t*)A)[i * sa0 + k * sa1];
                int32_t b = (b_kind == ORC_S16) ? (int32_t)((const int16_t*)B)[k * sb0 + j * sb1]
                          : (b_kind == ORC_U8) ? (int32_t)((const uint8_t*)B)[k * sb0 + j * sb1]
                                               : (int32_t)((const int8_t*)B)[k * sb0 + j * sb1];
                acc += a * b;
            }
            if (epilogue == ORC_EPI_RELU && acc < 0) acc = 0;
            C[i * sc0 + j * sc1] = acc;
        }
    }
}

/*
 * ReduceMean over a rank-3 fp32 array (dense first-major), ONNX axes/keepdims.
 * axes_mask bit d set = dimension d is reduced.  For every output element:
 * zero-init, add the reduced elements in index order (remaining reduced
 * dimensions iterate innermost, in their original order), divide by the number
 * of reduced elements cast to fp32.  The output is dense first-major over the
 * kept dimensions (keepdims only changes its shape, not its element order).
 */
void orc_reduce_mean_rank3(const float* data, int64_t d0, int64_t d1, int64_t d2,
                           float* reduced, int axes_mask)
{
    const int64_t dims[3] = { d0, d1, d2 };
    const int64_t strides[3] = { d1 * d2, d2, 1 };
    int64_t kd[3], ks[3], rd[3], rs[3];
    int nk = 0, nr = 0;
    for (int d = 0; d < 3; ++d) {
        if (axes_mask & (1 << d)) { rd[nr] = dims[d]; rs[nr] = strides[d]; ++nr; }
        else { kd[nk] = dims[d]; ks[nk] = strides[d]; ++nk; }
    }
    for (int d = nk; d < 3; ++d) { kd[d] = 1; ks[d] = 0; }
    for (int d = nr; d < 3; ++d) { rd[d] = 1; rs[d] = 0; }
    const int64_t count = rd[0] * rd[1] * rd[2];
    const int64_t n_out = kd[0] * kd[1] * kd[2];
#pragma omp parallel for schedule(static)
    for (int64_t o = 0; o < n_out; ++o) {
        int64_t o2 = o % kd[2], o1 = (o / kd[2]) % kd[1], o0 = o / (kd[2] * kd[1]);
        const float* base = data + o0 * ks[0] + o1 * ks[1] + o2 * ks[2];
        float acc = 0.0f;
        for (int64_t r0 = 0; r0 < rd[0]; ++r0)
            for (int64_t r1 = 0; r1 < rd[1]; ++r1)
                for (int64_t r2 = 0; r2 < rd[2]; ++r2)
                    acc += base[r0 * rs[0] + r1 * rs[1] + r2 * rs[2]];
        reduced[o] = acc / (float)count;
    }
}

/* Output dimensions of the rank-3 ReduceMean.  Returns the output rank. */
int orc_reduce_mean_rank3_dims(int64_t d0, int64_t d1, int64_t d2, int axes_mask, int keepdims, int64_t* out_dims)
{
    const int64_t dims[3] = { d0, d1, d2 };
    int n = 0;
    for (int d = 0; d < 3; ++d) {
        if (axes_mask & (1 << d)) { if (keepdims) out_dims[n++] = 1; }
        else out_dims[n++] = dims[d];
    }
    if (n == 0) out_dims[n++] = 1;
    return n;
}

/*
 * Gather, rank-2 data and rank-2 int64 indices, dense first-major.
 *   axis 0: Output[i,j,k] = Data[Indices[i,j], k]   shape (I0, I1, D1)
 *   axis 1: Output[i,j,k] = Data[i, Indices[j,k]]   shape (D0, I0, I1)
 * Negative indices are not supported and there is no bounds check, exactly as
 * in the reference.  elem_bytes-wide elements are copied bit for bit.
 */
void orc_gather_rank2(const void* data, int64_t d0, int64_t d1,
                      const int64_t* indices, int64_t i0, int64_t i1,
                      void* output, int axis, int64_t elem_bytes)
{
    const char* src = (const char*)data;
    char* dst = (char*)output;
    if (axis == 0) {
#pragma omp parallel for schedule(static)
        for (int64_t ij = 0; ij < i0 * i1; ++ij) {
            int64_t row = indices[ij];
            memcpy(dst + ij * d1 * elem_bytes, src + row * d1 * elem_bytes, (size_t)(d1 * elem_bytes));
        }
    } else {
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < d0; ++i)
            for (int64_t jk = 0; jk < i0 * i1; ++jk)
                memcpy(dst + (i * i0 * i1 + jk) * elem_bytes, src + (i * d1 + indices[jk]) * elem_bytes, (size_t)elem_bytes);
    }
}

void orc_gather_rank2_dims(int64_t d0, int64_t d1, int64_t i0, int64_t i1, int axis, int64_t* out_dims)
{
    if (axis == 0) { out_dims[0] = i0; out_dims[1] = i1; out_dims[2] = d1; }
    else { out_dims[0] = d0; out_dims[1] = i0; out_dims[2] = i1; }
}

/*
 * Range (the ONNX operator as the reference writes it).
 *   size:   floor((limit - start) / delta) in fp32, cast to int64
 *           (accera/python/accera/test/dsl_tests.py:1452-1454; kernels/range/naive_runtime_sized.py:21)
 *   result: for i in [0, n): output[i] = start; start = start + delta      - one fp32 addition per element,
 *           each rounded, in index order; the scalar is an in/out argument and ends as the value after n additions
 *           (dsl_tests.py:1459-1462, 1490-1491; kernels/range/naive_runtime_sized.py:25-28, 52-54)
 * A quotient that is negative, not finite or not representable gives size 0 (the reference leaves those undefined).
 * The volatile keeps the additions separately rounded under any optimisation flags.
 */
int64_t orc_range_count_f32(float start, float limit, float delta)
{
    volatile float span = limit - start;
    volatile float q = span / delta;
    float f = floorf(q);
    if (!(f >= 0.0f) || f >= 9.2e18f) return 0;
    return (int64_t)f;
}

void orc_range_f32(int64_t n, float* output, float* start_inout, float delta)
{
    volatile float x = *start_inout;
    for (int64_t i = 0; i < n; ++i) {
        output[i] = x;
        x = x + delta;
    }
    *start_inout = x;
}

/* conversions exported for the tests */
void orc_f32_to_bf16(const float* src, uint16_t* dst, int64_t n) { for (int64_t i = 0; i < n; ++i) dst[i] = f32_to_bf16(src[i]); }
void orc_bf16_to_f32(const uint16_t* src, float* dst, int64_t n) { for (int64_t i = 0; i < n; ++i) dst[i] = bf16_to_f32(src[i]); }
void orc_f32_to_f16(const float* src, uint16_t* dst, int64_t n) { for (int64_t i = 0; i < n; ++i) dst[i] = f32_to_f16(src[i]); }
void orc_f16_to_f32(const uint16_t* src, float* dst, int64_t n) { for (int64_t i = 0; i < n; ++i) dst[i] = f16_to_f32(src[i]); }

int orc_max_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void orc_set_threads(int n)
{
#ifdef _OPENMP
    omp_set_num_threads(n);
#else
    (void)n;
#endif
}
