"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU oracle
on identical seeded inputs.

Tolerances (stated by the task for this path):
  * int8 -> int32 GEMM and gather: bit-exact
  * fp32 SIMT GEMM and reduce_mean: rel <= 1e-5
  * fp16 / bf16 / TF32 tensor-core GEMM: rel <= 2e-2
"Rel" for a dot product or a mean is measured against the magnitude the sum was
formed from (|A| @ |B|, mean |x|), which is what bounds the rounding error of any
summation order; for all-positive inputs it coincides with the element-wise
relative error the reference's tests use (verifiers.py:22-38).
"""
import numpy as np
import pytest

import oracle
from accera_b200 import runtime as rt

pytestmark = pytest.mark.gpu

RTOL_F32 = 1e-5
RTOL_TENSOR = 2e-2


def _layout(a, order):
    return np.asfortranarray(a) if order == "F" else np.ascontiguousarray(a)


def _assert_close(got, want, scale, rtol, what=""):
    got64, want64 = np.asarray(got, np.float64), np.asarray(want, np.float64)
    err = np.abs(got64 - want64)
    tol = rtol * np.maximum(np.abs(want64), scale)
    bad = err > tol
    if bad.any():
        idx = np.argwhere(bad)
        first = tuple(idx[0])
        raise AssertionError(
            f"{what}: {bad.sum()} of {bad.size} elements differ (rtol {rtol}); first at {first}: got {got64[first]!r} "
            f"want {want64[first]!r}; max err {err.max():.3e}; rows with errors: {np.unique(idx[:, 0])[:16]}, "
            f"cols: {np.unique(idx[:, -1])[:16]}")


def _gemm_scale(A, B):
    """|A| @ |B| in fp64: the magnitude that bounds the rounding error of the dot products."""
    return np.abs(A.astype(np.float64)) @ np.abs(B.astype(np.float64))


# ---------------------------------------------------------------------------
# fp32 SIMT GEMM (+ReLU): the quickstart case and the layout / ragged matrix
# ---------------------------------------------------------------------------

def test_quickstart_matmul_relu_f32_512():
    A, B, C = oracle.inputs_matmul_relu_f32()
    want = oracle.gemm(A, B, C.copy(), relu=True)
    got = C.copy()
    rt.gemm(A, B, got, relu=True, compute="simt")
    np.testing.assert_allclose(got, want, rtol=RTOL_F32)           # element-wise, as the reference's tests do
    np.testing.assert_allclose(got, np.maximum(A @ B, 0), atol=1e-3)  # README.md:133


@pytest.mark.parametrize("oa,ob,oc", [("C", "C", "C"), ("C", "F", "C"), ("F", "C", "C"), ("F", "F", "F"), ("C", "C", "F")])
def test_simt_f32_layouts_ragged(oa, ob, oc):
    rng = np.random.default_rng(7)
    m, n, k = 123, 234, 345     # the reference's runtime-size test shape (dsl_tests.py:893-1430)
    A = _layout(rng.random((m, k), dtype=np.float32) - 0.5, oa)
    B = _layout(rng.random((k, n), dtype=np.float32) - 0.5, ob)
    C0 = _layout(rng.random((m, n), dtype=np.float32) - 0.5, oc)
    want = oracle.gemm(A, B, C0.copy(order="K"), relu=True)
    got = C0.copy(order="K")
    rt.gemm(A, B, got, relu=True, compute="simt")
    _assert_close(got, want, _gemm_scale(A, B) + np.abs(C0), RTOL_F32, f"simt f32 {oa}{ob}{oc}")


@pytest.mark.parametrize("alpha,beta,relu,use_bias", [(1.0, 0.0, False, False), (5.0, 0.0, False, False),
                                                      (1.0, 0.5, True, False), (2.0, 3.0, False, True),
                                                      (1.0, 1.0, True, True)])
def test_simt_f32_alpha_beta_bias(alpha, beta, relu, use_bias):
    rng = np.random.default_rng(11)
    m, n, k = 96, 160, 72
    A = rng.standard_normal((m, k), dtype=np.float32)
    B = rng.standard_normal((k, n), dtype=np.float32)
    C0 = rng.standard_normal((m, n), dtype=np.float32)
    bias = rng.standard_normal(n, dtype=np.float32) if use_bias else None
    want = oracle.gemm(A, B, C0.copy(), alpha=alpha, beta=beta, bias=bias, relu=relu)
    got = C0.copy()
    rt.gemm(A, B, got, alpha=alpha, beta=beta, bias=bias, relu=relu, compute="simt")
    scale = abs(alpha) * _gemm_scale(A, B) + abs(beta) * np.abs(C0) + (np.abs(bias) if use_bias else 0)
    _assert_close(got, want, scale, RTOL_F32, "simt alpha/beta/bias")


def test_simt_k_zero_and_empty():
    C0 = np.full((8, 8), -2.0, dtype=np.float32)
    got = C0.copy()
    rt.gemm(np.zeros((8, 0), np.float32), np.zeros((0, 8), np.float32), got, relu=True, compute="simt")
    assert (got == 0).all()                    # relu(C + 0)
    rt.gemm(np.zeros((0, 4), np.float32), np.zeros((4, 8), np.float32), np.zeros((0, 8), np.float32))


@pytest.mark.parametrize("kind", ["float16", "bfloat16", "int8", "uint8"])
def test_simt_narrow_inputs(kind):
    rng = np.random.default_rng(13)
    m, n, k = 70, 90, 130
    if kind in ("int8", "uint8"):
        lo, hi = (-128, 128) if kind == "int8" else (0, 256)
        A = rng.integers(lo, hi, size=(m, k)).astype(kind)
        B = np.asfortranarray(rng.integers(lo, hi, size=(k, n)).astype(kind))
        C0 = rng.integers(-1000, 1000, size=(m, n)).astype(np.int32)
        want = oracle.gemm(A, B, C0.copy(), relu=True)
        got = C0.copy()
        rt.gemm(A, B, got, relu=True, compute="simt")
        assert np.array_equal(got, want)
        return
    Af = rng.standard_normal((m, k), dtype=np.float32)
    Bf = rng.standard_normal((k, n), dtype=np.float32)
    if kind == "float16":
        A, B = Af.astype(np.float16), np.asfortranarray(Bf.astype(np.float16))
        A64, B64 = A.astype(np.float64), B.astype(np.float64)
        k_arg = {}
    else:
        A, B = oracle.f32_to_bf16_bits(Af), np.asfortranarray(oracle.f32_to_bf16_bits(Bf))
        A64, B64 = oracle.bf16_bits_to_f32(A).astype(np.float64), oracle.bf16_bits_to_f32(B).astype(np.float64)
        k_arg = {"kind": "bfloat16"}
    C0 = np.zeros((m, n), dtype=np.float32)
    want = oracle.gemm(A, B, C0.copy(), in_kind=kind, relu=True)
    got = C0.copy()
    rt.gemm(A, B, got, relu=True, compute="simt", **k_arg)
    _assert_close(got, want, np.abs(A64) @ np.abs(B64), RTOL_F32, f"simt {kind}")


# ---------------------------------------------------------------------------
# tensor-core (tcgen05) GEMM
# ---------------------------------------------------------------------------

def _tensor_case(kind, out_kind, m, n, k, compute, *, beta=0.0, relu=True, use_bias=False, alpha=1.0, seed=0,
                 a_order="C", b_order="F"):
    """a_order "C" = row-major A (K-contiguous), "F" = column-major A (M-contiguous);
    b_order "F" = column-major B (K-contiguous), "C" = row-major B (N-contiguous)."""
    rng = np.random.default_rng(seed + m * 7 + n * 3 + k)
    _a = (lambda x: np.asfortranarray(x)) if a_order == "F" else (lambda x: np.ascontiguousarray(x))
    _b = (lambda x: np.asfortranarray(x)) if b_order == "F" else (lambda x: np.ascontiguousarray(x))
    if kind in ("int8", "uint8"):
        lo, hi = (-128, 128) if kind == "int8" else (0, 256)
        A = _a(rng.integers(lo, hi, size=(m, k)).astype(kind))
        B = _b(rng.integers(lo, hi, size=(k, n)).astype(kind))
        C0 = rng.integers(-1000, 1000, size=(m, n)).astype(np.int32) if beta else np.zeros((m, n), np.int32)
        want = oracle.gemm(A, B, C0.copy(), beta=beta, relu=relu)
        got = C0.copy()
        rt.gemm(A, B, got, beta=beta, relu=relu, compute=compute)
        if not np.array_equal(got, want):
            bad = np.argwhere(got != want)
            raise AssertionError(f"int8 {compute} {m}x{n}x{k}: {len(bad)} mismatches, first {bad[0]}, got {got[tuple(bad[0])]} "
                                 f"want {want[tuple(bad[0])]}; rows {np.unique(bad[:, 0])[:12]} cols {np.unique(bad[:, 1])[:12]}")
        return
    Af = rng.standard_normal((m, k), dtype=np.float32)
    Bf = rng.standard_normal((k, n), dtype=np.float32) / np.float32(np.sqrt(k))
    kw = {}
    if kind == "float16":
        A, B = _a(Af.astype(np.float16)), _b(Bf.astype(np.float16))
        A64, B64 = A.astype(np.float64), B.astype(np.float64)
    elif kind == "bfloat16":
        A, B = _a(oracle.f32_to_bf16_bits(Af)), _b(oracle.f32_to_bf16_bits(Bf))
        A64, B64 = oracle.bf16_bits_to_f32(A).astype(np.float64), oracle.bf16_bits_to_f32(B).astype(np.float64)
        kw["kind"] = "bfloat16"
    else:   # float32 computed as TF32
        A, B = _a(Af), _b(Bf)
        A64, B64 = A.astype(np.float64), B.astype(np.float64)
    C0f = rng.standard_normal((m, n), dtype=np.float32) if beta else np.zeros((m, n), np.float32)
    if out_kind == "float32":
        C0 = C0f
    elif out_kind == "float16":
        C0 = C0f.astype(np.float16)
    else:
        C0 = oracle.f32_to_bf16_bits(C0f)
        kw["out_kind"] = "bfloat16"
    bias = rng.standard_normal(n, dtype=np.float32) if use_bias else None
    want = oracle.gemm(A, B, C0.copy(), in_kind=kind, out_kind=out_kind, alpha=alpha, beta=beta, bias=bias, relu=relu)
    got = C0.copy()
    rt.gemm(A, B, got, alpha=alpha, beta=beta, bias=bias, relu=relu, compute=compute, **kw)
    if out_kind == "bfloat16":
        got_f, want_f = oracle.bf16_bits_to_f32(got), oracle.bf16_bits_to_f32(want)
    else:
        got_f, want_f = got, want
    scale = abs(alpha) * (np.abs(A64) @ np.abs(B64)) + abs(beta) * np.abs(C0f) + (np.abs(bias) if use_bias else 0)
    # the inputs are exact in fp32, the accumulator is fp32 on both sides: the tensor path is in
    # practice far inside 2e-2; 16-bit outputs add one rounding of the result
    _assert_close(got_f, want_f, scale, RTOL_TENSOR, f"{kind}->{out_kind} {compute} {m}x{n}x{k}")
    tight = 2e-3 if kind == "float32" else (1e-2 if out_kind != "float32" else 1e-4)
    _assert_close(got_f, want_f, scale, tight, f"{kind}->{out_kind} {compute} {m}x{n}x{k} (tight)")


TENSOR_MODES = ["tensor", "tensor_2sm"]


@pytest.mark.parametrize("compute", TENSOR_MODES)
@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (256, 256, 256), (128, 512, 1024), (384, 768, 320), (1024, 1024, 512)])
def test_tensor_bf16_tiles(compute, m, n, k):
    _tensor_case("bfloat16", "float32", m, n, k, compute)


@pytest.mark.parametrize("compute", TENSOR_MODES)
@pytest.mark.parametrize("m,n,k", [(200, 300, 136), (1, 8, 8), (129, 257, 72), (500, 100, 1000)])
def test_tensor_bf16_ragged(compute, m, n, k):
    _tensor_case("bfloat16", "float32", m, n, k, compute, beta=1.0, use_bias=True)


@pytest.mark.parametrize("compute", TENSOR_MODES)
@pytest.mark.parametrize("kind,out_kind", [("float16", "float32"), ("float16", "float16"), ("bfloat16", "bfloat16"),
                                           ("float32", "float32")])
def test_tensor_types(compute, kind, out_kind):
    _tensor_case(kind, out_kind, 256, 512, 384, compute, beta=1.0)
    _tensor_case(kind, out_kind, 300, 264, 200, compute, beta=0.0, relu=False, alpha=0.5)


@pytest.mark.parametrize("compute", TENSOR_MODES)
@pytest.mark.parametrize("kind", ["int8", "uint8"])
def test_tensor_int8_exact(compute, kind):
    _tensor_case(kind, "int32", 256, 512, 512, compute)
    _tensor_case(kind, "int32", 200, 136, 1040, compute, beta=1.0)


def test_tensor_persistent_many_tiles():
    # more tiles than SMs: exercises the persistent loop, both TMEM accumulators and the stage ring wrap-around
    _tensor_case("bfloat16", "bfloat16", 4096, 4096, 256, "tensor", beta=1.0)
    _tensor_case("bfloat16", "bfloat16", 4096, 4096, 256, "tensor_2sm", beta=1.0)


def test_auto_dispatch_falls_back_to_simt_for_unaligned_pitch():
    # a row pitch that is not a multiple of 16 bytes cannot be described to TMA: AUTO must still give the
    # right answer (SIMT kernel), an explicit tensor request must fail loudly
    rng = np.random.default_rng(5)
    A = rng.standard_normal((64, 100), dtype=np.float32).astype(np.float16)        # pitch 200 bytes
    B = np.asfortranarray(rng.standard_normal((100, 96), dtype=np.float32).astype(np.float16))
    C = np.zeros((64, 96), np.float32)
    want = oracle.gemm(A, B, C.copy(), relu=True)
    rt.gemm(A, B, C, relu=True)
    _assert_close(C, want, _gemm_scale(A, B), 1e-4, "auto fallback")
    with pytest.raises(rt.AccbError):
        rt.gemm(A, B, C, relu=True, compute="tensor")


# ---------------------------------------------------------------------------
# reduce_mean
# ---------------------------------------------------------------------------

def _check_reduce(x3, axes, keepdims=1):
    want = oracle.reduce_mean_rank3(x3, axes, keepdims)
    dims, mask = rt.reduce_mean_rank3_dims(*x3.shape, axes, keepdims)
    assert dims == want.shape
    got = np.full(want.shape, np.nan, dtype=np.float32)
    rt.reduce_mean_rank3(x3, got, axes)
    ax = tuple(range(3)) if not axes else tuple(axes)
    scale = np.abs(x3).astype(np.float64).mean(axis=ax, keepdims=bool(keepdims)).reshape(want.shape)
    _assert_close(got, want, scale, RTOL_F32, f"reduce_mean {x3.shape} axes={axes}")
    exact = x3.astype(np.float64).mean(axis=ax, keepdims=bool(keepdims)).reshape(want.shape)
    _assert_close(got, exact, scale, RTOL_F32, f"reduce_mean vs fp64 {x3.shape} axes={axes}")


def test_reduce_mean_last_axis_bench_shape_slice():
    x = oracle.inputs_reduce_mean(1024, 4096)
    _check_reduce(x.reshape(1, 1024, 4096), [2], 0)


@pytest.mark.parametrize("axes", [[0], [1], [2], [0, 1], [0, 2], [1, 2], [0, 1, 2], []])
@pytest.mark.parametrize("shape", [(4, 16, 1000), (3, 5, 7), (17, 33, 257), (2, 128, 4096)])
def test_reduce_mean_all_axes(axes, shape):
    rng = np.random.default_rng(sum(shape))
    x = rng.standard_normal(shape, dtype=np.float32)
    _check_reduce(x, axes, 1)
    _check_reduce(x, axes, 0)


def test_reduce_mean_split_paths():
    rng = np.random.default_rng(3)
    _check_reduce(rng.standard_normal((1, 4, 1 << 20), dtype=np.float32), [2])      # few long rows -> split rows
    _check_reduce(rng.standard_normal((1, 1, (1 << 21) + 3), dtype=np.float32), [0, 1, 2])  # unaligned length
    _check_reduce(rng.standard_normal((8192, 1, 256), dtype=np.float32), [0])       # tall, few columns -> split cols
    _check_reduce(rng.standard_normal((3, 5000, 36), dtype=np.float32), [1])


def test_reduce_mean_positive_elementwise():
    # all-positive input: plain element-wise rtol, the convention of the reference's own tests
    rng = np.random.default_rng(4)
    x = rng.random((2, 300, 4096), dtype=np.float32)
    want = oracle.reduce_mean_rank3(x, [2], 0)
    got = np.empty_like(want)
    rt.reduce_mean_rank3(x, got, [2])
    np.testing.assert_allclose(got, want, rtol=RTOL_F32)


def test_reduce_mean_full_config():
    x = oracle.inputs_reduce_mean()            # [8192, 4096]
    want = oracle.reduce_mean_last_axis(x)
    got = np.empty(8192, np.float32)
    rt.reduce_mean_rank3(x.reshape(1, 8192, 4096), got, [2])
    _assert_close(got, want, np.abs(x).mean(axis=1, dtype=np.float64), RTOL_F32, "reduce_mean [8192,4096]")


# ---------------------------------------------------------------------------
# gather
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("axis", [0, 1])
@pytest.mark.parametrize("dtype", [np.float32, np.float64, np.int8, np.float16])
@pytest.mark.parametrize("d0,d1,i0,i1", [(5, 4, 2, 2), (100, 4096, 37, 3), (1000, 130, 64, 1), (33, 1024, 1, 200)])
def test_gather_bit_exact(axis, dtype, d0, d1, i0, i1):
    rng = np.random.default_rng(d0 + d1 + i0)
    data = (rng.standard_normal((d0, d1)) * 50).astype(dtype)
    idx = rng.integers(0, d0 if axis == 0 else d1, size=(i0, i1), dtype=np.int64)
    want = oracle.gather_rank2(data, idx, axis)
    assert rt.gather_rank2_dims(d0, d1, i0, i1, axis) == want.shape
    got = np.empty(want.shape, dtype=dtype)
    got.view(np.uint8)[...] = 0xAB
    rt.gather_rank2(data, idx, got, axis)
    assert got.tobytes() == want.tobytes()
    assert got.tobytes() == np.take(data, idx, axis).tobytes()


def test_gather_out_of_range_index_is_reported_not_dereferenced():
    data = np.arange(40, dtype=np.float32).reshape(10, 4)
    idx = np.array([[1, 10], [-1, 3]], dtype=np.int64)
    out = np.full((2, 2, 4), 7.0, np.float32)
    with pytest.raises(rt.AccbError) as ei:
        rt.gather_rank2(data, idx, out, 0)
    assert ei.value.code == rt.ERR_INDEX
    assert np.array_equal(out[0, 0], data[1]) and np.array_equal(out[1, 1], data[3])
    assert (out[0, 1] == 0).all() and (out[1, 0] == 0).all()
    # the next call starts clean
    out2 = np.empty((1, 1, 4), np.float32)
    rt.gather_rank2(data, np.array([[2]], dtype=np.int64), out2, 0)
    assert np.array_equal(out2[0, 0], data[2])


def test_gather_full_config():
    T, idx = oracle.inputs_gather()           # T[32000,4096], idx[16384,1]
    got = np.empty((16384, 1, 4096), np.float32)
    rt.gather_rank2(T, idx, got, 0)
    assert np.array_equal(got.reshape(16384, 4096), T[idx[:, 0]])
    rows = np.arange(0, 16384, 257)
    want = oracle.gather_rank2(T, idx[rows], 0)
    assert got[rows].tobytes() == want.tobytes()


# ---------------------------------------------------------------------------
# device pointers (torch tensors on torch's current stream)
# ---------------------------------------------------------------------------

def test_device_pointers_and_stream():
    import torch
    dev = torch.device("cuda:0")
    A, B, C = oracle.inputs_gemm_bf16(512, 512, 512)
    want = oracle.gemm(A, B, C.copy(), in_kind="bfloat16", out_kind="bfloat16", relu=True)
    At = torch.from_numpy(A.view(np.int16)).to(dev).view(torch.bfloat16)
    Bt = torch.from_numpy(np.ascontiguousarray(B.T).view(np.int16)).to(dev).view(torch.bfloat16).t()   # [K,N] column-major view
    Ct = torch.zeros(512, 512, dtype=torch.bfloat16, device=dev)
    s = torch.cuda.Stream(device=dev)
    s.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(s):
        before = rt.launch_count()
        rt.gemm(At, Bt, Ct, relu=True, compute="tensor")
        assert rt.launch_count() == before + 1
        rt.synchronize()
    got = Ct.view(torch.int16).cpu().numpy().view(np.uint16)
    _assert_close(oracle.bf16_bits_to_f32(got), oracle.bf16_bits_to_f32(want),
                  np.abs(oracle.bf16_bits_to_f32(A).astype(np.float64)) @ np.abs(oracle.bf16_bits_to_f32(B).astype(np.float64)),
                  1e-2, "device-pointer bf16 gemm")

    x = torch.randn(1, 256, 4096, device=dev)
    y = torch.empty(256, device=dev)
    rt.reduce_mean_rank3(x, y, [2])
    rt.synchronize()
    want_y = oracle.reduce_mean_rank3(x.cpu().numpy(), [2], 0).reshape(256)
    _assert_close(y.cpu().numpy(), want_y, np.abs(x.cpu().numpy()).mean(axis=2).reshape(256), RTOL_F32, "device reduce")

    T = torch.randn(1000, 512, device=dev)
    idx = torch.randint(0, 1000, (64, 2), device=dev, dtype=torch.int64)
    out = torch.empty(64, 2, 512, device=dev)
    rt.gather_rank2(T, idx, out, 0)
    rt.synchronize()
    assert torch.equal(out, T[idx])


# ---------------------------------------------------------------------------
# full-size configurations: sampled rows against the oracle + whole-matrix properties
# ---------------------------------------------------------------------------

def _freivalds(A64, B64, C64, rng, tol):
    v = rng.standard_normal(C64.shape[1])
    lhs = C64 @ v
    rhs = A64 @ (B64 @ v)
    denom = np.abs(A64) @ (np.abs(B64) @ np.abs(v)) + 1e-30
    assert (np.abs(lhs - rhs) / denom).max() <= tol


def test_gemm_f16_4096_config():
    A, B, C = oracle.inputs_gemm_f16()
    got = C.copy()
    rt.gemm(A, B, got, relu=True, compute="tensor")
    rows = (0, 64)
    want = oracle.gemm(A, B, C.copy(), relu=True, rows=rows)
    scale = np.abs(A[:64].astype(np.float64)) @ np.abs(B.astype(np.float64))
    _assert_close(got[:64], want[:64], scale, 1e-4, "f16 4096^3 rows 0..63")
    for r0 in (1234, 4095 - 7):
        want = oracle.gemm(A, B, C.copy(), relu=True, rows=(r0, r0 + 8))
        sc = np.abs(A[r0:r0 + 8].astype(np.float64)) @ np.abs(B.astype(np.float64))
        _assert_close(got[r0:r0 + 8], want[r0:r0 + 8], sc, 1e-4, f"f16 4096^3 rows {r0}..")
    # whole matrix without ReLU: Freivalds product check in fp64
    got2 = C.copy()
    rt.gemm(A, B, got2, relu=False, compute="tensor_2sm")
    _freivalds(A.astype(np.float64), B.astype(np.float64), got2.astype(np.float64), np.random.default_rng(1), 1e-5)
    # ReLU epilogue == max(plain result, 0), and the CTA-pair kernel agrees with the single-CTA one
    np.testing.assert_allclose(np.maximum(got2, 0), got, rtol=1e-5, atol=1e-4)


def test_gemm_int8_8192_config():
    A, B, C = oracle.inputs_gemm_s8()
    got = C.copy()
    rt.gemm(A, B, got, compute="tensor")
    for r0 in (0, 4000, 8192 - 16):
        want = oracle.gemm(A, B, C.copy(), rows=(r0, r0 + 16))
        assert np.array_equal(got[r0:r0 + 16], want[r0:r0 + 16])
    # exact Freivalds check over the whole matrix in int64
    rng = np.random.default_rng(2)
    v = rng.integers(-8, 8, size=8192).astype(np.int64)
    lhs = got.astype(np.int64) @ v
    rhs = A.astype(np.int64) @ (B.astype(np.int64) @ v)
    assert np.array_equal(lhs, rhs)


# ---------------------------------------------------------------------------
# golden vectors made from the reference's own Python sources (tests/golden/make_golden.py)
# ---------------------------------------------------------------------------

import os as _os

_GOLDEN = _os.path.join(_os.path.dirname(_os.path.abspath(__file__)), "golden")


def test_golden_matmul_relu_quickstart():
    g = np.load(_os.path.join(_GOLDEN, "matmul_relu.npz"))
    for name in ("unit", "signed"):
        A, B, C0, want = g[f"{name}_A"], g[f"{name}_B"], g[f"{name}_C_in"], g[f"{name}_C_out"]
        got = C0.copy()
        rt.gemm(A, B, got, relu=True, compute="simt")
        _assert_close(got, want, _gemm_scale(A, B) + np.abs(C0), RTOL_F32, f"golden matmul_relu {name}")
        assert np.array_equal(got == 0, want == 0) or name == "signed"


def test_golden_reduce_mean_all_axes():
    g = np.load(_os.path.join(_GOLDEN, "reduce_mean.npz"))
    data = g["data"]
    for k in [k for k in g.files if k != "data"]:
        axes, keep = [int(c) for c in k.split("_")[0][4:]], int(k[-1])
        want = g[k]
        dims, _ = rt.reduce_mean_rank3_dims(*data.shape, axes, keep)
        assert dims == want.shape
        got = np.full(want.shape, np.nan, np.float32)
        rt.reduce_mean_rank3(data, got, axes)
        scale = np.abs(data).astype(np.float64).mean(axis=tuple(axes), keepdims=bool(keep)).reshape(want.shape)
        _assert_close(got, want, scale, RTOL_F32, f"golden reduce_mean {k}")


def test_golden_gather():
    g = np.load(_os.path.join(_GOLDEN, "gather.npz"))
    for name in ("verify", "wide", "single"):
        data, idx = g[f"{name}_data"], g[f"{name}_indices"]
        for axis in (0, 1):
            want = g[f"{name}_axis{axis}"]
            got = np.empty_like(want)
            rt.gather_rank2(data, idx, got, axis)
            assert got.tobytes() == want.tobytes(), (name, axis)


def test_large_host_buffers_take_the_pipelined_staging_path():
    # >= 4096 rows and >= 64 MiB of A + C: rows are staged in chunks on two streams; the result must be the
    # same as one launch on device-resident buffers, and right against the oracle on sampled rows
    import torch
    m, n, k = 8192 + 300, 2048, 4096           # ragged last chunk
    A, B, C = oracle.inputs_gemm_bf16(m, n, k, seed=77)
    rng = np.random.default_rng(78)
    C0 = oracle.f32_to_bf16_bits(rng.standard_normal((m, n), dtype=np.float32))
    got = C0.copy()
    rt.set_stream(0)
    rt.gemm(A, B, got, relu=True, kind="bfloat16", out_kind="bfloat16")
    dev = torch.device("cuda:0")
    At = torch.from_numpy(A.view(np.int16)).to(dev).view(torch.bfloat16)
    Bt = torch.from_numpy(np.ascontiguousarray(B.T).view(np.int16)).to(dev).view(torch.bfloat16).t()
    Ct = torch.from_numpy(C0.view(np.int16).copy()).to(dev).view(torch.bfloat16)
    rt.gemm(At, Bt, Ct, relu=True, compute="tensor_2sm")
    rt.synchronize()
    ref_dev = Ct.view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.array_equal(got, ref_dev)
    for r0 in (0, 1020, 1024, 5000, m - 9):       # 1020..1028 straddles the first chunk boundary (1024 rows)
        want = oracle.gemm(A, B, C0.copy(), in_kind="bfloat16", out_kind="bfloat16", relu=True, rows=(r0, r0 + 9))
        a64 = oracle.bf16_bits_to_f32(A[r0:r0 + 9]).astype(np.float64)
        scale = np.abs(a64) @ np.abs(oracle.bf16_bits_to_f32(B).astype(np.float64)) + np.abs(oracle.bf16_bits_to_f32(C0[r0:r0 + 9]))
        _assert_close(oracle.bf16_bits_to_f32(got[r0:r0 + 9]), oracle.bf16_bits_to_f32(want[r0:r0 + 9]), scale, 1e-2,
                      f"pipelined host path rows {r0}")


@pytest.mark.parametrize("m,n,k,lda,ldb", [(123, 236, 344, 344, 236), (130, 70, 345, 348, 72), (1, 4, 1, 4, 4), (700, 900, 130, 132, 900)])
def test_simt_f32_cp_async_path_ragged(m, n, k, lda, ldb):
    # row-major operands with 16-byte aligned row pitches take the multi-stage cp.async kernel;
    # pitches larger than the logical width and K not a multiple of 4 exercise its zero-filled edges
    rng = np.random.default_rng(m + n + k)
    Abig = rng.standard_normal((m, lda), dtype=np.float32)
    Bbig = rng.standard_normal((k, ldb), dtype=np.float32)
    A, B = Abig[:, :k], Bbig[:, :n]
    C0 = rng.standard_normal((m, n), dtype=np.float32)
    bias = rng.standard_normal(n, dtype=np.float32)
    want = oracle.gemm(np.ascontiguousarray(A), np.ascontiguousarray(B), C0.copy(), bias=bias, relu=True)
    got = C0.copy()
    rt.gemm(A, B, got, bias=bias, relu=True, compute="simt")
    _assert_close(got, want, _gemm_scale(A, B) + np.abs(C0) + np.abs(bias), RTOL_F32, f"simt cp.async {m}x{n}x{k}")


@pytest.mark.parametrize("kind,out_kind", [("bfloat16", "bfloat16"), ("float16", "float32"), ("int8", "int32")])
@pytest.mark.parametrize("m,n,k", [(512, 768, 256), (300, 264, 200)])
def test_gemm_replicated_writes_every_replica(kind, out_kind, m, n, k):
    # the multi-destination epilogue, exercised on one GPU: three replicas of C in local memory
    import torch
    if kind == "int8":
        k = (k + 15) // 16 * 16            # the tensor path needs a 16-byte row pitch
    dev = torch.device("cuda:0")
    tmap = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32, "int8": torch.int8, "int32": torch.int32}
    g = torch.Generator(device="cpu").manual_seed(m + n)
    if kind == "int8":
        A = torch.randint(-128, 128, (m, k), generator=g, dtype=torch.int8).to(dev)
        Bt = torch.randint(-128, 128, (n, k), generator=g, dtype=torch.int8).to(dev)
        C0 = torch.randint(-1000, 1000, (m, n), generator=g, dtype=torch.int32).to(dev)
    else:
        A = torch.randn(m, k, generator=g).to(dev).to(tmap[kind])
        Bt = (torch.randn(n, k, generator=g) / k ** 0.5).to(dev).to(tmap[kind])
        C0 = torch.randn(m, n, generator=g).to(dev).to(tmap[out_kind])
    B = Bt.t()
    want = C0.clone()
    rt.gemm(A, B, want, beta=1.0, relu=True, compute="tensor_2sm")
    reps = [C0.clone(), torch.zeros_like(C0), torch.full_like(C0, 3)]
    rt.gemm_replicated(A, B, reps, beta=1.0, relu=True)
    rt.synchronize()
    for r in reps:
        assert torch.equal(r, want)
    # and against the oracle
    a_np, b_np = A.cpu().view(torch.int16 if kind == "bfloat16" else A.dtype).numpy(), Bt.cpu().view(torch.int16 if kind == "bfloat16" else Bt.dtype).numpy().T
    if kind == "bfloat16":
        a_np, b_np = a_np.view(np.uint16), b_np.view(np.uint16)
    c_np = C0.cpu().view(torch.int16 if out_kind == "bfloat16" else C0.dtype).numpy().copy()
    if out_kind == "bfloat16":
        c_np = c_np.view(np.uint16)
    want_o = oracle.gemm(a_np, b_np, c_np, in_kind=kind, out_kind=out_kind, relu=True)
    got_np = reps[1].cpu().view(torch.int16 if out_kind == "bfloat16" else C0.dtype).numpy()
    if kind == "int8":
        assert np.array_equal(got_np, want_o)
    else:
        gf = oracle.bf16_bits_to_f32(got_np.view(np.uint16)) if out_kind == "bfloat16" else got_np
        wf = oracle.bf16_bits_to_f32(want_o) if out_kind == "bfloat16" else want_o
        assert np.abs(gf - wf).max() <= 2e-2 * max(1.0, np.abs(wf).max())


def test_direct_store_epilogue_still_matches():
    # the epilogue without shared-memory staging (column-major or unaligned C), forced on an aligned C
    with rt.options(**{"gemm.staged_store": 0}):
        _tensor_case("bfloat16", "bfloat16", 384, 520, 320, "tensor_2sm", beta=1.0, use_bias=True)
        _tensor_case("float16", "float32", 200, 300, 136, "tensor", beta=1.0)
        _tensor_case("bfloat16", "bfloat16", 4096, 2304, 192, "tensor_2sm", beta=1.0)
    _tensor_case("bfloat16", "bfloat16", 384, 520, 320, "tensor_2sm", beta=1.0, use_bias=True)


@pytest.mark.parametrize("store", [1, 0])
@pytest.mark.parametrize("compute", TENSOR_MODES)
@pytest.mark.parametrize("kind,out_kind", [("bfloat16", "bfloat16"), ("float16", "float32"), ("float16", "float16"),
                                           ("int8", "int32"), ("float32", "float32")])
@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (384, 520, 320), (200, 300, 144), (1, 8, 16), (129, 257, 80)])
def test_both_epilogue_paths_on_ragged_shapes(store, compute, kind, out_kind, m, n, k):
    # staged TMA stores (1, the default for a storable C) and stores straight from registers (0) on the same shapes
    with rt.options(**{"gemm.staged_store": store}):
        _tensor_case(kind, out_kind, m, n, k, compute, beta=1.0, relu=True, use_bias=(kind != "int8"), alpha=1.0 if kind == "int8" else 0.5)


def test_tensor_gemm_random_shapes_fuzz():
    # seeded sweep over ragged shapes, all element types, both CTA modes, beta / bias / relu on and off;
    # every K whose row pitch is 16-byte aligned is legal, including K shorter than one 128-byte slab
    rng = np.random.default_rng(20251)
    kinds = [("bfloat16", "float32", 8), ("bfloat16", "bfloat16", 8), ("float16", "float16", 8), ("float16", "float32", 8),
             ("float32", "float32", 4), ("int8", "int32", 16), ("uint8", "int32", 16)]
    for it in range(48):
        kind, out_kind, kq = kinds[it % len(kinds)]
        m = int(rng.integers(1, 700))
        n = int(rng.integers(1, 900))
        k = int(rng.integers(1, 40)) * kq
        compute = "tensor" if it % 2 else "tensor_2sm"
        beta = float(rng.integers(0, 2))
        _tensor_case(kind, out_kind, m, n, k, compute, beta=beta, relu=bool(rng.integers(0, 2)),
                     use_bias=bool(rng.integers(0, 2)) and kind not in ("int8", "uint8"), seed=it)


@pytest.mark.parametrize("compute", TENSOR_MODES)
@pytest.mark.parametrize("a_order,b_order", [("F", "F"), ("C", "C"), ("F", "C")])
@pytest.mark.parametrize("kind,out_kind", [("bfloat16", "float32"), ("float16", "float16"), ("uint8", "int32"), ("int8", "int32")])
def test_tensor_mn_major_operands(compute, a_order, b_order, kind, out_kind):
    # column-major A and / or row-major B: the M- / N-contiguous operand layouts of the tensor path
    # (the reference tensorizes every FIRST_MAJOR / LAST_MAJOR combination, mfma_tests.py:2797-2894)
    _tensor_case(kind, out_kind, 256, 512, 256, compute, a_order=a_order, b_order=b_order)
    _tensor_case(kind, out_kind, 304, 272, 208, compute, beta=1.0, a_order=a_order, b_order=b_order)


def test_tf32_mn_major_is_refused_by_the_tensor_path_and_served_by_fp32_simt():
    rng = np.random.default_rng(8)
    A = np.asfortranarray(rng.standard_normal((128, 64), dtype=np.float32))
    B = np.asfortranarray(rng.standard_normal((64, 96), dtype=np.float32))
    C = np.zeros((128, 96), np.float32)
    with pytest.raises(rt.AccbError):
        rt.gemm(A, B, C, compute="tensor")
    rt.gemm(A, B, C, compute="tensor_preferred")
    np.testing.assert_allclose(C, A.astype(np.float64) @ B.astype(np.float64), rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("m,n,k", [(512, 512, 512), (256, 384, 1000), (1024, 1024, 1024), (130, 260, 4096), (128, 128, 64),
                                   (2304, 2304, 96)])
def test_simt_f32_8x8_tiles_and_split_k(m, n, k):
    # row-major fp32: 128 x 128 tiles with 8 x 8 register tiles; small problems are split along K and the
    # partial tiles are folded in a fixed order, so two runs give bit-identical results
    rng = np.random.default_rng(m * 3 + n * 5 + k)
    A = rng.standard_normal((m, k), dtype=np.float32)
    B = rng.standard_normal((k, n), dtype=np.float32)
    C0 = rng.standard_normal((m, n), dtype=np.float32)
    bias = rng.standard_normal(n, dtype=np.float32)
    want = oracle.gemm(A, B, C0.copy(), bias=bias, relu=True)
    got1, got2 = C0.copy(), C0.copy()
    rt.gemm(A, B, got1, bias=bias, relu=True, compute="simt")
    rt.gemm(A, B, got2, bias=bias, relu=True, compute="simt")
    _assert_close(got1, want, _gemm_scale(A, B) + np.abs(C0) + np.abs(bias), RTOL_F32, f"simt 8x8 {m}x{n}x{k}")
    assert np.array_equal(got1, got2)


def test_host_c_view_with_padded_rows_keeps_the_gaps():
    # C is a column range of a wider host array and beta = 0: the bytes between C's rows are not part of the
    # result and must come back unchanged
    rng = np.random.default_rng(31)
    m, n, k, ld = 96, 80, 64, 112
    A = rng.standard_normal((m, k), dtype=np.float32)
    B = rng.standard_normal((k, n), dtype=np.float32)
    wide = rng.standard_normal((m, ld), dtype=np.float32)
    before = wide.copy()
    rt.gemm(A, B, wide[:, :n], beta=0.0, compute="simt")
    assert np.array_equal(wide[:, n:], before[:, n:])
    want = oracle.gemm(A, B, np.zeros((m, n), np.float32), beta=0.0)
    _assert_close(wide[:, :n], want, _gemm_scale(A, B), RTOL_F32, "padded C view")


# ---------------------------------------------------------------------------
# tile counts that fill the last round of the persistent grid badly, and both tile widths
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("compute", TENSOR_MODES)
@pytest.mark.parametrize("kind,out_kind", [("bfloat16", "bfloat16"), ("float16", "float32"), ("int8", "int32"), ("float32", "float32")])
@pytest.mark.parametrize("m,n,k", [(1024, 1024, 2048),      # 16 pair tiles on 74 pairs
                                   (2000, 1500, 1552),      # ragged everywhere
                                   (768, 512, 4112),        # 6 tiles, K tail of 16
                                   (4096, 5120, 1024)])     # 320 pair tiles = 4 rounds + 24
def test_tensor_awkward_tile_counts(compute, kind, out_kind, m, n, k):
    _tensor_case(kind, out_kind, m, n, k, compute, beta=1.0, relu=True, use_bias=(kind != "int8"), alpha=1.0 if kind == "int8" else 0.5)


def test_tile_width_does_not_change_the_result():
    # 128- and 256-column tiles accumulate every output element over K in the same order: identical bits
    import torch
    dev = torch.device("cuda:0")
    torch.manual_seed(9)
    m, n, k = 1536, 1100, 2048
    A8 = torch.randint(-128, 128, (m, k), device=dev, dtype=torch.int8)
    B8 = torch.randint(-128, 128, (n, k), device=dev, dtype=torch.int8).t()
    A = torch.randn(m, k, device=dev).to(torch.bfloat16)
    B = (torch.randn(n, k, device=dev) / k ** 0.5).to(torch.bfloat16).t()
    for a, b, cdt in ((A8, B8, torch.int32), (A, B, torch.float32), (A, B, torch.bfloat16)):
        for compute in TENSOR_MODES:
            outs = []
            for cols in (256, 128):
                with rt.options(**{"gemm.tile_cols": cols}):
                    C = torch.zeros(m, n, device=dev, dtype=cdt)
                    rt.gemm(a, b, C, beta=0.0, compute=compute)
                    rt.synchronize()
                outs.append(C.clone())
            assert torch.equal(outs[0], outs[1]), (cdt, compute)


def test_concurrent_threads_and_streams():
    """Four host threads, each with its own stream and its own operands, issue tensor-core GEMMs, reductions and
    gathers through the C ABI at the same time (the stream and the last error are per thread; pacing counters,
    the reduction's scratch buffer and launch set-up are shared per device, the scratch buffer ordered between
    streams by an event)."""
    import threading
    import torch
    dev = torch.device("cuda:0")
    torch.manual_seed(4)
    m, n, k = 1024, 768, 512
    jobs = []
    for t in range(4):
        A = torch.randn(m, k, device=dev).to(torch.bfloat16)
        B = (torch.randn(n, k, device=dev) / k ** 0.5).to(torch.bfloat16).t()
        x = torch.randn(1, 8, 262144, device=dev) + t       # 8 outputs of 262144 elements: the split path with scratch
        table = torch.randn(500, 1024, device=dev)
        idx = torch.randint(0, 500, (64, 2), device=dev)
        jobs.append((A, B, x, table, idx))
    torch.cuda.synchronize()
    results, errors = [None] * 4, []

    def work(t):
        try:
            A, B, x, table, idx = jobs[t]
            stream = torch.cuda.Stream(device=dev)
            with torch.cuda.stream(stream):
                outs = []
                for rep in range(8):
                    C = torch.zeros(m, n, device=dev, dtype=torch.float32)
                    rt.gemm(A, B, C, beta=0.0, relu=True, compute="tensor_2sm" if rep % 2 else "tensor")
                    red = torch.empty(1, 8, device=dev)
                    rt.reduce_mean_rank3(x, red, [2])
                    g = torch.empty(64, 2, 1024, device=dev)
                    rt.gather_rank2(table, idx, g, 0)
                    outs.append((C, red, g))
                stream.synchronize()
                rt.synchronize()
            results[t] = outs
        except Exception as e:          # noqa: BLE001 - reported below, in the main thread
            errors.append((t, repr(e)))

    threads = [threading.Thread(target=work, args=(t,)) for t in range(4)]
    for th in threads:
        th.start()
    for th in threads:
        th.join()
    assert not errors, errors
    for t in range(4):
        A, B, x, table, idx = jobs[t]
        want_c = torch.relu(A.float() @ B.float())
        want_r = x.mean(dim=2)
        want_g = table[idx]
        for C, red, g in results[t]:
            assert (C - want_c).abs().max().item() <= 2e-2 * want_c.abs().max().item()
            assert torch.allclose(red, want_r, rtol=1e-5, atol=1e-5)
            assert torch.equal(g, want_g)


def test_tutorial_known_answers():
    """What the reference's compiled packages print in its tutorials (see tests/test_oracle_golden.py).  The fp32
    kernels that do not split K start their accumulators from C and add the products in k order, as the reference's
    nest does, and print the same digits; the cluster split-K kernel (chosen for 1024 x 512 x 256) adds C to the
    folded partial sums and is one ulp away."""
    from test_oracle_golden import TUTORIAL_OUTPUTS, tutorial_inputs
    for m, n, k, printed in TUTORIAL_OUTPUTS:
        A, B, C = tutorial_inputs(m, n, k)
        want = oracle.gemm(A, B, C.copy(), beta=1.0)
        got = C.copy()
        rt.gemm(A, B, got, beta=1.0, compute="simt")
        np.testing.assert_allclose(got, want, rtol=RTOL_F32)
        values = {"%f" % v for v in got.ravel()}
        if k == 128:
            assert values == {printed}
        else:
            assert values <= {printed, "1536.420044"}
    # the same sizes with column-major B take the generic kernel: accumulators from C there too
    A, B, C = tutorial_inputs(784, 512, 128)
    got = C.copy()
    rt.gemm(A, np.asfortranarray(B), got, beta=1.0, compute="simt")
    assert {"%f" % v for v in got.ravel()} == {"768.419983"}
    A, B, C = tutorial_inputs(1024, 512, 256)
    got = C.copy()
    rt.gemm(A, np.asfortranarray(B), got, beta=1.0, compute="simt")
    assert {"%f" % v for v in got.ravel()} == {"1536.419922"}
