"""The CPU oracle against the golden vectors produced from the reference's own Python sources
(tests/golden/make_golden.py), and against numpy on the seeded benchmark inputs.  CPU only."""
import os

import numpy as np
import pytest

import oracle

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _axes_of(key):
    return [int(c) for c in key.split("_")[0][4:]], int(key[-1])


def test_matmul_relu_quickstart_bit_exact():
    g = np.load(os.path.join(GOLDEN, "matmul_relu.npz"))
    for name in ("unit", "signed"):
        got = oracle.gemm(g[f"{name}_A"], g[f"{name}_B"], g[f"{name}_C_in"].copy(), relu=True)
        assert np.array_equal(got, g[f"{name}_C_out"]), name
    assert (g["signed_C_out"] == 0).mean() > 0.2           # the ReLU actually clips in the signed case


def test_reduce_mean_all_axes_bit_exact():
    g = np.load(os.path.join(GOLDEN, "reduce_mean.npz"))
    keys = [k for k in g.files if k != "data"]
    assert len(keys) == 14
    for k in keys:
        axes, keep = _axes_of(k)
        got = oracle.reduce_mean_rank3(g["data"], axes, keep)
        assert got.shape == g[k].shape and np.array_equal(got, g[k]), k


def test_gather_bit_exact_and_matches_np_take():
    g = np.load(os.path.join(GOLDEN, "gather.npz"))
    for name in ("verify", "wide", "single"):
        data, idx = g[f"{name}_data"], g[f"{name}_indices"]
        for axis in (0, 1):
            want = g[f"{name}_axis{axis}"]
            if axis == 1 and idx.max() >= data.shape[1]:
                continue
            got = oracle.gather_rank2(data, idx, axis)
            assert got.tobytes() == want.tobytes()
            assert np.array_equal(want, np.take(data, idx, axis))      # the reference's own check (verify())


def test_fast_build_agrees_with_strict_within_tolerance():
    A, B, C = oracle.inputs_matmul_relu_f32(96, 80, 200)
    s = oracle.gemm(A, B, C.copy(), relu=True)
    f = oracle.gemm(A, B, C.copy(), relu=True, fast=True)
    np.testing.assert_allclose(f, s, rtol=1e-5)
    x = oracle.inputs_reduce_mean(64, 4096)
    np.testing.assert_allclose(oracle.reduce_mean_last_axis(x, fast=True), oracle.reduce_mean_last_axis(x),
                               atol=1e-5 * np.abs(x).mean())


def test_mixed_precision_and_int8_against_numpy():
    A, B, C = oracle.inputs_gemm_s8(48, 40, 300)
    assert np.array_equal(oracle.gemm(A, B, C.copy()), A.astype(np.int64) @ B.astype(np.int64))
    A, B, C = oracle.inputs_gemm_f16(40, 56, 128)
    ref = np.maximum(A.astype(np.float64) @ B.astype(np.float64), 0)
    np.testing.assert_allclose(oracle.gemm(A, B, C.copy(), relu=True), ref, atol=1e-4)
    A, B, C = oracle.inputs_gemm_bf16(64, 32, 256)
    ref = np.maximum(oracle.bf16_bits_to_f32(A).astype(np.float64) @ oracle.bf16_bits_to_f32(B).astype(np.float64), 0)
    got = oracle.bf16_bits_to_f32(oracle.gemm(A, B, C.copy(), in_kind="bfloat16", out_kind="bfloat16", relu=True))
    np.testing.assert_allclose(got, ref, rtol=2 ** -8, atol=1e-6)
    assert B.strides == (2, 2 * 256)                      # column-major view, as the benchmark feeds it


def test_bf16_and_f16_conversions_round_to_nearest_even():
    x = np.array([1.0, 1.00390625, 1.005859375, -2.5, 3.0e38, 1e-40, 65504.0, 65520.0], dtype=np.float32)
    b = oracle.f32_to_bf16_bits(x)
    assert b[0] == 0x3F80 and b[1] == 0x3F80 and b[2] == 0x3F81     # tie to even, then above the tie
    h = np.empty(x.size, np.uint16)
    oracle.lib().orc_f32_to_f16(x.ctypes.data, h.ctypes.data, x.size)
    with np.errstate(over="ignore"):
        assert np.array_equal(h, x.astype(np.float16).view(np.uint16))


def test_alpha_beta_bias_semantics():
    rng = np.random.default_rng(1)
    A = rng.standard_normal((8, 16), dtype=np.float32); B = rng.standard_normal((16, 12), dtype=np.float32)
    C = rng.standard_normal((8, 12), dtype=np.float32); bias = rng.standard_normal(12, dtype=np.float32)
    got = oracle.gemm(A, B, C.copy(), alpha=2.0, beta=0.5, bias=bias, relu=True)
    ref = np.maximum(2.0 * (A.astype(np.float64) @ B) + 0.5 * C + bias, 0)
    np.testing.assert_allclose(got, ref, rtol=1e-5, atol=1e-5)
    rows = oracle.gemm(A, B, C.copy(), rows=(2, 5))
    assert np.array_equal(rows[:2], C[:2]) and np.array_equal(rows[5:], C[5:]) and not np.array_equal(rows[2:5], C[2:5])


# The only outputs of the reference's COMPILED packages that its tree holds: what its two matmul tutorials print.
# A = 2, B = 3, C = 0.42 everywhere, C += A @ B in fp32.
#   docs/Tutorials/Optimized_MatMul.md:277-280        HOST package, M=784 K=128 N=512:  768.419983
#   docs/Tutorials/GPU/Hello_MatMul_GPU.md:277-281    GPU package,  M=1024 K=256 N=512: 1536.419922
# The second value tells the accumulation order apart: adding the 256 products of 6 to 0.42 one by one gives
# 1536.419922, summing the products first and adding 0.42 last gives 1536.420044.
TUTORIAL_OUTPUTS = [(784, 512, 128, "768.419983"), (1024, 512, 256, "1536.419922")]


def tutorial_inputs(m, n, k):
    return (np.full((m, k), 2.0, np.float32), np.full((k, n), 3.0, np.float32), np.full((m, n), 0.42, np.float32))


@pytest.mark.parametrize("m,n,k,printed", TUTORIAL_OUTPUTS)
def test_oracle_reproduces_what_the_compiled_reference_prints(m, n, k, printed):
    A, B, C = tutorial_inputs(m, n, k)
    got = oracle.gemm(A, B, C, beta=1.0)
    assert {"%f" % v for v in got.ravel()} == {printed}
    if k == 256:
        # the other order, for the record: it is NOT what the reference printed
        assert "%f" % np.float32(np.float32(6.0 * k) + np.float32(0.42)) == "1536.420044"
