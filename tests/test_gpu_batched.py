"""GPU parity tests of the batched GEMM (accb_gemm_batched): every problem of the batch against the CPU
oracle's GEMM on the same seeded inputs, through the C ABI (host buffers, device buffers) and through a HAT
package built from the reference's batch matmul nest (mfma_tests.py:435-466).

Tolerances as for the single GEMM: bit-exact for int8 -> int32, rel <= 1e-5 for the fp32 SIMT path,
rel <= 2e-2 for the fp16 / bf16 tensor-core path (measured against |A| @ |B|).
"""
import numpy as np
import pytest

import accera_b200 as acc
import oracle
from accera_b200 import hat, runtime as rt

pytestmark = pytest.mark.gpu


def _close(got, want, scale, rtol, what):
    err = np.abs(np.asarray(got, np.float64) - np.asarray(want, np.float64))
    tol = rtol * np.maximum(np.abs(np.asarray(want, np.float64)), scale)
    assert not (err > tol).any(), f"{what}: {(err > tol).sum()} elements differ, max err {err.max():.3e}, first {np.argwhere(err > tol)[0]}"


def _operands(kind, batch, m, n, k, rng, b_kmajor, share_b=False):
    """-> A [batch,m,k], B [batch,k,n] (memory [batch,n,k] when b_kmajor), fp64 copies of both."""
    nb = 1 if share_b else batch
    if kind in ("int8", "uint8"):
        lo, hi = (-128, 128) if kind == "int8" else (0, 256)
        A = rng.integers(lo, hi, size=(batch, m, k)).astype(kind)
        Bm = rng.integers(lo, hi, size=(nb, n, k) if b_kmajor else (nb, k, n)).astype(kind)
    else:
        A = rng.standard_normal((batch, m, k), dtype=np.float32)
        Bm = rng.standard_normal((nb, n, k) if b_kmajor else (nb, k, n), dtype=np.float32) / np.float32(np.sqrt(k))
        if kind == "float16":
            A, Bm = A.astype(np.float16), Bm.astype(np.float16)
        elif kind == "bfloat16":
            A, Bm = oracle.f32_to_bf16_bits(A), oracle.f32_to_bf16_bits(Bm)
    B = Bm.transpose(0, 2, 1) if b_kmajor else Bm
    if share_b:
        B = np.broadcast_to(B, (batch,) + B.shape[1:])      # batch stride 0
    return A, B


def _as64(x, kind):
    return (oracle.bf16_bits_to_f32(x) if kind == "bfloat16" else x).astype(np.float64)


def _run_case(kind, out_kind, batch, m, n, k, compute, *, beta=1.0, relu=False, alpha=1.0, b_kmajor=True, share_b=False,
              use_bias=False, rtol=2e-2, seed=0):
    rng = np.random.default_rng(seed + 1000 * batch + m * 7 + n * 3 + k)
    A, B = _operands(kind, batch, m, n, k, rng, b_kmajor, share_b)
    kw = {}
    if kind == "bfloat16":
        kw["kind"] = "bfloat16"
    if out_kind == "int32":
        C0 = rng.integers(-1000, 1000, size=(batch, m, n)).astype(np.int32)
    else:
        C0f = rng.standard_normal((batch, m, n), dtype=np.float32)
        C0 = {"float32": C0f, "float16": C0f.astype(np.float16)}.get(out_kind)
        if C0 is None:
            C0 = oracle.f32_to_bf16_bits(C0f)
            kw["out_kind"] = "bfloat16"
    bias = rng.standard_normal(n, dtype=np.float32) if use_bias else None
    got = C0.copy()
    rt.gemm_batched(A, B, got, alpha=alpha, beta=beta, relu=relu, bias=bias, compute=compute, **kw)
    for b in range(batch):
        want = C0[b].copy()
        oracle.gemm(np.ascontiguousarray(A[b]), B[b], want, in_kind=kind, out_kind=out_kind, alpha=alpha, beta=beta,
                    bias=bias, relu=relu)
        what = f"{kind}->{out_kind} {compute} batch {b}/{batch} {m}x{n}x{k}"
        if out_kind == "int32":
            assert np.array_equal(got[b], want), what
            continue
        g, w = (oracle.bf16_bits_to_f32(got[b]), oracle.bf16_bits_to_f32(want)) if out_kind == "bfloat16" else (got[b], want)
        c0 = _as64(C0[b], out_kind)
        scale = abs(alpha) * (np.abs(_as64(A[b], kind)) @ np.abs(_as64(np.asarray(B[b]), kind))) + abs(beta) * np.abs(c0) \
            + (np.abs(bias) if use_bias else 0)
        _close(g, w, scale, rtol, what)


@pytest.mark.parametrize("compute", ["tensor", "tensor_2sm"])
@pytest.mark.parametrize("batch,m,n,k", [(2, 128, 256, 64), (3, 256, 256, 192), (5, 200, 136, 264), (7, 64, 48, 40),
                                         (4, 384, 520, 128), (1, 256, 256, 128)])
def test_batched_bf16_tensor(compute, batch, m, n, k):
    _run_case("bfloat16", "float32", batch, m, n, k, compute, beta=1.0, relu=True)


@pytest.mark.parametrize("compute", ["tensor", "tensor_2sm"])
@pytest.mark.parametrize("kind,out_kind", [("float16", "float16"), ("bfloat16", "bfloat16"), ("float16", "float32")])
@pytest.mark.parametrize("b_kmajor", [True, False])
def test_batched_types_and_b_layouts(compute, kind, out_kind, b_kmajor):
    # b_kmajor False is the reference test's layout: B[b] first-major [K, N] (N-contiguous)
    _run_case(kind, out_kind, 3, 256, 264, 328, compute, beta=0.5, alpha=2.0, relu=False, b_kmajor=b_kmajor, use_bias=True)


@pytest.mark.parametrize("compute", ["tensor", "tensor_2sm", "simt"])
@pytest.mark.parametrize("kind", ["int8", "uint8"])
def test_batched_int8_exact(compute, kind):
    _run_case(kind, "int32", 4, 200, 264, 144, compute, beta=1.0, relu=True)
    _run_case(kind, "int32", 2, 128, 256, 512, compute, beta=0.0, relu=False, b_kmajor=False)


@pytest.mark.parametrize("batch,m,n,k", [(3, 70, 90, 130), (2, 512, 512, 512), (9, 128, 128, 64), (5, 33, 17, 1000),
                                         (40, 64, 64, 64)])
def test_batched_f32_simt(batch, m, n, k):
    # the reference's batch matmul tests default to fp32 arrays, all first-major (mfma_tests.py:441-443)
    _run_case("float32", "float32", batch, m, n, k, "simt", beta=1.0, b_kmajor=False, rtol=1e-5)
    _run_case("float32", "float32", batch, m, n, k, "simt", beta=0.0, alpha=3.0, relu=True, b_kmajor=True, rtol=1e-5)


def test_batched_shared_b_and_fallbacks():
    # one B for all problems (batch stride 0): tensor path and SIMT path
    _run_case("bfloat16", "float32", 6, 256, 256, 128, "tensor_2sm", share_b=True)
    _run_case("float32", "float32", 6, 100, 60, 72, "simt", share_b=True, b_kmajor=False, rtol=1e-5)
    # row pitch of A / B not a multiple of 16 bytes: tensor_preferred / auto fall back to SIMT, tensor refuses
    _run_case("float16", "float32", 3, 9, 40, 20, "tensor_preferred", rtol=1e-5)
    _run_case("float16", "float32", 3, 9, 40, 20, "auto", rtol=1e-5)
    with pytest.raises(rt.AccbError):
        _run_case("float16", "float32", 3, 9, 40, 20, "tensor")


def test_batched_padded_batch_strides():
    # problems 4 elements further apart than dense: 8-byte misaligned for fp16 (SIMT fallback), and 8 elements
    # further apart (16-byte aligned: tensor path)
    rng = np.random.default_rng(21)
    batch, m, n, k = 3, 64, 72, 32
    for pad, compute, rtol in ((4, "tensor_preferred", 1e-5), (8, "tensor", 2e-2), (8, "tensor_2sm", 2e-2)):
        def padded(rows, cols):
            buf = rng.standard_normal(batch * (rows * cols + pad), dtype=np.float32).astype(np.float16)
            return np.lib.stride_tricks.as_strided(buf, shape=(batch, rows, cols),
                                                   strides=((rows * cols + pad) * 2, cols * 2, 2))
        A, Bt = padded(m, k), padded(n, k)
        B = Bt.transpose(0, 2, 1)
        cbuf = rng.standard_normal(batch * (m * n + pad), dtype=np.float32)
        C = np.lib.stride_tricks.as_strided(cbuf, shape=(batch, m, n), strides=((m * n + pad) * 4, n * 4, 4))
        C0 = C.copy()
        guard = cbuf.copy()
        beta = 1.0 if pad == 4 else 0.0            # beta = 0: C is not read, yet the gaps must survive the staging
        rt.gemm_batched(A, B, C, beta=beta, compute=compute)
        for b in range(batch):
            want = C0[b].copy()
            oracle.gemm(np.ascontiguousarray(A[b]), np.asfortranarray(B[b]), want, beta=beta)
            scale = np.abs(A[b].astype(np.float64)) @ np.abs(B[b].astype(np.float64)) + beta * np.abs(C0[b])
            _close(C[b], want, scale, rtol, f"padded batch stride {pad} {compute} problem {b}")
            # the padding between the problems' results is untouched
            lo = b * (m * n + pad) + m * n
            assert np.array_equal(cbuf[lo:lo + pad], guard[lo:lo + pad])
    with pytest.raises(rt.AccbError):
        _misaligned_batch_stride_on_tensor_path(batch, m, n, k)


def _misaligned_batch_stride_on_tensor_path(batch, m, n, k):
    pad = 4
    buf = np.zeros(batch * (m * k + pad), np.float16)
    A = np.lib.stride_tricks.as_strided(buf, shape=(batch, m, k), strides=((m * k + pad) * 2, k * 2, 2))
    B = np.zeros((batch, n, k), np.float16).transpose(0, 2, 1)
    C = np.zeros((batch, m, n), np.float32)
    rt.gemm_batched(A, B, C, compute="tensor")          # batch stride of A is 8 bytes off a 16-byte multiple


def test_batched_matches_looped_single_gemm_bitwise():
    # the batched launch runs the same tile arithmetic as one launch per problem
    rng = np.random.default_rng(5)
    batch, m, n, k = 4, 384, 512, 256
    A = oracle.f32_to_bf16_bits(rng.standard_normal((batch, m, k), dtype=np.float32))
    B = oracle.f32_to_bf16_bits(rng.standard_normal((batch, n, k), dtype=np.float32)).transpose(0, 2, 1)
    C0 = rng.standard_normal((batch, m, n), dtype=np.float32)
    got = C0.copy()
    rt.gemm_batched(A, B, got, beta=1.0, relu=True, compute="tensor_2sm", kind="bfloat16")
    for b in range(batch):
        one = C0[b].copy()
        rt.gemm(A[b], B[b], one, beta=1.0, relu=True, compute="tensor_2sm", kind="bfloat16")
        assert np.array_equal(one, got[b])


def test_batched_argument_checks():
    A = np.zeros((2, 8, 16), np.float32)
    B = np.zeros((2, 16, 8), np.float32)
    C = np.zeros((2, 8, 8), np.float32)
    rt.gemm_batched(A, B, C, compute="simt")
    with pytest.raises(ValueError):
        rt.gemm_batched(A, B[:, :8], C, compute="simt")
    # overlapping results: C's batch stride smaller than one C
    Cov = np.lib.stride_tricks.as_strided(np.zeros(200, np.float32), shape=(2, 8, 8), strides=(16 * 4, 8 * 4, 4))
    with pytest.raises(rt.AccbError):
        rt.gemm_batched(A, B, Cov, compute="simt")
    # an empty batch is a no-op
    rt.gemm_batched(A[:0], B[:0], C[:0], compute="simt")


def test_batched_device_pointers_torch():
    import torch
    torch.manual_seed(3)
    dev = torch.device("cuda:0")
    batch, m, n, k = 8, 512, 384, 256
    A = torch.randn(batch, m, k, device=dev).to(torch.bfloat16)
    B = (torch.randn(batch, n, k, device=dev) / k ** 0.5).to(torch.bfloat16).transpose(1, 2)     # [batch, k, n], K-contiguous
    C = torch.randn(batch, m, n, device=dev).to(torch.bfloat16)
    want = torch.relu(torch.bmm(A.float(), B.float()) + C.float())
    rt.gemm_batched(A, B, C, beta=1.0, relu=True, compute="tensor_2sm")
    rt.synchronize()
    err = (C.float() - want).abs().max().item()
    assert err <= 2e-2 * want.abs().max().item()
    # A shared via expand(): batch stride 0
    A1 = torch.randn(m, k, device=dev).to(torch.bfloat16)
    C2 = torch.zeros(batch, m, n, device=dev, dtype=torch.float32)
    rt.gemm_batched(A1.expand(batch, m, k), B, C2, beta=0.0, compute="tensor")
    rt.synchronize()
    want2 = torch.matmul(A1.float(), B.float())
    assert (C2 - want2).abs().max().item() <= 2e-2 * want2.abs().max().item()


@pytest.mark.parametrize("dtype,out_dtype,tensorize", [("float32", "float32", False), ("float32", "float32", True),
                                                       ("float16", "float32", True), ("float16", "float16", True)])
def test_batch_matmul_hat_package(tmp_path, dtype, out_dtype, tensorize):
    """The reference's batch matmul nest (all arrays first-major), built into a HAT package and called through
    the loader with host arrays, against the oracle problem by problem."""
    batch, M, N, K = 4, 128, 192, 160
    et, ot = getattr(acc.ScalarType, dtype), getattr(acc.ScalarType, out_dtype)
    A = acc.Array(role=acc.Role.INPUT, element_type=et, shape=(batch, M, K))
    B = acc.Array(role=acc.Role.INPUT, element_type=et, shape=(batch, K, N))
    C = acc.Array(role=acc.Role.INPUT_OUTPUT, element_type=ot, shape=(batch, M, N))
    nest = acc.Nest(shape=(batch, M, N, K))
    b, i, j, k = nest.get_indices()

    @nest.iteration_logic
    def _():
        C[b, i, j] += A[b, i, k] * B[b, k, j]

    schedule = nest.create_schedule()
    target = acc.Target(acc.Target.Model.NVIDIA_B200)
    if tensorize:
        ii, jj, kk = schedule.tile({i: 64, j: 64, k: 64})
        splits = target.tensor_core_info.compute_tensor_splits(acc.MMAShape.M16xN16xK16_B1, 1)
        iii, jjj, kkk = schedule.tile({ii: splits[0], jj: splits[1], kk: splits[2]})
        plan, tensor_indices = schedule._create_tensorizable_plan(
            target, block_indices=(i, j), warp_indices=(ii, jj), tensor_indices=(iii, jjj, kkk),
            outer_nest_order=(b, i, j, k, ii, jj, kk))
        plan.tensorize(indices=tensor_indices, mma_shape=acc.MMAShape.M16xN16xK16_B1)
    else:
        plan = schedule.create_plan(target)
    pkg = acc.Package()
    fn = pkg.add(plan, args=(A, B, C), base_name="batch_matmul")
    hat_path = pkg.build(f"bmm_{dtype}_{out_dtype}_{int(tensorize)}", output_dir=str(tmp_path))[0]
    _, fns = hat.load(hat_path)
    rng = np.random.default_rng(11)
    a = rng.standard_normal((batch, M, K), dtype=np.float32).astype(dtype)
    bm = (rng.standard_normal((batch, K, N), dtype=np.float32) / np.float32(np.sqrt(K))).astype(dtype)
    c0 = rng.standard_normal((batch, M, N), dtype=np.float32).astype(out_dtype)
    got = c0.copy()
    fns[fn.name](a, bm, got)
    # fp32 arrays: tensorize on K-strided B cannot use TF32, so both fp32 variants run true fp32 arithmetic
    rtol = 1e-5 if dtype == "float32" else 2e-2
    for p in range(batch):
        want = c0[p].copy()
        oracle.gemm(a[p], bm[p], want, beta=1.0)
        scale = np.abs(a[p].astype(np.float64)) @ np.abs(bm[p].astype(np.float64)) + np.abs(c0[p].astype(np.float64))
        _close(got[p], want, scale, rtol, f"hat batch matmul problem {p}")
