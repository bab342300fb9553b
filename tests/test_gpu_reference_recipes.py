"""GPU parity on the headline configuration and on the reference's own test recipes.

  * the benchmark configuration at full size (bf16 65536 x 8192 x 8192, C += A @ B then ReLU), called through the
    HAT function of a built package: sampled row bands against the oracle plus a whole-matrix product check;
  * the long-launch pacing path of the tensor-core kernel on a problem that is cheap to check;
  * the checks the reference runs on its tensorized GPU packages, restated with its input generators and its
    element-wise tolerances (accera/python/accera/test/mfma_tests.py:139-147, 187-196, 1573-1693):
    A, B, C ~ U[0,1) (integers ~ U{-2..1} / U{0..1}), C_ref = alpha * (A @ B) + beta * C,
    numpy.testing.assert_allclose(rtol = 1e-2 fp16, 1e-5 bf16 / int8, 1e-3 fp32-as-TF32);
  * the runtime-size functions called on the GPU with the sizes the reference uses (dsl_tests.py:1051-1069:
    M, N, K = 123, 234, 345);
  * a replicated GEMM with forwarding CTAs on one GPU, and the time-out path of the bounded device-side waits.
"""
import numpy as np
import pytest

import accera_b200 as acc
import oracle
from accera_b200 import hat
from accera_b200 import runtime as rt

pytestmark = pytest.mark.gpu


# ---------------------------------------------------------------------------
# the benchmark configuration, full size, through the HAT function
# ---------------------------------------------------------------------------

def _bf16_relu_package(m, n, k, tmp_path, name):
    A = acc.Array(role=acc.Role.INPUT, element_type=acc.ScalarType.bfloat16, shape=(m, k))
    B = acc.Array(role=acc.Role.INPUT, element_type=acc.ScalarType.bfloat16, shape=(k, n), layout=acc.Array.Layout.LAST_MAJOR)
    C = acc.Array(role=acc.Role.INPUT_OUTPUT, element_type=acc.ScalarType.bfloat16, shape=(m, n))
    nest = acc.Nest((m, n, k))
    i, j, kk = nest.get_indices()

    @nest.iteration_logic
    def _():
        C[i, j] += A[i, kk] * B[kk, j]
    plan = nest.create_schedule().create_plan(acc.Target(acc.Target.Model.NVIDIA_B200))
    plan.tensorize(indices=(i, j, kk), mma_shape=acc.MMAShape.M16xN16xK16_B1, epilogue_op=acc.MMAFragmentOp.ReLU)
    pkg = acc.Package()
    fn = pkg.add(plan, args=(A, B, C), base_name="matmul_relu_bf16")
    plan2 = nest.create_schedule().create_plan(acc.Target(acc.Target.Model.NVIDIA_B200))
    plan2.tensorize(indices=(i, j, kk), mma_shape=acc.MMAShape.M16xN16xK16_B1)
    fn2 = pkg.add(plan2, args=(A, B, C), base_name="matmul_bf16")
    return pkg.build(name, output_dir=str(tmp_path))[0], fn.name, fn2.name


def _bf16_tensor(bits, dev):
    import torch
    return torch.from_numpy(bits.view(np.int16)).to(dev).view(torch.bfloat16)


def test_gemm_bf16_65536_config(tmp_path):
    import torch
    m, n, k = 65536, 8192, 8192
    assert rt.gemm_tile_plan(m, n, k) == {"cta_pairs": True, "tile_cols": 256, "tiles": 8192, "rounds": 111}   # the paced path
    A, B, _ = oracle.inputs_gemm_bf16(m, n, k)                     # the benchmark's distributions, seed 1005
    rng = np.random.default_rng(77)
    C0 = oracle.f32_to_bf16_bits(rng.standard_normal((m, n), dtype=np.float32))   # beta = 1 from a C that is not zero
    hat_path, relu_name, plain_name = _bf16_relu_package(m, n, k, tmp_path, "c5_pkg")
    _, fns = hat.load(hat_path)
    dev = torch.device("cuda:0")
    a_d = _bf16_tensor(A, dev)
    b_d = _bf16_tensor(np.ascontiguousarray(B.T), dev).t()          # [K, N] column-major, as the package declares
    c_relu = _bf16_tensor(C0, dev)
    fns[relu_name](a_d, b_d, c_relu)
    rt.synchronize()
    got = c_relu.cpu().view(torch.int16).numpy().view(np.uint16)
    # row bands: the first tile row, one deep inside the launch (tile row 137 of 256: paced rounds), the last rows
    for r0 in (0, 137 * 256 + 40, m - 16):
        want = oracle.gemm(A[r0:r0 + 16], B, C0[r0:r0 + 16].copy(), in_kind="bfloat16", out_kind="bfloat16", relu=True)
        a64 = oracle.bf16_bits_to_f32(A[r0:r0 + 16]).astype(np.float64)
        b64 = oracle.bf16_bits_to_f32(B).astype(np.float64)
        scale = np.abs(a64) @ np.abs(b64) + np.abs(oracle.bf16_bits_to_f32(C0[r0:r0 + 16]).astype(np.float64))
        g, w = oracle.bf16_bits_to_f32(got[r0:r0 + 16]).astype(np.float64), oracle.bf16_bits_to_f32(want).astype(np.float64)
        err = np.abs(g - w)
        assert (err <= 2e-2 * np.maximum(np.abs(w), scale)).all(), (r0, float(err.max()))
        # the stated tolerance is 2e-2; what is observed is at most one bf16 ulp (2^-7 relative) where the two
        # summation orders round the result to different neighbours
        assert (err <= 2.0 ** -7 * np.abs(w) + 1e-6 * scale).all(), (r0, float(err.max()))
    # whole matrix: C + A @ B without the ReLU is linear, so C.v must equal C0.v + A.(B.v); fp64 on the device
    c_plain = _bf16_tensor(C0, dev)
    fns[plain_name](a_d, b_d, c_plain)
    rt.synchronize()
    assert torch.equal(torch.relu(c_plain), c_relu)                 # the fused ReLU is max(result, 0) of the same result
    gen = torch.Generator(device="cpu").manual_seed(5)
    v = torch.randn(n, generator=gen, dtype=torch.float64).to(dev)
    bv = b_d.double() @ v
    babs = b_d.double().abs() @ v.abs()
    c0_d = _bf16_tensor(C0, dev)
    worst = 0.0
    for r0 in range(0, m, 8192):
        a_blk = a_d[r0:r0 + 8192].double()
        lhs = c_plain[r0:r0 + 8192].double() @ v
        c0_blk = c0_d[r0:r0 + 8192].double()
        rhs = c0_blk @ v + a_blk @ bv
        denom = a_blk.abs() @ babs + c0_blk.abs() @ v.abs()
        worst = max(worst, float(((lhs - rhs).abs() / denom).max()))
    # each output element carries one bf16 rounding (2^-9 relative); the rounding errors of a row average out in the product
    assert worst <= 1e-3, worst


@pytest.mark.parametrize("compute", ["tensor", "tensor_2sm"])
def test_paced_launch_matches_unpaced(compute):
    # 16384 x 8192 x 512: 2048 pair tiles / 4096 single tiles, at least 8 rounds, so the producers pace themselves
    # tile by tile; the result must not depend on it
    import torch
    m, n, k = 16384, 8192, 512
    plan = rt.gemm_tile_plan(m, n, k, compute=compute)
    assert plan["rounds"] >= 8
    A, B, _ = oracle.inputs_gemm_bf16(m, n, k, seed=2005)
    dev = torch.device("cuda:0")
    a_d, b_d = _bf16_tensor(A, dev), _bf16_tensor(np.ascontiguousarray(B.T), dev).t()
    outs = []
    for pace in (-1, 0):
        c = torch.zeros(m, n, device=dev, dtype=torch.bfloat16)
        with rt.options(**{"gemm.pace_pct": pace}):
            rt.gemm(a_d, b_d, c, beta=0.0, relu=True, compute=compute)
        rt.synchronize()
        outs.append(c)
    assert torch.equal(outs[0], outs[1])
    got = outs[0].cpu().view(torch.int16).numpy().view(np.uint16)
    for r0 in (0, 9000, m - 32):
        want = oracle.gemm(A[r0:r0 + 32], B, np.zeros((32, n), np.uint16), in_kind="bfloat16", out_kind="bfloat16", beta=0.0, relu=True)
        g, w = oracle.bf16_bits_to_f32(got[r0:r0 + 32]).astype(np.float64), oracle.bf16_bits_to_f32(want).astype(np.float64)
        scale = np.abs(oracle.bf16_bits_to_f32(A[r0:r0 + 32]).astype(np.float64)) @ np.abs(oracle.bf16_bits_to_f32(B).astype(np.float64))
        assert (np.abs(g - w) <= 2e-2 * np.maximum(np.abs(w), scale)).all()
        assert (np.abs(g - w) <= 2.0 ** -7 * np.abs(w) + 1e-6 * scale).all()


# ---------------------------------------------------------------------------
# the reference's tensorize tests: same shapes, types, input generators and tolerances
# ---------------------------------------------------------------------------

_ST = {"float16": acc.ScalarType.float16, "bfloat16": acc.ScalarType.bfloat16, "float32": acc.ScalarType.float32,
       "int8": acc.ScalarType.int8, "uint8": acc.ScalarType.uint8, "int32": acc.ScalarType.int32}

# (M, N, K, mma shape, input type, output type, tolerance): mfma_tests.py:1573-1693
_REFERENCE_CASES = [
    (16, 16, 16, "M16xN16xK16_B1", "float16", "float16", 1e-3),
    (16, 16, 32, "M16xN16xK16_B1", "float16", "float16", 1e-2),
    (16, 16, 384, "M16xN16xK16_B1", "float16", "float32", 1e-2),
    (64, 128, 64, "M16xN16xK16_B1", "float16", "float16", 1e-2),
    (1024, 512, 1024, "M16xN16xK16_B1", "float16", "float16", 1e-2),
    (1024, 1024, 1024, "M16xN16xK16_B1", "float16", "float32", 1e-2),
    (16, 16, 256, "M16xN16xK16_B1", "bfloat16", "float32", 1e-5),
    (16, 16, 128, "M16xN16xK16_B1", "int8", "int32", 1e-5),
    (64, 16, 128, "M16xN16xK16_B1", "uint8", "int32", 1e-5),
    (32, 8, 384, "M32xN8xK16_B1", "float16", "float32", 1e-2),
    (1024, 1024, 2048, "M32xN8xK16_B1", "float16", "float16", 1e-2),
    (32, 8, 192, "M32xN8xK16_B1", "bfloat16", "float32", 1e-5),
    (32, 8, 96, "M32xN8xK16_B1", "int8", "int32", 1e-5),
    (32, 64, 48, "M32xN8xK16_B1", "uint8", "int32", 1e-5),
    (1024, 1024, 2048, "M8xN32xK16_B1", "float16", "float32", 1e-2),
    (512, 512, 1024, "M8xN32xK16_B1", "bfloat16", "float32", 1e-5),
    (512, 512, 64, "M8xN32xK16_B1", "int8", "int32", 1e-5),
    (512, 256, 64, "M8xN32xK16_B1", "uint8", "int32", 1e-5),
    (16, 16, 16, "M16xN16xK8_B1", "float32", "float32", 1e-3),
    (16, 16, 384, "M16xN16xK8_B1", "float32", "float32", 1e-3),
    (64, 64, 64, "M16xN16xK8_B1", "float32", "float32", 1e-3),
    (1024, 1024, 1024, "M16xN16xK8_B1", "float32", "float32", 1e-3),
]


def _random_like_the_reference(rng, shape, kind):
    """mfma_tests.py:139-147: integers from {-2..1} (unsigned: {0, 1}), floats from U[0, 1) rounded to the type."""
    if kind in ("int8", "int32"):
        return rng.integers(-2, 2, size=shape).astype(kind)
    if kind == "uint8":
        return rng.integers(0, 2, size=shape).astype(kind)
    x = rng.random(shape)
    if kind == "bfloat16":
        return oracle.f32_to_bf16_bits(x.astype(np.float32))
    return x.astype(kind)


def _as_float64(x, kind):
    return oracle.bf16_bits_to_f32(x).astype(np.float64) if kind == "bfloat16" else x.astype(np.float64)


@pytest.mark.parametrize("m,n,k,mma,in_kind,out_kind,tolerance", _REFERENCE_CASES)
def test_reference_tensorize_recipe(tmp_path, m, n, k, mma, in_kind, out_kind, tolerance):
    A = acc.Array(role=acc.Role.INPUT, element_type=_ST[in_kind], shape=(m, k))
    B = acc.Array(role=acc.Role.INPUT, element_type=_ST[in_kind], shape=(k, n))
    C = acc.Array(role=acc.Role.INPUT_OUTPUT, element_type=_ST[out_kind], shape=(m, n))
    nest = acc.Nest((m, n, k))
    i, j, kk = nest.get_indices()

    @nest.iteration_logic
    def _():
        C[i, j] += A[i, kk] * B[kk, j]
    plan = nest.create_schedule().create_plan(acc.Target(acc.Target.Model.NVIDIA_B200))
    plan.tensorize(indices=(i, j, kk), mma_shape=getattr(acc.MMAShape, mma))
    pkg = acc.Package()
    fn = pkg.add(plan, args=(A, B, C), base_name="test_cuda_tensorize")
    _, fns = hat.load(pkg.build("recipe_pkg", output_dir=str(tmp_path))[0])
    rng = np.random.default_rng(m * 31 + n * 7 + k)
    a, b, c = (_random_like_the_reference(rng, s, t) for s, t in (((m, k), in_kind), ((k, n), in_kind), ((m, n), out_kind)))
    c_ref = _as_float64(a, in_kind) @ _as_float64(b, in_kind) + _as_float64(c, out_kind)       # alpha = beta = 1
    fns[fn.name](a, b, c)
    # verifiers.py:31-38: both sides as doubles, element-wise relative tolerance
    np.testing.assert_allclose(_as_float64(c, out_kind), c_ref, rtol=tolerance)


@pytest.mark.parametrize("alpha,beta", [(1.0, 0.0), (5.0, 0.0), (1.0, 3.0), (2.0, 0.5)])
def test_reference_alpha_beta_recipe(tmp_path, alpha, beta):
    # docs/Tutorials/GPU/Tensor_MatMul_ElementWiseOps_GPU.md:88-99: beta = 0 is a SET 0 prologue, beta != 1 a SCALE
    # prologue, alpha != 1 a SCALE epilogue; checked as mfma_tests.py:194 does
    m, n, k = 192, 320, 256
    A = acc.Array(role=acc.Role.INPUT, element_type=acc.ScalarType.float16, shape=(m, k))
    B = acc.Array(role=acc.Role.INPUT, element_type=acc.ScalarType.float16, shape=(k, n))
    C = acc.Array(role=acc.Role.INPUT_OUTPUT, element_type=acc.ScalarType.float32, shape=(m, n))
    nest = acc.Nest((m, n, k))
    i, j, kk = nest.get_indices()

    @nest.iteration_logic
    def _():
        C[i, j] += A[i, kk] * B[kk, j]
    plan = nest.create_schedule().create_plan(acc.Target(acc.Target.Model.NVIDIA_B200))
    kw = {}
    if beta == 0.0:
        kw.update(prologue_op=acc.MMAFragmentOp.SET, prologue_arg=0)
    elif beta != 1.0:
        kw.update(prologue_op=acc.MMAFragmentOp.SCALE, prologue_arg=beta)
    if alpha != 1.0:
        kw.update(epilogue_op=acc.MMAFragmentOp.SCALE, epilogue_arg=alpha)
    plan.tensorize(indices=(i, j, kk), mma_shape=acc.MMAShape.M16xN16xK16_B1, **kw)
    pkg = acc.Package()
    fn = pkg.add(plan, args=(A, B, C), base_name="mm_alpha_beta")
    _, fns = hat.load(pkg.build("ab_pkg", output_dir=str(tmp_path))[0])
    rng = np.random.default_rng(17)
    a, b = rng.random((m, k)).astype(np.float16), rng.random((k, n)).astype(np.float16)
    c = rng.random((m, n)).astype(np.float32)
    # the reference scales the accumulator fragment: SCALE(beta) on C before the products, SCALE(alpha) on the sum
    c_ref = alpha * (a.astype(np.float64) @ b.astype(np.float64) + beta * c.astype(np.float64))
    fns[fn.name](a, b, c)
    np.testing.assert_allclose(c.astype(np.float64), c_ref, rtol=1e-2)
    np.testing.assert_allclose(c.astype(np.float64), c_ref, rtol=1e-5)


# ---------------------------------------------------------------------------
# runtime-size functions on the GPU
# ---------------------------------------------------------------------------

def _runtime_sized_package(tmp_path):
    M, N, K = acc.create_dimensions()
    A = acc.Array(role=acc.Role.INPUT, element_type=acc.ScalarType.float32, shape=(M, K))
    B = acc.Array(role=acc.Role.INPUT, element_type=acc.ScalarType.float32, shape=(K, N))
    C = acc.Array(role=acc.Role.INPUT_OUTPUT, element_type=acc.ScalarType.float32, shape=(M, N))
    nest = acc.Nest((M, N, K))
    i, j, k = nest.get_indices()

    @nest.iteration_logic
    def _():
        C[i, j] += A[i, k] * B[k, j]
    pkg = acc.Package()
    mm = pkg.add(nest, args=(A, B, C, M, N, K), base_name="matmul_dyn")
    R, L = acc.create_dimensions()
    data = acc.Array(role=acc.Role.INPUT, shape=(R, L))
    red = acc.Array(role=acc.Role.INPUT_OUTPUT, shape=(R,))
    n0 = acc.Nest((R,)); a0, = n0.get_indices()

    @n0.iteration_logic
    def _():
        red[a0] = 0.0
    n1 = acc.Nest((R, L)); r, c = n1.get_indices()

    @n1.iteration_logic
    def _():
        red[r] += data[r, c]
    n2 = acc.Nest((R,)); a2, = n2.get_indices()

    @n2.iteration_logic
    def _():
        red[a2] /= acc.cast(L, acc.ScalarType.float32)
    rm = pkg.add(acc.fuse((n0, n1, n2), partial=1), args=(R, L, data, red), base_name="ReduceMean_dyn")
    return pkg.build("dyn_gpu_pkg", output_dir=str(tmp_path))[0], mm.name, rm.name


def test_runtime_sized_matmul_and_reduce_mean_on_the_gpu(tmp_path):
    import torch
    hat_path, mm, rm = _runtime_sized_package(tmp_path)
    _, fns = hat.load(hat_path)
    # the sizes of the reference's runtime-size matmul test (dsl_tests.py:1051-1069), its inputs and its check
    M, N, K = 123, 234, 345
    rng = np.random.default_rng(3)
    a, b, c = (rng.random(s).astype(np.float32) for s in ((M, K), (K, N), (M, N)))
    c_ref = c + a @ b
    want = oracle.gemm(a, b, c.copy())
    got = c.copy()
    fns[mm](a.reshape(-1), b.reshape(-1), got.reshape(-1), M, N, K)
    np.testing.assert_allclose(got, c_ref, rtol=1e-5)                    # the reference's own tolerance
    np.testing.assert_allclose(got, want, rtol=1e-5)
    # the same function at other sizes, no rebuild; and on device tensors
    for (m2, n2, k2) in ((1, 1, 1), (64, 7, 1000), (300, 513, 17)):
        a2, b2, c2 = (rng.random(s).astype(np.float32) for s in ((m2, k2), (k2, n2), (m2, n2)))
        want2 = oracle.gemm(a2, b2, c2.copy())
        dev = torch.device("cuda:0")
        c_dev = torch.from_numpy(c2.copy()).to(dev)
        fns[mm](torch.from_numpy(a2).to(dev).reshape(-1), torch.from_numpy(b2).to(dev).reshape(-1), c_dev.reshape(-1), m2, n2, k2)
        rt.synchronize()
        np.testing.assert_allclose(c_dev.cpu().numpy(), want2, rtol=1e-5)
    # runtime-size reduce_mean over the last axis
    for (r, l) in ((123, 345), (1, 7), (4096, 512), (3, 100000)):
        x = rng.standard_normal((r, l)).astype(np.float32)
        out = np.full(r, np.nan, np.float32)
        fns[rm](r, l, x.reshape(-1), out)
        want_r = oracle.reduce_mean_last_axis(x)
        scale = np.abs(x).mean(axis=1)
        assert (np.abs(out - want_r) <= 1e-5 * np.maximum(np.abs(want_r), scale)).all()
        assert (np.abs(out - x.astype(np.float64).mean(axis=1)) <= 1e-5 * np.maximum(np.abs(want_r), scale)).all()


# ---------------------------------------------------------------------------
# replicated GEMM with forwarding CTAs (all replicas in this GPU's memory), time-out path
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("copy_ctas", [2, 8, 24])
@pytest.mark.parametrize("kind,out_kind,m,n,k", [("bfloat16", "bfloat16", 4096, 2048, 512), ("bfloat16", "bfloat16", 1000, 520, 192),
                                                 ("float16", "float32", 777, 1032, 320), ("int8", "int32", 2048, 1024, 256)])
def test_gemm_replicated_with_forwarding_ctas(copy_ctas, kind, out_kind, m, n, k):
    import torch
    dev = torch.device("cuda:0")
    tmap = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32, "int8": torch.int8, "int32": torch.int32}
    g = torch.Generator(device="cpu").manual_seed(m + n + copy_ctas)
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
    for compute in ("tensor_2sm", "tensor"):
        reps = [C0.clone(), torch.zeros_like(C0), torch.full_like(C0, 3), torch.full_like(C0, 5)]
        with rt.options(**{"gemm.copy_ctas": copy_ctas}):
            rt.gemm_replicated(A, B, reps, beta=1.0, relu=True, compute=compute)
        rt.synchronize()
        for r in reps:
            assert torch.equal(r, want), (compute, copy_ctas)


@pytest.mark.parametrize("compute,m,n", [("tensor", 128, 128), ("tensor_2sm", 256, 256), ("tensor_2sm", 1024, 768)])
def test_bounded_wait_times_out_and_the_context_survives(compute, m, n):
    """The MMA issuer leaves out the commit that completes each CTA's last accumulator (a flag nothing sets), so the
    epilogue's bounded wait runs out after the limit set here; the kernel records where, frees its TMEM and returns,
    the host reports ACCB_ERR_TIMEOUT, and the next launch is not affected by the record of the old failure."""
    import torch
    dev = torch.device("cuda:0")
    k = 128
    torch.manual_seed(m + n)
    A = torch.randn(m, k, device=dev).to(torch.bfloat16)
    B = (torch.randn(n, k, device=dev) / k ** 0.5).to(torch.bfloat16).t()
    C = torch.zeros(m, n, device=dev)
    rt.synchronize()
    with rt.options(**{"gemm.wait_limit_us": 2000, "gemm.test_drop_commit": 1}):
        rt.gemm(A, B, C, beta=0.0, compute=compute)                 # device pointers: the error is deferred ...
        # ... and a launch made while the failure is still uncollected runs normally
    C2 = torch.zeros(m, n, device=dev)
    rt.gemm(A, B, C2, beta=0.0, compute=compute)
    with pytest.raises(rt.AccbError) as ei:
        rt.synchronize()
    assert ei.value.code == rt.ERR_TIMEOUT
    assert "epilogue waiting for the accumulator" in str(ei.value) and "bounded wait ran out" in str(ei.value)
    rt.synchronize()                                                # reported once, then cleared
    want = A.float() @ B.float()
    assert (C2 - want).abs().max().item() <= 2e-2 * want.abs().max().item()
    # host pointers: the call that failed returns the error itself, the next one is clean
    a_np = A.cpu().view(torch.int16).numpy().view(np.uint16)
    b_np = Bt_np = B.t().contiguous().cpu().view(torch.int16).numpy().view(np.uint16).T
    c_np = np.zeros((m, n), np.float32)
    with rt.options(**{"gemm.wait_limit_us": 2000, "gemm.test_drop_commit": 1}):
        with pytest.raises(rt.AccbError) as ei:
            rt.gemm(a_np, b_np, c_np, beta=0.0, compute=compute, kind="bfloat16")
    assert ei.value.code == rt.ERR_TIMEOUT
    rt.gemm(a_np, b_np, c_np, beta=0.0, compute=compute, kind="bfloat16")
    assert np.abs(c_np - want.cpu().numpy()).max() <= 2e-2 * float(want.abs().max())


def test_a_stale_gather_error_is_not_blamed_on_a_later_call():
    import torch
    dev = torch.device("cuda:0")
    rt.synchronize()
    data = torch.arange(40, device=dev, dtype=torch.float32).reshape(10, 4)
    idx = torch.tensor([[3], [12]], device=dev)                     # 12 is outside the table
    out = torch.full((2, 1, 4), -1.0, device=dev)
    rt.gather_rank2(data, idx, out, 0)                              # device pointers: deferred
    # a host-pointer GEMM and a host-pointer gather that are fine must not inherit it
    a = np.ones((8, 8), np.float32)
    c = np.zeros((8, 8), np.float32)
    rt.gemm(a, a, c, compute="simt")
    t = np.arange(12, dtype=np.float32).reshape(3, 4)
    o = np.zeros((1, 1, 4), np.float32)
    rt.gather_rank2(t, np.array([[2]], np.int64), o, 0)
    assert o.reshape(-1).tolist() == [8.0, 9.0, 10.0, 11.0]
    with pytest.raises(rt.AccbError) as ei:
        rt.synchronize()
    assert ei.value.code == rt.ERR_INDEX
    assert out[1].abs().sum().item() == 0.0 and out[0].reshape(-1).tolist() == [12.0, 13.0, 14.0, 15.0]
    rt.synchronize()


# ---------------------------------------------------------------------------
# the reference's int16 matmul test (accera/python/accera/test/int_matmul_tests.py:40-68)
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("m,n,k", [(1, 8, 2), (4, 16, 64), (100, 72, 515)])
def test_reference_int16_matmul_recipe(tmp_path, m, n, k):
    # C[i, j] += cast(A[i, k], int32) * cast(B[j, k], int32) with B stored [N, K]; inputs from {0..99}; the reference
    # compares with (A @ B.T).astype(int32) exactly
    A = acc.Array(role=acc.Role.INPUT, element_type=acc.ScalarType.int16, shape=(m, k))
    B = acc.Array(role=acc.Role.INPUT, element_type=acc.ScalarType.int16, shape=(n, k))
    C = acc.Array(role=acc.Role.INPUT_OUTPUT, element_type=acc.ScalarType.int32, shape=(m, n))
    nest = acc.Nest((m, n, k))
    i, j, kk = nest.get_indices()

    @nest.iteration_logic
    def _():
        C[i, j] += acc.cast(A[i, kk], acc.ScalarType.int32) * acc.cast(B[j, kk], acc.ScalarType.int32)
    pkg = acc.Package()
    fn = pkg.add(nest.create_schedule(), args=(A, B, C), base_name="test_int16_matmul")
    _, fns = hat.load(pkg.build("int16_pkg", output_dir=str(tmp_path))[0])
    rng = np.random.default_rng(m + n)
    a = rng.integers(0, 100, (m, k)).astype(np.int16)
    b = rng.integers(0, 100, (n, k)).astype(np.int16)
    c = np.zeros((m, n), np.int32)
    c_ref = (a.astype(np.int32) @ b.astype(np.int32).transpose()).astype(np.int32)
    fns[fn.name](a, b, c)
    assert np.array_equal(c, c_ref)
    assert np.array_equal(c, oracle.gemm(a, b.T, np.zeros((m, n), np.int32)))
    fns[fn.name](a, b, c)                            # C is INPUT_OUTPUT: a second call accumulates
    assert np.array_equal(c, 2 * c_ref)


@pytest.mark.parametrize("kind,out_kind,m,n,k,a_order,b_order", [
    ("bfloat16", "bfloat16", 768, 320, 3053, "C", "C"),      # odd K, row-major A: rows of 6106 bytes
    ("float16", "float32", 300, 264, 1001, "C", "F"),        # both operands K-contiguous with an odd K
    ("int8", "int32", 520, 128, 1999, "C", "F"),
    ("bfloat16", "float32", 1001, 512, 256, "F", "C"),       # column-major A with an odd M, row-major B
])
def test_operands_with_unaligned_rows_are_repacked_for_the_tensor_cores(kind, out_kind, m, n, k, a_order, b_order):
    # "tensor_preferred" (what a tensorized plan asks for) must give the tensor-core result for operands whose rows are
    # not a multiple of 16 bytes - the reference's BERT list has K = 30522 - and must not fall back to the slow kernel
    before = rt.launch_count()
    _tensor_case_preferred(kind, out_kind, m, n, k, a_order, b_order)
    # one pitched copy per repacked operand + the GEMM: more launches than the single CUDA-core kernel would count
    assert rt.launch_count() - before >= 2
    with pytest.raises(rt.AccbError):                       # an explicit tensor request still refuses the layout
        _tensor_case_preferred(kind, out_kind, m, n, k, a_order, b_order, compute="tensor")


def _tensor_case_preferred(kind, out_kind, m, n, k, a_order, b_order, compute="tensor_preferred"):
    rng = np.random.default_rng(m + n + k)
    lay = lambda x, o: np.asfortranarray(x) if o == "F" else np.ascontiguousarray(x)
    if kind == "int8":
        A = lay(rng.integers(-128, 128, size=(m, k)).astype(np.int8), a_order)
        B = lay(rng.integers(-128, 128, size=(k, n)).astype(np.int8), b_order)
        C0 = rng.integers(-1000, 1000, size=(m, n)).astype(np.int32)
        want = oracle.gemm(A, B, C0.copy(), relu=True)
        got = C0.copy()
        rt.gemm(A, B, got, relu=True, compute=compute)
        assert np.array_equal(got, want)
        return
    Af = rng.standard_normal((m, k), dtype=np.float32)
    Bf = rng.standard_normal((k, n), dtype=np.float32) / np.float32(np.sqrt(k))
    kw = {}
    if kind == "float16":
        A, B = lay(Af.astype(np.float16), a_order), lay(Bf.astype(np.float16), b_order)
        A64, B64 = A.astype(np.float64), B.astype(np.float64)
    else:
        A, B = lay(oracle.f32_to_bf16_bits(Af), a_order), lay(oracle.f32_to_bf16_bits(Bf), b_order)
        A64, B64 = oracle.bf16_bits_to_f32(A).astype(np.float64), oracle.bf16_bits_to_f32(B).astype(np.float64)
        kw["kind"] = "bfloat16"
    C0f = rng.standard_normal((m, n), dtype=np.float32)
    if out_kind == "bfloat16":
        C0 = oracle.f32_to_bf16_bits(C0f)
        kw["out_kind"] = "bfloat16"
    else:
        C0 = C0f
    want = oracle.gemm(A, B, C0.copy(), in_kind=kind, out_kind=out_kind, relu=True)
    got = C0.copy()
    rt.gemm(A, B, got, relu=True, compute=compute, **kw)
    gf = oracle.bf16_bits_to_f32(got) if out_kind == "bfloat16" else got
    wf = oracle.bf16_bits_to_f32(want) if out_kind == "bfloat16" else want
    scale = np.abs(A64) @ np.abs(B64) + np.abs(C0f)
    assert (np.abs(gf.astype(np.float64) - wf) <= 2e-2 * np.maximum(np.abs(wf), scale)).all()
    tight = 1e-2 if out_kind == "bfloat16" else 1e-4
    assert (np.abs(gf.astype(np.float64) - wf) <= tight * np.maximum(np.abs(wf), scale)).all()


@pytest.mark.parametrize("kind,out_kind,m,n,k,a_order,b_order", [
    ("bfloat16", "bfloat16", 256, 512, 16384, "C", "F"),     # 2 tiles, K cut into 16 slices
    ("float16", "float32", 512, 1024, 16384, "F", "C"),      # 8 wide tiles, 8 slices, column-major A / row-major B
    ("int8", "int32", 256, 256, 16384, "C", "F"),            # exact
    ("bfloat16", "float32", 200, 300, 12800, "C", "C"),      # ragged M and N
    ("bfloat16", "bfloat16", 768, 320, 30522, "C", "C"),     # the BERT vocabulary shape: repacked, K padded to 30720, 12 slices
])
def test_few_tiles_and_a_long_k_are_split_along_k(kind, out_kind, m, n, k, a_order, b_order):
    before = rt.launch_count()
    _tensor_case_preferred(kind, out_kind, m, n, k, a_order, b_order)
    assert rt.launch_count() - before >= 2                  # the batched launch over the slices and the reduction pass
    # the split is deterministic: the same bits on every run
    import torch
    dev = torch.device("cuda:0")
    if kind != "int8":
        dt = torch.bfloat16 if kind == "bfloat16" else torch.float16
        A = torch.randn(m, k, device=dev).to(dt)
        B = (torch.randn(n, k, device=dev) / k ** 0.5).to(dt).t()
        outs = []
        for _ in range(2):
            C = torch.zeros(m, n, device=dev)
            rt.gemm(A, B, C, beta=0.0, compute="tensor_preferred")
            rt.synchronize()
            outs.append(C)
        assert torch.equal(outs[0], outs[1])
        if (k * 2) % 16:
            return                                          # the explicit tensor modes refuse rows that are not 16-byte aligned
        # and close to the unsplit launch of the same problem
        C1 = torch.zeros(m, n, device=dev)
        rt.gemm(A, B, C1, beta=0.0, compute="tensor_2sm" if m > 128 else "tensor")
        rt.synchronize()
        assert (outs[0] - C1).abs().max().item() <= 1e-4 * (A.float().abs() @ B.float().abs()).max().item()


# ---------------------------------------------------------------------------
# the three ways the tensor-core epilogue brings C in and out give the same bits
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("compute", ["tensor", "tensor_2sm"])
@pytest.mark.parametrize("kind,out_kind,m,n,k", [
    ("bfloat16", "bfloat16", 1024, 1024, 1024),     # one tile per CTA: the old C of the first boxes is copied during the K loop
    ("bfloat16", "bfloat16", 2500, 1000, 320),      # several tiles per CTA on the narrow grid below, ragged M and N
    ("float16", "float32", 700, 520, 256),          # 4-byte results: one chunk per box
    ("float16", "float16", 130, 72, 64),            # a single partial tile
    ("int8", "int32", 900, 264, 512),               # integer accumulators
])
def test_epilogue_paths_agree_bit_for_bit(compute, kind, out_kind, m, n, k):
    """C <- relu(alpha * A @ B + beta * C + bias) from a non-zero C: results stored from registers, through staging
    boxes stored by TMA, and through boxes the epilogue warps move themselves (with the old C copied in ahead, and
    with the old C read row by row; with eight epilogue warps and with four) must be identical; one of them is checked
    against fp64."""
    import torch
    dev = torch.device("cuda:0")
    g = torch.Generator(device="cpu").manual_seed(m * 7 + n)
    if kind == "int8":
        A = torch.randint(-4, 5, (m, k), generator=g, dtype=torch.int8).to(dev)
        B = torch.randint(-4, 5, (n, k), generator=g, dtype=torch.int8).to(dev).t()
        C0 = torch.randint(-100, 100, (m, n), generator=g, dtype=torch.int32).to(dev)
        bias, alpha, beta = None, 1.0, 1.0
    else:
        dt = torch.bfloat16 if kind == "bfloat16" else torch.float16
        odt = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32}[out_kind]
        A = torch.randn(m, k, generator=g).to(dt).to(dev)
        B = (torch.randn(n, k, generator=g) / k ** 0.5).to(dt).to(dev).t()
        C0 = torch.randn(m, n, generator=g).to(odt).to(dev)
        bias, alpha, beta = torch.randn(n, generator=g).to(dev), 0.5, 2.0
    results = {}
    variants = {"registers": {"gemm.staged_store": 0}, "tma boxes": {"gemm.staged_store": 1},
                "warp-moved boxes, C copied ahead": {"gemm.staged_store": 2, "gemm.c_in": 1},
                "warp-moved boxes": {"gemm.staged_store": 2, "gemm.c_in": 0},
                "warp-moved boxes, C copied ahead, four epilogue warps": {"gemm.staged_store": 2, "gemm.c_in": 1, "gemm.epi_warps": 4},
                "warp-moved boxes, four epilogue warps": {"gemm.staged_store": 2, "gemm.c_in": 0, "gemm.epi_warps": 4}}
    for name, opts in variants.items():
        C = C0.clone()
        with rt.options(**opts):
            # a grid of 8 CTAs makes every CTA walk several tiles, so that copies run ahead across tile boundaries
            rt.gemm(A, B, C, bias=bias, alpha=alpha, beta=beta, relu=True, compute=compute, max_ctas=8 if m > 1024 else 0)
        rt.synchronize()
        results[name] = C
    base = results["tma boxes"]
    for name, C in results.items():
        assert torch.equal(C, base), name
    want = alpha * (A.double() @ B.double()) + beta * C0.double()
    if bias is not None:
        want = want + bias.double()
    want = want.clamp_min(0)
    if kind == "int8":
        assert torch.equal(base.double(), want)
    else:
        scale = (alpha * (A.double().abs() @ B.double().abs()) + beta * C0.double().abs()).clamp_min(1.0)
        assert ((base.double() - want).abs() / scale).max().item() <= 2e-2


# ---------------------------------------------------------------------------
# kernels that may be scheduled before their predecessor has finished still see its results
# ---------------------------------------------------------------------------

def test_back_to_back_launches_see_their_predecessors_results():
    """Every kernel here is launched with programmatic stream serialization: its blocks may become resident while
    the kernel before it in the stream is still running, and must not touch memory before that kernel is done.
    A chain GEMM -> reduce_mean -> gather on one stream, with no synchronisation in between and fresh inputs every
    round, is checked against the same chain computed by torch."""
    import torch
    dev = torch.device("cuda:0")
    g = torch.Generator(device="cpu").manual_seed(5)
    m, n, k = 2048, 1024, 512
    idx = torch.randint(0, m, (300, 1), generator=g).to(dev)
    for round_ in range(12):
        A = torch.randn(m, k, generator=g).to(torch.float16).to(dev)
        B = (torch.randn(n, k, generator=g) / k ** 0.5).to(torch.float16).to(dev).t()
        C = torch.full((m, n), float(round_), device=dev)                  # fp32 result, beta = 1 from a known C
        mean = torch.full((m,), float("nan"), device=dev)
        rows = torch.full((300, 1, n), float("nan"), device=dev)
        cols = torch.full((n,), float("nan"), device=dev)
        rt.gemm(A, B, C, beta=1.0, relu=True, compute="tensor_preferred")
        rt.reduce_mean_rank3(C.view(1, m, n), mean, [2])                    # reads what the GEMM wrote
        rt.reduce_mean_rank3(C.view(1, m, n), cols, [1])                    # split reduction: two dependent launches
        rt.gather_rank2(C, idx, rows, 0)
        rt.gemm(A, B, C, beta=1.0, relu=False, compute="tensor_preferred")  # overwrites what the three kernels above read
        rt.synchronize()
        want_c = torch.relu(A.float() @ B.float() + float(round_))
        scale = (A.float().abs() @ B.float().abs()).max().item() + round_
        assert (mean - want_c.mean(dim=1)).abs().max().item() <= 2e-2 * scale
        assert (cols - want_c.mean(dim=0)).abs().max().item() <= 2e-2 * scale
        assert (rows.view(300, n) - want_c[idx.view(-1)]).abs().max().item() <= 2e-2 * scale
        # the consumers read exactly the first GEMM's output, bit for bit: recompute them from a saved copy
        C1 = torch.full((m, n), float(round_), device=dev)
        rt.gemm(A, B, C1, beta=1.0, relu=True, compute="tensor_preferred")
        rt.synchronize()
        mean1 = torch.empty(m, device=dev)
        rt.reduce_mean_rank3(C1.view(1, m, n), mean1, [2])
        rt.synchronize()
        assert torch.equal(mean, mean1)
        assert torch.equal(rows.view(300, n), C1[idx.view(-1)])


def test_fp32_operands_with_unaligned_rows_take_the_tf32_path_when_asked():
    """4-byte elements through the same repacking: fp32 rows of 1001 elements (4004 bytes) are not 16-byte aligned;
    "tensor_preferred" repacks them and computes in TF32 (tolerance 1e-3 of the |A| @ |B| scale, the reference's
    fp32-as-TF32 bar)."""
    import torch
    dev = torch.device("cuda:0")
    g = torch.Generator(device="cpu").manual_seed(17)
    m, n, k = 300, 264, 1001
    A = torch.randn(m, k, generator=g).to(dev)
    B = (torch.randn(n, k, generator=g) / k ** 0.5).to(dev).t()        # K-contiguous, rows of 4004 bytes
    C0 = torch.randn(m, n, generator=g).to(dev)
    C = C0.clone()
    before = rt.launch_count()
    rt.gemm(A, B, C, beta=1.0, relu=True, compute="tensor_preferred")
    rt.synchronize()
    assert rt.launch_count() - before >= 3                              # two repacks and the GEMM
    want = torch.relu(A.double() @ B.double() + C0.double())
    scale = A.double().abs() @ B.double().abs() + C0.double().abs()
    assert ((C.double() - want).abs() / scale).max().item() <= 1e-3
