"""End-to-end through the HAT surface on the GPU: describe with the DSL subset, Package.build, load the .hat,
call the exported functions with numpy arrays (hatlib's call shape), compare with the oracle."""
import numpy as np
import pytest

import accera_b200 as acc
import oracle
from accera_b200 import hat

from test_host_layer import gather_package, quickstart_package

pytestmark = pytest.mark.gpu


def test_quickstart_package_end_to_end(tmp_path):
    files = quickstart_package().build(name="hello_accera", format=acc.Package.Format.HAT_DYNAMIC, output_dir=str(tmp_path))
    _, functions = hat.load(files[0])
    A_test = np.random.default_rng(0).random((512, 512)).astype(np.float32)
    B_test = np.random.default_rng(1).random((512, 512)).astype(np.float32)
    for name in ("matmul_relu_fusion_transformed", "matmul_relu_fusion_naive"):
        C_test = np.zeros((512, 512)).astype(np.float32)
        C_numpy = np.maximum(C_test + A_test @ B_test, 0.0)
        functions[name](A_test, B_test, C_test)
        np.testing.assert_allclose(C_test, C_numpy, atol=1e-3)                       # README.md:127-133
        want = oracle.gemm(A_test, B_test, np.zeros((512, 512), np.float32), relu=True)
        np.testing.assert_allclose(C_test, want, rtol=1e-5)
    # C is INPUT_OUTPUT: a second call accumulates on top of the first result; device_id names the GPU, as in
    # the reference's benchmarker (tools/benchmarkers/accera_gemm.py:614)
    C2 = C_test.copy()
    functions.matmul_relu_fusion_naive(A_test, B_test, C2, device_id=0)
    np.testing.assert_allclose(C2, 2 * want, rtol=1e-5)


def test_tensorized_f16_package_with_column_major_b(tmp_path):
    m, n, k = 256, 512, 320
    A = acc.Array(role=acc.Role.INPUT, element_type=acc.ScalarType.float16, shape=(m, k))
    B = acc.Array(role=acc.Role.INPUT, element_type=acc.ScalarType.float16, shape=(k, n), layout=acc.Array.Layout.LAST_MAJOR)
    C = acc.Array(role=acc.Role.INPUT_OUTPUT, element_type=acc.ScalarType.float32, shape=(m, n))
    nest = acc.Nest((m, n, k))
    i, j, kk = nest.get_indices()

    @nest.iteration_logic
    def _():
        C[i, j] += A[i, kk] * B[kk, j]
    target = acc.Target(acc.Target.Model.NVIDIA_B200)
    sched = nest.create_schedule()
    plan = sched.create_plan(target)
    plan.tensorize(indices=(i, j, kk), mma_shape=acc.MMAShape.M16xN16xK16_B1, epilogue_op=acc.MMAFragmentOp.ReLU)
    pkg = acc.Package()
    pkg.add(plan, args=(A, B, C), base_name="matmul_relu_f16")
    files = pkg.build("tc_pkg", output_dir=str(tmp_path))
    _, fns = hat.load(files[0])
    rng = np.random.default_rng(3)
    a = (rng.random((m, k), dtype=np.float32) * 2 - 1).astype(np.float16)
    b = np.asfortranarray((rng.random((k, n), dtype=np.float32) * 2 - 1).astype(np.float16))
    c0 = rng.standard_normal((m, n)).astype(np.float32)
    want = oracle.gemm(a, b, c0.copy(), relu=True)
    got = c0.copy()
    fns.matmul_relu_f16(a, b, got)
    scale = np.abs(a.astype(np.float64)) @ np.abs(b.astype(np.float64)) + np.abs(c0)
    assert (np.abs(got - want) <= 2e-2 * np.maximum(np.abs(want), scale)).all()
    assert (np.abs(got - want) <= 1e-4 * np.maximum(np.abs(want), scale)).all()


@pytest.mark.parametrize("axis", [0, 1])
def test_gather_package_end_to_end(tmp_path, axis):
    files = gather_package(axis).build("test_output_array_gather_node", output_dir=str(tmp_path))
    _, fns = hat.load(files[0])
    rng = np.random.default_rng(5)
    data = rng.standard_normal((50, 64)).astype(np.float32)
    idx = rng.integers(0, 50 if axis == 0 else 64, size=(7, 3), dtype=np.int64)
    want = oracle.gather_rank2(data, idx, axis)
    od = [np.zeros(1, np.int64) for _ in range(3)]
    if axis == 0:
        fns[f"Gather_rank_2_dim_axis_{axis}"](64, 7, 3, *od)
        out = np.zeros([int(d[0]) for d in od], np.float32)
        fns[f"Gather_rank_2_array_axis_{axis}"](7, 3, 50, 64, out.reshape(-1), data.reshape(-1), idx.reshape(-1))
    else:
        fns[f"Gather_rank_2_dim_axis_{axis}"](50, 7, 3, *od)
        out = np.zeros([int(d[0]) for d in od], np.float32)
        fns[f"Gather_rank_2_array_axis_{axis}"](50, 7, 3, 64, out.reshape(-1), data.reshape(-1), idx.reshape(-1))
    assert out.shape == want.shape and out.tobytes() == want.tobytes()


def test_run_benchmark_reports_hatlib_fields(tmp_path):
    files = quickstart_package().build(name="bench_pkg", output_dir=str(tmp_path))
    rows = hat.run_benchmark(files[0], batch_size=2, min_time_in_sec=0.2)
    assert len(rows) == 2
    for r in rows:
        d = r.as_dict()
        assert d["function_name"].startswith("matmul_relu_fusion_") and 0 < d["min_of_means"] <= d["mean"]


@pytest.mark.parametrize("a_layout,b_layout,c_layout", [("F", "C", "C"), ("C", "C", "F"), ("F", "F", "F")])
def test_tensorized_plan_with_any_layout(tmp_path, a_layout, b_layout, c_layout):
    # the reference tensorizes every FIRST/LAST_MAJOR combination (mfma_tests.py:2797-2894); here layouts the
    # tcgen05 kernel cannot take directly still give the right answer (SIMT kernel)
    lay = {"C": acc.Array.Layout.FIRST_MAJOR, "F": acc.Array.Layout.LAST_MAJOR}
    m, n, k = 96, 80, 64
    A = acc.Array(role=acc.Role.INPUT, element_type=acc.ScalarType.float16, shape=(m, k), layout=lay[a_layout])
    B = acc.Array(role=acc.Role.INPUT, element_type=acc.ScalarType.float16, shape=(k, n), layout=lay[b_layout])
    C = acc.Array(role=acc.Role.INPUT_OUTPUT, element_type=acc.ScalarType.float32, shape=(m, n), layout=lay[c_layout])
    nest = acc.Nest((m, n, k))
    i, j, kk = nest.get_indices()

    @nest.iteration_logic
    def _():
        C[i, j] += A[i, kk] * B[kk, j]
    plan = nest.create_schedule().create_plan(acc.Target(acc.Target.Model.NVIDIA_B200))
    plan.tensorize(indices=(i, j, kk), mma_shape=acc.MMAShape.M16xN16xK16_B1, prologue_op=acc.MMAFragmentOp.SET,
                   prologue_arg=0, epilogue_op=acc.MMAFragmentOp.SCALE, epilogue_arg=5.0)
    pkg = acc.Package()
    pkg.add(plan, args=(A, B, C), base_name="mm")
    _, fns = hat.load(pkg.build("lay_pkg", output_dir=str(tmp_path))[0])
    rng = np.random.default_rng(9)
    a = np.asarray(rng.random((m, k)), dtype=np.float16, order=a_layout)
    b = np.asarray(rng.random((k, n)), dtype=np.float16, order=b_layout)
    c = np.asarray(rng.random((m, n)), dtype=np.float32, order=c_layout)
    fns.mm(a, b, c)
    want = 5.0 * (a.astype(np.float64) @ b.astype(np.float64))        # alpha = 5, beta = 0 (mfma_tests.py:194)
    np.testing.assert_allclose(c, want, rtol=1e-3)


def _tensorized_bf16_package(m, n, k, tmp_path, name):
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
    return pkg.build(name, output_dir=str(tmp_path))[0], fn.name


def test_hat_function_on_device_tensors(tmp_path):
    """The loader takes torch CUDA tensors for the arrays: used in place, on torch's current stream, no staging."""
    import torch
    m, n, k = 512, 384, 256
    hat_path, name = _tensorized_bf16_package(m, n, k, tmp_path, "dev_pkg")
    _, fns = hat.load(hat_path)
    dev = torch.device("cuda:0")
    torch.manual_seed(2)
    A = torch.randn(m, k, device=dev).to(torch.bfloat16)
    B = (torch.randn(n, k, device=dev) / k ** 0.5).to(torch.bfloat16).t()          # column-major [k, n]
    C = torch.randn(m, n, device=dev).to(torch.bfloat16)
    want = torch.relu(A.float() @ B.float() + C.float())
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fns[name](A, B, C)
    side.synchronize()
    assert (C.float() - want).abs().max().item() <= 2e-2 * want.abs().max().item()
    # the descriptor is enforced for tensors too
    with pytest.raises(ValueError):
        fns[name](A, B.contiguous(), C)                                # row-major B where the package says column-major
    with pytest.raises(TypeError):
        fns[name](A.float(), B, C)
    with pytest.raises(TypeError):
        fns[name](A.cpu(), B, C)


def test_run_benchmark_device_resident(tmp_path):
    """hatlib times GPU functions on device-resident buffers; TFLOP/s of the reference's GEMM benchmarker is
    2*M*N*K / min_of_means of that timing (accera_gemm.py:640-660)."""
    m = n = k = 2048
    hat_path, name = _tensorized_bf16_package(m, n, k, tmp_path, "bench_dev_pkg")
    on_dev = hat.run_benchmark(hat_path, batch_size=5, min_time_in_sec=0.3, device_resident=True, device_id=0)
    on_host = hat.run_benchmark(hat_path, batch_size=2, min_time_in_sec=0.3, device_id=0, device_resident=False)
    by_default = hat.run_benchmark(hat_path, batch_size=5, min_time_in_sec=0.3, device_id=0)   # a GPU-target package
    assert by_default[0].min_of_means < 0.5 * on_host[0].min_of_means
    assert [r.function_name for r in on_dev] == [name]
    t_dev, t_host = on_dev[0].min_of_means, on_host[0].min_of_means
    tflops = 2.0 * m * n * k / t_dev * 1e-12
    assert 0 < t_dev < t_host              # no PCIe staging in the device-resident timing
    assert tflops > 100.0, tflops           # a 2048^3 bf16 GEMM on the tensor cores is far above any SIMT rate
