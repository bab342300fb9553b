"""Range (ONNX) - the fourth operator family behind the HAT surface.

CPU tier: the oracle against the golden vectors made by the reference's own numpy loop
(kernels/range/naive_runtime_sized.py:44-56), the host-side plan of the GPU kernel (segments of constant
bit-pattern step) expanded in numpy against the same vectors and against the oracle on random ranges, DSL
recognition of the reference's range-node nests (dsl_tests.py:1436-1506) and the package they build.
GPU tier: the kernel through the C ABI and through a HAT package, bit for bit against the oracle.
"""
import os

import numpy as np
import pytest

import oracle
from accera_b200 import hat, patterns, runtime as rt

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "range.npz")


def _cases():
    g = np.load(GOLDEN)
    for name in sorted({k.rsplit("_", 1)[0] for k in g.files}):
        yield name, g[name + "_args"], g[name + "_out"]


def _expand(first, bits, step, n):
    """numpy restatement of what the fill kernel computes from a plan."""
    out = np.empty(n, dtype=np.uint32)
    for j in range(len(first)):
        end = int(first[j + 1]) if j + 1 < len(first) else n
        idx = np.arange(int(first[j]), end, dtype=np.int64)
        out[int(first[j]):end] = ((int(bits[j]) + (idx - int(first[j])) * int(step[j])) & 0xFFFFFFFF).astype(np.uint32)
    return out


def _same_bits(a, b):
    return np.array_equal(np.asarray(a, np.float32).view(np.uint32), np.asarray(b, np.float32).view(np.uint32))


def test_oracle_matches_the_reference_numpy_loop():
    for name, (start, limit, delta), want in _cases():
        got, final = oracle.range_f32(start, delta, len(want))
        assert _same_bits(got, want), name
        # the size as the DSL test computes it: np.floor((limit - start) / delta) (dsl_tests.py:1482); the numpy
        # prototype's `//` (floor_divide) is one smaller for "tenths" and "thirds", where the fp32 quotient rounds
        # up to an integer, so the golden vectors there are one element shorter than the size
        size = oracle.range_count(start, limit, delta)
        assert size == int(np.floor((limit - start) / delta)), name
        assert size - len(want) == (1 if name in ("tenths", "thirds") else 0), name
    assert oracle.range_count(5.0, 1.0, 1.0) == 0 and oracle.range_count(1.0, 5.0, 0.0) == 0
    assert oracle.range_count(1.0, 5.0, float("nan")) == 0


def test_plan_reproduces_the_serial_loop_on_golden_vectors():
    for name, (start, limit, delta), want in _cases():
        first, bits, step, final = rt.range_plan(start, delta, len(want))
        assert first[0] == 0 and np.all(np.diff(first) > 0), name
        assert _same_bits(_expand(first, bits, step, len(want)).view(np.float32), want), name
        assert _same_bits(final, oracle.range_f32(start, delta, len(want))[1]), name
        assert rt.range_count(start, limit, delta) == oracle.range_count(start, limit, delta), name
        assert len(first) <= 32, (name, len(first))           # a handful of segments, not one per element
    # a stalled recurrence (delta below half an ulp) and a tie that rounds back to even are one constant segment
    for name in ("stall", "tie"):
        start, _, delta = dict((n, a) for n, a, _ in _cases())[name]
        first, bits, step, _ = rt.range_plan(start, delta, 1000)
        assert len(first) == 1 and step[0] == 0


def test_plan_fuzz_against_the_oracle():
    rng = np.random.default_rng(20)
    for it in range(1500):
        mode = it % 8
        if mode == 0:
            s, d = rng.standard_normal() * 10 ** rng.uniform(-3, 3), rng.standard_normal() * 10 ** rng.uniform(-3, 3)
        elif mode == 1:
            s, d = 0.0, 10 ** rng.uniform(-45, -30)                                     # denormals
        elif mode == 2:
            s, d = rng.standard_normal() * 10 ** rng.uniform(-40, 38), rng.standard_normal() * 10 ** rng.uniform(-40, 38)
        elif mode == 3:
            s, d = -abs(rng.standard_normal()) * 100, abs(rng.standard_normal())        # through zero
        elif mode == 4:
            s, d = 2.0 ** rng.integers(-20, 30), 2.0 ** rng.integers(-30, 20) * rng.choice([1, 1.5, 0.5, 3, -1, -0.5])  # ties
        elif mode == 5:
            s, d = 3e38, 1e37 * rng.standard_normal()                                   # into infinity
        elif mode == 6:
            s = rng.standard_normal() * 10 ** rng.uniform(-2, 2)
            d = -np.sign(s) * abs(rng.standard_normal()) * abs(s) * 10 ** rng.uniform(-5, -1)   # towards zero
        else:
            s, d = rng.standard_normal(), rng.standard_normal() * 1e-3
        s, d = np.float32(s), np.float32(d)
        n = int(rng.integers(1, 30000))
        with np.errstate(all="ignore"):
            want, want_final = oracle.range_f32(s, d, n)
        first, bits, step, final = rt.range_plan(s, d, n)
        assert np.array_equal(_expand(first, bits, step, n), want.view(np.uint32)), (s, d, n)
        assert _same_bits(final, want_final), (s, d, n)


def _range_node_package():
    """The nests of the reference's range-node test, as written there (dsl_tests.py:1436-1474)."""
    from accera_b200 import Array, Dimension, Nest, Package, Role, Scalar, ScalarType, cast, create_dimensions, floor

    start = Scalar(ScalarType.float32)
    limit = Scalar(ScalarType.float32)
    delta = Scalar(ScalarType.float32)

    inputDim = create_dimensions()

    outputDim = Dimension(role=Role.OUTPUT)
    output = Array(shape=(inputDim, ), role=Role.INPUT_OUTPUT)
    output_start = Scalar(ScalarType.float32, Role.INPUT_OUTPUT)

    nest1 = Nest((1, ))

    @nest1.iteration_logic
    def _():
        outputDim.set(cast(floor((limit - start) / delta), ScalarType.int64))

    nest2 = Nest([inputDim])
    i = nest2.get_indices()

    @nest2.iteration_logic
    def _():
        output[i] = output_start
        output_start.set(output_start + delta)

    package = Package()
    get_size_fn = package.add(nest1, args=(start, limit, delta, outputDim), base_name="get_size")
    get_result_fn = package.add(nest2, args=(inputDim, output, output_start, delta), base_name="get_result")
    return package, get_size_fn, get_result_fn


def test_range_node_nests_are_recognised_and_packaged(tmp_path):
    package, get_size_fn, get_result_fn = _range_node_package()
    assert get_size_fn.spec.kind == "range_size" and get_result_fn.spec.kind == "range"
    src = package._stub_source("range_pkg")
    # the prototypes the reference's comment gives (dsl_tests.py:1464-1466)
    assert f"void {get_size_fn.name}(float a0, float a1, float a2, int64_t* a3)" in src
    assert f"void {get_result_fn.name}(int64_t a0, float* a1, float* a2, float a3)" in src
    assert "*a3 = accb_range_count_f32(a0, a1, a2);" in src and "accb_range_f32(a0, a1, a2, a3)" in src
    hat_path, lib_path = package.build("range_pkg", output_dir=str(tmp_path))[:2]
    hf = hat.HATFile.read(hat_path)
    size_fn, result_fn = hf.functions
    assert [a.declared_type for a in size_fn.arguments] == ["float", "float", "float", "int64_t*"]
    assert [a.declared_type for a in result_fn.arguments] == ["int64_t", "float*", "float*", "float"]
    assert [a.logical_type for a in result_fn.arguments] == ["element", "runtime_array", "element", "element"]
    assert result_fn.arguments[1].size == "inputDim" and result_fn.arguments[2].usage == "input_output"
    # the size function is host code: callable without a GPU, with the values of the reference's test
    _, fns = hat.load(hat_path)
    out_dim = np.zeros(1, dtype=np.int64)
    fns.get_size(np.float32(1.0), np.float32(5.0), np.float32(0.5), out_dim)
    assert out_dim[0] == 8


def test_range_rejections():
    from accera_b200 import Array, Nest, Package, Role, Scalar, ScalarType
    out = Array(shape=(16, ), role=Role.INPUT_OUTPUT)
    run, delta = Scalar(ScalarType.float32, Role.INPUT_OUTPUT), Scalar(ScalarType.float32)
    nest = Nest([16])
    i = nest.get_indices()

    @nest.iteration_logic
    def _():
        out[i] = run
        run.set(run * delta)                     # a geometric sequence is not Range

    with pytest.raises(patterns.UnsupportedNestError):
        Package().add(nest, args=(out, run, delta), base_name="geo")
    run_in = Scalar(ScalarType.float32)          # the running scalar must be in/out
    nest2 = Nest([16])
    j = nest2.get_indices()

    @nest2.iteration_logic
    def _():
        out[j] = run_in
        run_in.set(run_in + delta)

    with pytest.raises(patterns.UnsupportedNestError):
        Package().add(nest2, args=(out, run_in, delta), base_name="bad_role")


def test_range_compute_fails_loudly_without_gpu():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(rt.AccbError):
        rt.range_f32(np.zeros(8, np.float32), 0.0, 1.0)


# ---------------------------------------------------------------------------------------------------------
# GPU tier
# ---------------------------------------------------------------------------------------------------------

@pytest.mark.gpu
def test_range_gpu_golden_bit_exact():
    for name, (start, limit, delta), want in _cases():
        out = np.full(len(want), np.nan, dtype=np.float32)
        final = rt.range_f32(out, start, delta)
        assert _same_bits(out, want), name
        assert _same_bits(final, oracle.range_f32(start, delta, len(want))[1]), name


@pytest.mark.gpu
@pytest.mark.parametrize("start,delta,n", [(0.0, 1.0, 1), (0.0, 1.0, 7), (1.0, 0.5, 8), (0.0, 0.1, 1 << 20), (-3.5, 1e-3, 3_000_001),
                                            (1e-3, 0.37, 999_999), (16777216.0, 0.75, 100_000), (1e-40, 1.7e-41, 50_000),
                                            (5.0, -1e-4, 2_000_003), (3e38, 1e36, 4096), (0.0, 0.0, 1000)])
def test_range_gpu_matches_the_serial_loop(start, delta, n):
    with np.errstate(all="ignore"):
        want, want_final = oracle.range_f32(start, delta, n)
    out = np.full(n, np.nan, dtype=np.float32)
    final = rt.range_f32(out, start, delta)
    assert _same_bits(out, want) and _same_bits(final, want_final)


@pytest.mark.gpu
def test_range_gpu_long_segment_tables_and_device_output():
    import torch
    dev = torch.device("cuda:0")
    # an unaligned slice of a device buffer: the vector stores must cope with the odd base address, and nothing
    # outside the slice may be written
    n = 1 << 22
    buf = torch.full((n + 7,), float("nan"), device=dev, dtype=torch.float32)
    final = rt.range_f32(buf[3:n + 3], np.float32(1e-38), np.float32(1e-38))
    rt.synchronize()
    want, want_final = oracle.range_f32(1e-38, 1e-38, n)
    assert torch.isnan(buf[:3]).all() and torch.isnan(buf[n + 3:]).all()
    assert _same_bits(buf[3:n + 3].cpu().numpy(), want) and _same_bits(final, want_final)
    # a sweep through zero crosses some 25 binades on each side: more segments than one launch carries, so the
    # table is issued in parts, each starting at an arbitrary element index
    for start, delta, count in ((-1.0, 1e-7, 1 << 24), (-1.0, 2.0 ** -24, (1 << 25) + 5)):
        first, _, _, _ = rt.range_plan(start, delta, count)
        assert len(first) > 64, len(first)
        out = torch.full((count,), float("nan"), device=dev, dtype=torch.float32)
        final = rt.range_f32(out, start, delta)
        rt.synchronize()
        want, want_final = oracle.range_f32(start, delta, count)
        assert _same_bits(out.cpu().numpy(), want) and _same_bits(final, want_final)


@pytest.mark.gpu
def test_range_node_package_end_to_end(tmp_path):
    """The correctness values of the reference's test (dsl_tests.py:1479-1504): start 1, limit 5, delta 0.5."""
    package, get_size_fn, get_result_fn = _range_node_package()
    hat_path = package.build("test_output_array_range_node1", output_dir=str(tmp_path))[0]
    _, fns = hat.load(hat_path)
    start_test, limit_test, delta_test = np.float32(1.0), np.float32(5.0), np.float32(0.5)
    size_test = np.floor((limit_test - start_test) / delta_test).astype(np.int64)
    y_ref = np.arange(start_test, limit_test, delta_test, dtype=np.float32)
    out_dim = np.zeros(1, dtype=np.int64)
    fns[get_size_fn.name](start_test, limit_test, delta_test, out_dim)
    assert out_dim[0] == size_test
    x = np.random.random((int(size_test), )).astype(np.float32)
    start_array = np.array([start_test], dtype=np.float32)
    fns[get_result_fn.name](int(size_test), x, start_array, delta_test)
    np.testing.assert_array_equal(x, y_ref)
    post = start_test
    for _ in range(int(size_test)):
        post += delta_test
    assert start_array[0] == post
    # the alias works too, and a longer range through the same function is bit-exact against the oracle
    n = 123457
    big = np.zeros(n, dtype=np.float32)
    run = np.array([0.25], dtype=np.float32)
    fns.get_result(n, big, run, np.float32(0.001))
    want, want_final = oracle.range_f32(0.25, 0.001, n)
    assert _same_bits(big, want) and _same_bits(run[0], want_final)
