"""CPU-only tests of the host side: DSL capture, operator recognition, package build (.hat + stub library),
HAT round trip, loader argument checks, C-ABI exports.  No compute call is made (there is no GPU here and
no CPU fallback in the product)."""
import ctypes
import os
import re
import subprocess

import numpy as np
import pytest

import accera_b200 as acc
from accera_b200 import hat, patterns, runtime

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def quickstart_package():
    """The reference's README quickstart (README.md:53-91), verbatim apart from the import name."""
    A = acc.Array(role=acc.Role.INPUT, shape=(512, 512))
    B = acc.Array(role=acc.Role.INPUT, shape=(512, 512))
    C = acc.Array(role=acc.Role.INPUT_OUTPUT, shape=(512, 512))
    matmul = acc.Nest(shape=(512, 512, 512))
    i1, j1, k1 = matmul.get_indices()

    @matmul.iteration_logic
    def _():
        C[i1, j1] += A[i1, k1] * B[k1, j1]

    relu = acc.Nest(shape=(512, 512))
    i2, j2 = relu.get_indices()

    @relu.iteration_logic
    def _():
        C[i2, j2] = acc.max(C[i2, j2], 0.0)

    package = acc.Package()
    schedule = acc.fuse(matmul.create_schedule(), relu.create_schedule(), partial=2)
    package.add(schedule, args=(A, B, C), base_name="matmul_relu_fusion_naive")
    i, j, f, k = schedule.get_indices()
    ii, jj = schedule.tile({i: 16, j: 16})
    schedule.reorder(j, i, f, k, jj, ii)
    plan = schedule.create_plan()
    plan.unroll(ii)
    package.add(plan, args=(A, B, C), base_name="matmul_relu_fusion_transformed")
    return package


def test_c_abi_library_exports_every_declared_symbol():
    lib = runtime.lib()
    header = open(os.path.join(ROOT, "include", "accera_b200.h")).read()
    declared = set(re.findall(r"\b(accb_\w+)\s*\(", header))
    assert declared == set(runtime.EXPORTED_SYMBOLS)
    out = subprocess.run(["nm", "-D", "--defined-only", runtime.LIB_PATH], capture_output=True, text=True, check=True).stdout
    exported = set(re.findall(r"\bT (accb_\w+)", out))
    assert declared <= exported
    for sym in declared:
        getattr(lib, sym)
    assert b"sm_100a" in lib.accb_version()


def test_no_cpu_fallback_compute_fails_loudly_without_gpu():
    if runtime.device_count() > 0:
        pytest.skip("a GPU is visible")
    a = np.zeros((4, 4), np.float32)
    with pytest.raises(runtime.AccbError) as ei:
        runtime.gemm(a, a, a.copy())
    assert ei.value.code == runtime.ERR_CUDA
    with pytest.raises(runtime.AccbError):
        runtime.reduce_mean_rank3(np.zeros((1, 2, 3), np.float32), np.zeros(2, np.float32), [2])
    with pytest.raises(runtime.AccbError):
        runtime.gather_rank2(a, np.zeros((1, 1), np.int64), np.zeros((1, 1, 4), np.float32), 0)


def test_host_only_dim_helpers():
    assert runtime.gather_rank2_dims(5, 4, 2, 3, 0) == (2, 3, 4)
    assert runtime.gather_rank2_dims(5, 4, 2, 3, 1) == (5, 2, 3)
    assert runtime.reduce_mean_rank3_dims(2, 3, 4, [2], 0)[0] == (2, 3)
    assert runtime.reduce_mean_rank3_dims(2, 3, 4, [0, 2], 1)[0] == (1, 3, 1)
    assert runtime.reduce_mean_rank3_dims(2, 3, 4, [], 0)[0] == (1,)


def test_argument_validation_happens_before_any_cuda_call():
    lib = runtime.lib()
    d = runtime.GemmDesc()
    d.m, d.n, d.k = 4, 4, -1
    assert lib.accb_gemm(ctypes.byref(d), None, None, None, None) == runtime.ERR_ARG
    assert b"negative" in lib.accb_last_error()
    assert lib.accb_gemm(None, None, None, None, None) == runtime.ERR_ARG
    assert lib.accb_gather_rank2(None, 1, 1, None, 1, 1, None, 2, 4) == runtime.ERR_ARG
    assert lib.accb_gather_rank2(None, 1, 1, None, 1, 1, None, 0, 3) == runtime.ERR_ARG
    assert lib.accb_reduce_mean_rank3(None, 1, 1, 1, None, 9) == runtime.ERR_ARG


def test_quickstart_builds_hat_dynamic_package(tmp_path):
    package = quickstart_package()
    files = package.build(name="hello_accera", format=acc.Package.Format.HAT_DYNAMIC, output_dir=str(tmp_path))
    assert [os.path.basename(f) for f in files] == ["hello_accera.hat", "hello_accera.so"]
    hf = hat.HATFile.Deserialize(files[0])
    assert hf.name == "hello_accera"
    names = [f.name for f in hf.functions]
    assert len(names) == 2 and re.fullmatch(r"matmul_relu_fusion_naive_[0-9a-f]{16}", names[0])
    f0 = hf.functions[0]
    assert f0.calling_convention == "cdecl"
    assert [a.usage for a in f0.arguments] == ["input", "input", "input_output"]
    assert all(a.logical_type == "affine_array" and a.declared_type == "float*" and a.shape == [512, 512]
               and a.affine_map == [512, 1] and a.affine_offset == 0 for a in f0.arguments)
    assert f0.return_info.logical_type == "void"
    assert f0.auxiliary["accera"]["parameters"] == {}
    assert f0.auxiliary["accera_b200"]["relu"] is True and f0.auxiliary["accera_b200"]["compute"] == "simt"
    assert hf.dependencies["link_target"] == "hello_accera.so"
    assert hf.target["required"]["GPU"]["instruction_set_version"] == "sm_100a"
    # header text: unnamed-parameter prototypes and guarded aliases (TranslateToHeader.cpp:402-506)
    assert f"void {names[0]}(float*, float*, float*);" in hf.declaration_code
    assert f"void (*matmul_relu_fusion_naive)(float*, float*, float*) = {names[0]};" in hf.declaration_code
    assert "#ifndef __matmul_relu_fusion_naive_DEFINED__" in hf.declaration_code
    # the library exports exactly those symbols
    out = subprocess.run(["nm", "-D", "--defined-only", files[1]], capture_output=True, text=True, check=True).stdout
    for n in names:
        assert re.search(rf"\bT {n}\b", out)
    # and the same file is a usable C header
    src = tmp_path / "client.c"
    src.write_text('#include "hello_accera.hat"\nint main(void) { return matmul_relu_fusion_naive == 0; }\n')
    subprocess.run(["gcc", "-c", str(src), "-I", str(tmp_path), "-o", str(tmp_path / "client.o")], check=True)


def test_function_names_are_stable_and_depend_on_signature():
    p1, p2 = quickstart_package(), quickstart_package()
    assert list(p1._fns) == list(p2._fns)
    A = acc.Array(role=acc.Role.INPUT, shape=(256, 512))
    B = acc.Array(role=acc.Role.INPUT, shape=(512, 512))
    C = acc.Array(role=acc.Role.INPUT_OUTPUT, shape=(256, 512))
    n = acc.Nest(shape=(256, 512, 512))
    i, j, k = n.get_indices()

    @n.iteration_logic
    def _():
        C[i, j] += A[i, k] * B[k, j]
    p3 = acc.Package()
    fn = p3.add(n, args=(A, B, C), base_name="matmul_relu_fusion_naive")
    assert fn.name not in p1._fns and fn.name.startswith("matmul_relu_fusion_naive_")
    assert p3.add(n, args=(A, B, C)).name.startswith("_")          # no base name: anonymous hashed name


def _gemm_nest(m, n, k, et_in, et_out, b_layout=acc.Layout.FIRST_MAJOR, transposed_b=False):
    A = acc.Array(role=acc.Role.INPUT, element_type=et_in, shape=(m, k))
    B = acc.Array(role=acc.Role.INPUT, element_type=et_in, shape=(n, k) if transposed_b else (k, n), layout=b_layout)
    C = acc.Array(role=acc.Role.INPUT_OUTPUT, element_type=et_out, shape=(m, n))
    nest = acc.Nest(shape=(m, n, k))
    i, j, kk = nest.get_indices()

    @nest.iteration_logic
    def _():
        if transposed_b:
            C[i, j] += acc.cast(A[i, kk], et_out) * acc.cast(B[j, kk], et_out)
        else:
            C[i, j] += A[i, kk] * B[kk, j]
    return nest, (A, B, C)


def test_recognise_tensorized_gemm_with_fragment_ops():
    nest, (A, B, C) = _gemm_nest(4096, 4096, 4096, acc.ScalarType.float16, acc.ScalarType.float32, acc.Layout.LAST_MAJOR)
    target = acc.Target(acc.Target.Model.NVIDIA_B200)
    plan = nest.create_schedule().create_plan(target)
    i, j, k = nest.get_indices()
    plan.tensorize(indices=(i, j, k), mma_shape=acc.MMAShape.M16xN16xK16_B1, prologue_op=acc.MMAFragmentOp.SET,
                   prologue_arg=0, epilogue_op=acc.MMAFragmentOp.ReLU)
    spec = patterns.recognise(plan)
    assert spec.kind == "gemm" and spec.compute == "tensor" and spec.relu and spec.beta == 0.0 and spec.alpha == 1.0
    assert B.strides() == (1, 4096) and A.strides() == (4096, 1)
    plan2 = nest.create_schedule().create_plan(target)
    plan2.tensorize(indices=(i, j, k), mma_shape=acc.MMAShape.M16xN16xK16_B1, prologue_op=acc.MMAFragmentOp.SCALE,
                    prologue_arg=0.5, epilogue_op=acc.MMAFragmentOp.SCALE, epilogue_arg=4.0)
    spec2 = patterns.recognise(plan2)
    assert spec2.alpha == 4.0 and spec2.beta == 2.0 and not spec2.relu      # 4 * (0.5 * C + A @ B)


def test_recognise_transposed_operand_with_casts():
    # int_matmul_tests.py:55 form: C[i,j] += cast(A[i,k]) * cast(B[j,k])
    nest, _ = _gemm_nest(64, 32, 128, acc.ScalarType.int8, acc.ScalarType.int32, transposed_b=True)
    spec = patterns.recognise(nest)
    assert spec.kind == "gemm" and spec.b_transposed and not spec.a_transposed and (spec.m, spec.n, spec.k) == (64, 32, 128)


def test_bias_relu_fusion_and_rejections():
    m, n, k = 64, 48, 32
    A = acc.Array(role=acc.Role.INPUT, shape=(m, k)); B = acc.Array(role=acc.Role.INPUT, shape=(k, n))
    C = acc.Array(role=acc.Role.INPUT_OUTPUT, shape=(m, n)); bias = acc.Array(role=acc.Role.INPUT, shape=(n,))
    mm = acc.Nest((m, n, k)); i, j, kk = mm.get_indices()

    @mm.iteration_logic
    def _():
        C[i, j] += A[i, kk] * B[kk, j]
    bn = acc.Nest((m, n)); bi, bj = bn.get_indices()

    @bn.iteration_logic
    def _():
        C[bi, bj] += bias[bj]
    rn = acc.Nest((m, n)); ri, rj = rn.get_indices()

    @rn.iteration_logic
    def _():
        C[ri, rj] = acc.max(0.0, C[ri, rj])
    spec = patterns.recognise(acc.fuse((mm, bn, rn), partial=2))
    assert spec.bias is bias and spec.relu
    with pytest.raises(patterns.UnsupportedNestError):
        patterns.recognise(acc.fuse((mm, rn, bn), partial=2))          # nothing may follow the ReLU
    other = acc.Nest((m, n)); oi, oj = other.get_indices()

    @other.iteration_logic
    def _():
        C[oi, oj] = C[oi, oj] * 2.0
    with pytest.raises(patterns.UnsupportedNestError):
        patterns.recognise(other)                                       # not one of the implemented operators
    pkg = acc.Package()
    with pytest.raises(ValueError):
        pkg.add(acc.fuse((mm, bn, rn), partial=2), args=(A, B, C), base_name="x")   # bias missing from args


def test_single_target_rule_and_temp_args():
    nest, args = _gemm_nest(64, 64, 64, acc.ScalarType.float32, acc.ScalarType.float32)
    pkg = acc.Package()
    pkg.add(nest, args=args, base_name="host_fn")
    gpu_plan = nest.create_schedule().create_plan(acc.Target(acc.Target.Model.NVIDIA_B200))
    with pytest.raises(NotImplementedError):                             # unit_tests.py:218
        pkg.add(gpu_plan, args=args, base_name="gpu_fn")
    T = acc.Array(role=acc.Role.TEMP, shape=(4, 4))
    with pytest.raises(ValueError):
        pkg.add(nest, args=(T,) + tuple(args), base_name="bad")


def gather_package(axis):
    """dsl_tests.py:1571-1675: a dimension function and a compute function per axis."""
    DataDim0, DataDim1, IndicesDim0, IndicesDim1 = acc.create_dimensions()
    OutputDim0, OutputDim1, OutputDim2 = acc.create_dimensions(acc.Role.OUTPUT)
    Data = acc.Array(shape=(DataDim0, DataDim1), role=acc.Role.INPUT)
    Indices = acc.Array(shape=(IndicesDim0, IndicesDim1), role=acc.Role.INPUT, element_type=acc.ScalarType.index)
    package = acc.Package()
    if axis == 0:
        Output = acc.Array(shape=(IndicesDim0, IndicesDim1, DataDim1), role=acc.Role.INPUT_OUTPUT)
        nest_dims = acc.Nest((1, ))

        @nest_dims.iteration_logic
        def _():
            OutputDim0.set(IndicesDim0)
            OutputDim1.set(IndicesDim1)
            OutputDim2.set(DataDim1)
        nest_array = acc.Nest((IndicesDim0, IndicesDim1, DataDim1))
        i, j, k = nest_array.get_indices()

        @nest_array.iteration_logic
        def _():
            Output[i, j, k] = Data[Indices[i, j], k]
        package.add(nest_dims, args=(DataDim1, IndicesDim0, IndicesDim1, OutputDim0, OutputDim1, OutputDim2),
                    base_name=f"Gather_rank_2_dim_axis_{axis}")
        package.add(nest_array, args=(IndicesDim0, IndicesDim1, DataDim0, DataDim1, Output, Data, Indices),
                    base_name=f"Gather_rank_2_array_axis_{axis}")
    else:
        Output = acc.Array(shape=(DataDim0, IndicesDim0, IndicesDim1), role=acc.Role.INPUT_OUTPUT)
        nest_dims = acc.Nest((1, ))

        @nest_dims.iteration_logic
        def _():
            OutputDim0.set(DataDim0)
            OutputDim1.set(IndicesDim0)
            OutputDim2.set(IndicesDim1)
        nest_array = acc.Nest((DataDim0, IndicesDim0, IndicesDim1))
        i, j, k = nest_array.get_indices()

        @nest_array.iteration_logic
        def _():
            Output[i, j, k] = Data[i, Indices[j, k]]
        package.add(nest_dims, args=(DataDim0, IndicesDim0, IndicesDim1, OutputDim0, OutputDim1, OutputDim2),
                    base_name=f"Gather_rank_2_dim_axis_{axis}")
        package.add(nest_array, args=(DataDim0, IndicesDim0, IndicesDim1, DataDim1, Output, Data, Indices),
                    base_name=f"Gather_rank_2_array_axis_{axis}")
    return package


@pytest.mark.parametrize("axis", [0, 1])
def test_gather_package_prototypes_and_dimension_function(tmp_path, axis):
    package = gather_package(axis)
    files = package.build("test_output_array_gather_node", format=acc.Package.Format.HAT_DYNAMIC, output_dir=str(tmp_path))
    hf = hat.HATFile.read(files[0])
    dim_fn, arr_fn = hf.functions
    assert dim_fn.c_declaration().endswith("(int64_t, int64_t, int64_t, int64_t*, int64_t*, int64_t*);")
    assert arr_fn.c_declaration().endswith("(int64_t, int64_t, int64_t, int64_t, float*, float*, int64_t*);")
    out_arg = arr_fn.arguments[4]
    assert out_arg.logical_type == "runtime_array" and out_arg.usage == "input_output"
    assert out_arg.size == ("IndicesDim0*IndicesDim1*DataDim1" if axis == 0 else "DataDim0*IndicesDim0*IndicesDim1")
    assert arr_fn.arguments[6].element_type == "int64_t"
    # the dimension function is pure host code: call it through the loader
    _, fns = hat.load(files[0])
    o = [np.zeros(1, np.int64) for _ in range(3)]
    fns[f"Gather_rank_2_dim_axis_{axis}"](7, 2, 3, *o)
    assert [int(x[0]) for x in o] == [2, 3, 7] if axis == 0 else [7, 2, 3]


def test_reduce_mean_recognition_static_and_package(tmp_path):
    data = acc.Array(role=acc.Role.INPUT, shape=(8192, 4096))
    red = acc.Array(role=acc.Role.INPUT_OUTPUT, shape=(8192,))
    init = acc.Nest((8192,)); i0, = init.get_indices()

    @init.iteration_logic
    def _():
        red[i0] = acc.cast(0, acc.ScalarType.float32)
    accn = acc.Nest((8192, 4096)); r, c = accn.get_indices()

    @accn.iteration_logic
    def _():
        red[r] += data[r, c]
    div = acc.Nest((8192,)); i1, = div.get_indices()

    @div.iteration_logic
    def _():
        red[i1] /= acc.cast(4096, acc.ScalarType.float32)
    sched = acc.fuse((init, accn, div), partial=1)
    spec = patterns.recognise(sched)
    assert spec.kind == "reduce_mean" and spec.axes == (1,) and spec.keepdims == 0
    pkg = acc.Package()
    pkg.add(sched, args=(data, red), base_name="ReduceMean_rows")
    files = pkg.build("reduce_pkg", format=acc.Package.Format.HAT_DYNAMIC | acc.Package.Format.SOURCE, output_dir=str(tmp_path))
    src = open([f for f in files if f.endswith(".cpp")][0]).read()
    assert "accb_reduce_mean_rank3(a0, INT64_C(1), INT64_C(8192), INT64_C(4096), a1, 4)" in src


def test_hat_round_trip_preserves_description_and_functions(tmp_path):
    pkg = quickstart_package()
    pkg.add_description(author="someone", license="https://example.org/license", version="1.2",
                        other={"title": "quickstart", "nested": {"a": 1}})        # dsl_tests.py:6398-6449
    files = pkg.build("meta_pkg", output_dir=str(tmp_path))
    hf = hat.HATFile.Deserialize(files[0])
    assert hf.description["author"] == "someone" and hf.description["version"] == "1.2"
    assert hf.description["license_url"] == "https://example.org/license"
    assert hf.description["auxiliary"] == {"title": "quickstart", "nested": {"a": 1}}
    out = tmp_path / "copy.hat"
    hf.Serialize(str(out))
    again = hat.HATFile.Deserialize(str(out))
    assert [f.name for f in again.functions] == [f.name for f in hf.functions]
    assert again.functions[0].arguments == hf.functions[0].arguments
    assert again.declaration_code.strip() == hf.declaration_code.strip()
    assert again.dependencies == hf.dependencies and again.target == hf.target


def test_loader_checks_arguments_against_descriptor(tmp_path):
    nest, args = _gemm_nest(64, 32, 48, acc.ScalarType.float16, acc.ScalarType.float32, acc.Layout.LAST_MAJOR)
    pkg = acc.Package()
    pkg.add(nest, args=args, base_name="mm")
    files = pkg.build("chk", output_dir=str(tmp_path))
    package, fns = hat.load(files[0])
    assert len(fns.names) == 1 and "mm" in fns and fns.mm is fns[fns.names[0]]
    assert package.get_functions()[0].auxiliary["accera"]["parameters"] == {}      # dsl_tests.py:5787-5842
    A = np.zeros((64, 48), np.float16); B = np.zeros((48, 32), np.float16); C = np.zeros((64, 32), np.float32)
    with pytest.raises(ValueError, match="order='F'"):
        fns.mm(A, B, C)                                    # B is LAST_MAJOR in the descriptor
    with pytest.raises(TypeError):
        fns.mm(A.astype(np.float32), np.asfortranarray(B), C)
    with pytest.raises(ValueError):
        fns.mm(A[:32], np.asfortranarray(B), C)
    with pytest.raises(ValueError):
        fns.mm(A, np.asfortranarray(B))


def test_static_package_and_format_rules(tmp_path):
    pkg = quickstart_package()
    files = pkg.build("static_pkg", format=acc.Package.Format.HAT_STATIC, output_dir=str(tmp_path))
    assert [os.path.basename(f) for f in files] == ["static_pkg.hat", "static_pkg.a"]
    assert hat.HATFile.read(files[0]).dependencies["link_target"] == "static_pkg.a"
    with pytest.raises(RuntimeError):
        hat.load(files[0])
    with pytest.raises(NotImplementedError):
        pkg.build("dbg", mode=acc.Package.Mode.DEBUG, output_dir=str(tmp_path))


def test_benchmark_statistics_fields():
    import dataclasses
    r = hat.BenchmarkResult.from_batch_means("f", [3.0, 1.0, 2.0, 10.0, 1.5])
    d = r.as_dict()
    assert dataclasses.asdict(r) == d            # the reference's benchmarker calls asdict() on the records
    assert set(d) == {"function_name", "mean", "median_of_means", "mean_of_small_means", "robust_mean", "min_of_means"}
    assert d["min_of_means"] == 1.0 and d["median_of_means"] == 2.0 and d["mean"] == pytest.approx(3.5)
    assert d["robust_mean"] == pytest.approx((1.5 + 2.0 + 3.0) / 3)


def test_runtime_sized_matmul_and_reduce_mean_packages(tmp_path):
    # runtime-size matmul (dsl_tests.py:1051-1069 form): dimensions are int64 arguments, arrays are runtime_arrays
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
    pkg.add(nest, args=(A, B, C, M, N, K), base_name="matmul_dyn")
    # runtime-size reduce_mean over the last axis of a rank-2 array
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
    pkg.add(acc.fuse((n0, n1, n2), partial=1), args=(R, L, data, red), base_name="ReduceMean_dyn")
    files = pkg.build("dyn_pkg", format=acc.Package.Format.HAT_DYNAMIC | acc.Package.Format.SOURCE, output_dir=str(tmp_path))
    hf = hat.HATFile.read(files[0])
    mm, rm = hf.functions
    assert mm.c_declaration().endswith("(float*, float*, float*, int64_t, int64_t, int64_t);")
    assert [a.logical_type for a in mm.arguments] == ["runtime_array"] * 3 + ["element"] * 3
    assert mm.arguments[0].size == "M*K" and mm.arguments[2].size == "M*N" and mm.arguments[3].name == "M"
    assert rm.c_declaration().endswith("(int64_t, int64_t, float*, float*);")
    src = open([f for f in files if f.endswith(".cpp")][0]).read()
    assert "d.m = a3; d.n = a4; d.k = a5;" in src and "d.a_stride[0] = a5;" in src and "d.c_stride[0] = a4;" in src
    assert "accb_reduce_mean_rank3(a2, INT64_C(1), a0, a1, a3, 4)" in src


def test_gpu_target_functions_are_host_callable_and_record_the_true_launch(tmp_path):
    # The reference lists a GPU function's kernel as a device function that its loader compiles from the `.cu`
    # provider and launches itself (Package.py:714-743).  Here the exported function is a host-callable stub over a
    # prebuilt library, so it must look like one to any loader: no `launches`, no device-function table.  What the
    # stub ends up launching is recorded under auxiliary, from the library's own tile plan.
    nest, args = _gemm_nest(512, 512, 512, acc.ScalarType.float16, acc.ScalarType.float32, acc.Layout.LAST_MAJOR)
    plan = nest.create_schedule().create_plan(acc.Target(acc.Target.Model.NVIDIA_B200))
    plan.tensorize(indices=tuple(nest.get_indices()), mma_shape=acc.MMAShape.M16xN16xK16_B1)
    pkg = acc.Package()
    fn = pkg.add(plan, args=args, base_name="mm_gpu")
    big_nest, big_args = _gemm_nest(65536, 8192, 8192, acc.ScalarType.bfloat16, acc.ScalarType.bfloat16, acc.Layout.LAST_MAJOR)
    big_plan = big_nest.create_schedule().create_plan(acc.Target(acc.Target.Model.NVIDIA_B200))
    big_plan.tensorize(indices=tuple(big_nest.get_indices()), mma_shape=acc.MMAShape.M16xN16xK16_B1)
    big = pkg.add(big_plan, args=big_args, base_name="mm_big")
    hf = hat.HATFile.read(pkg.build("gpu_pkg", output_dir=str(tmp_path))[0])
    host = hf.function_map[fn.name]
    assert host.launches is None and host.runtime is None and host.calling_convention == "cdecl"
    assert hf.device_functions == [] and hf.device_function_map == {}
    meta = host.auxiliary["accera_b200"]
    assert meta["device_function"] == fn.name + "__gpu__" and meta["runtime"] == "CUDA" and meta["kernel"] == "gemm_umma_kernel"
    want = runtime.gemm_launch_geometry(512, 512, 512, in_type="float16", compute="tensor_preferred")
    # a short K loop: the launch with eight epilogue warps (320 threads); the long one below keeps four (192)
    assert meta["launch_parameters"] == want["grid"] + want["block"] and meta["launch_parameters"][3:] == [320, 1, 1]
    assert meta["dynamic_shared_mem_bytes"] == want["dynamic_shared_mem_bytes"] > 190000
    # the geometry is the variant's own: 16 single-CTA tiles of 128 columns here, 74 CTA pairs on the big problem
    assert meta["launch_parameters"][0] == 16 and meta["tile_cols"] == 128 and meta["cta_pairs"] is False
    bmeta = hf.function_map[big.name].auxiliary["accera_b200"]
    assert bmeta["launch_parameters"] == [148, 1, 1, 192, 1, 1] and bmeta["cta_pairs"] is True and bmeta["tile_cols"] == 256
    assert bmeta["tiles"] == 8192
    assert hf.target.required.gpu.model == "NVidia B200" and hf.target.required.gpu.runtime == "CUDA"
    _, fns = hat.load(hf.path)
    assert fns.names == [fn.name, big.name]


def test_plan_bind_gives_the_reference_launch_geometry_and_rejects_what_it_rejects():
    # the 4096^3 schedule with 64 x 64 block tiles and 16 x 16 warp tiles: grid 64 x 64, 16 warps (lang/Plan.py:879-956)
    t = acc.Target(acc.Target.Model.NVIDIA_B200)

    def build(block_tile, warp_tile, m=4096):
        nest, args = _gemm_nest(m, m, m, acc.ScalarType.float16, acc.ScalarType.float32)
        i, j, k = nest.get_indices()
        s = nest.create_schedule()
        ii, jj, kk = s.tile({i: block_tile, j: block_tile, k: 64})
        iii, jjj, kkk = s.tile({ii: warp_tile, jj: warp_tile, kk: 16})
        plan, tix = s._create_tensorizable_plan(t, block_indices=(i, j), warp_indices=(ii, jj), tensor_indices=(iii, jjj, kkk),
                                                outer_nest_order=(i, j, k, ii, jj, kk))
        plan.tensorize(indices=tix, mma_shape=acc.MMAShape.M16xN16xK16_B1)
        return plan, args
    plan, args = build(64, 16)
    assert plan.launch_request() == ([128, 4, 1], [64, 64, 1])
    pkg = acc.Package()
    fn = pkg.add(plan, args=args, base_name="bound")
    assert fn.launch_request == ([128, 4, 1], [64, 64, 1])
    # 256 x 256 block tiles of 16 x 16 warp tiles: 16 x 16 warps = 8192 threads
    bad, bad_args = build(256, 16)
    with pytest.raises(ValueError, match="Invalid block size"):
        acc.Package().add(bad, args=bad_args, base_name="too_big")
    # thread bindings beyond the per-dimension limit
    nest, args2 = _gemm_nest(4096, 4096, 64, acc.ScalarType.float32, acc.ScalarType.float32)
    i, j, k = nest.get_indices()
    s = nest.create_schedule()
    ii = s.split(i, 2048)
    p2 = s.create_plan(t)
    p2.bind({i: t.GridUnit.BLOCK_X, ii: t.GridUnit.THREAD_X})
    with pytest.raises(ValueError, match="Invalid block dimensions"):
        acc.Package().add(p2, args=args2, base_name="too_wide")
    # no bindings: 16 x 16 blocks following the split factors (lang/Plan.py:938-954)
    nest3, _ = _gemm_nest(512, 256, 64, acc.ScalarType.float32, acc.ScalarType.float32)
    i3, j3, k3 = nest3.get_indices()
    s3 = nest3.create_schedule()
    s3.split(i3, 32)
    assert s3.create_plan(t).launch_request() == ([32, 16, 1], [16, 16, 1])
    # CPU plans cannot be bound (lang/Plan.py:824-825)
    with pytest.raises(ValueError, match="Only supported on plans with GPU targets"):
        nest3.create_schedule().create_plan().bind({i3: t.GridUnit.BLOCK_X})


def _batch_matmul_plan(batch, M, N, K, dtype=None, out_dtype=None, layouts=None, tensorize=True, epilogue_op=None):
    """The reference's batch matmul test nest and schedule (mfma_tests.py:435-499), on static shapes."""
    dtype = dtype or acc.ScalarType.float32
    out_dtype = out_dtype or dtype
    layouts = layouts or [acc.Layout.FIRST_MAJOR] * 3
    A = acc.Array(role=acc.Role.INPUT, element_type=dtype, shape=(batch, M, K), layout=layouts[0])
    B = acc.Array(role=acc.Role.INPUT, element_type=dtype, shape=(batch, K, N), layout=layouts[1])
    C = acc.Array(role=acc.Role.INPUT_OUTPUT, element_type=out_dtype, shape=(batch, M, N), layout=layouts[2])
    nest = acc.Nest(shape=(batch, M, N, K))
    b, i, j, k = nest.get_indices()

    @nest.iteration_logic
    def _():
        C[b, i, j] += A[b, i, k] * B[b, k, j]

    schedule = nest.create_schedule()
    ii, jj, kk = schedule.tile({i: 64, j: 64, k: 64})
    target = acc.Target(acc.Target.Model.NVIDIA_B200)
    if not tensorize:
        return schedule.create_plan(target), (A, B, C)
    shape = acc.MMAShape.M16xN16xK16_B1
    splits = target.tensor_core_info.compute_tensor_splits(shape, 1)
    iii, jjj, kkk = schedule.tile({ii: splits[0], jj: splits[1], kk: splits[2]})
    plan, tensor_indices = schedule._create_tensorizable_plan(
        target, block_indices=(i, j), warp_indices=(ii, jj), tensor_indices=(iii, jjj, kkk),
        outer_nest_order=(b, i, j, k, ii, jj, kk))
    kw = {"epilogue_op": epilogue_op} if epilogue_op is not None else {}
    plan.tensorize(indices=tensor_indices, mma_shape=shape, **kw)
    plan.cache(A, index=ii, location=target.MemorySpace.SHARED)
    plan.cache(C, index=k, location=target.MemorySpace.MMA_FRAGMENT)
    return plan, (A, B, C)


def test_tensor_core_shape_helpers():
    info = acc.Target(acc.Target.Model.NVIDIA_B200).tensor_core_info
    assert info.mma_shape_to_tuple(acc.MMAShape.M16xN16xK16_B1) == (16, 16, 16)
    assert info.mma_shape_to_tuple(acc.MMAShape.M64xN64xK1_B4) == (64, 64, 1)
    assert info.mma_shape_to_tuple(acc.MMAShape.M32xN8xK16_B1) == (32, 8, 16)
    assert info.compute_tensor_splits(acc.MMAShape.M16xN16xK4_B1, 4) == (16, 16, 16)


def test_recognise_batch_matmul(tmp_path):
    plan, (A, B, C) = _batch_matmul_plan(3, 128, 192, 256, acc.ScalarType.float16, acc.ScalarType.float32,
                                         epilogue_op=acc.MMAFragmentOp.ReLU)
    spec = patterns.recognise(plan)
    assert spec.kind == "gemm" and spec.batch == 3 and (spec.m, spec.n, spec.k) == (128, 192, 256)
    assert spec.a is A and spec.b is B and spec.c is C and spec.compute == "tensor" and spec.relu
    assert spec.a_pos == (0, 1, 2) and spec.b_pos == (0, 1, 2) and spec.c_pos == (0, 1, 2)
    pkg = acc.Package()
    fn = pkg.add(plan, args=(A, B, C), base_name="bmm")
    src = pkg._stub_source("bmm_pkg")
    assert "accb_gemm_batched(&d, INT64_C(3), INT64_C(32768), INT64_C(49152), INT64_C(24576), a0, a1, a2, nullptr)" in src
    assert "d.a_stride[0] = INT64_C(256); d.a_stride[1] = INT64_C(1);" in src
    assert "d.b_stride[0] = INT64_C(192); d.b_stride[1] = INT64_C(1);" in src
    assert "d.epilogue = ACCB_EPI_RELU" in src and "ACCB_COMPUTE_TENSOR_PREFERRED" in src
    hat_path, lib_path = pkg.build("bmm_pkg", output_dir=str(tmp_path))[:2]
    hf = hat.HATFile.read(hat_path)
    f = hf.functions[0]
    assert f.name == fn.name and [a.shape for a in f.arguments] == [[3, 128, 256], [3, 256, 192], [3, 128, 192]]
    assert f.arguments[1].affine_map == [256 * 192, 192, 1]
    lib = ctypes.CDLL(lib_path)
    assert hasattr(lib, fn.name)


def test_batch_matmul_layouts_and_shared_operand():
    # last-major arrays: element (b, i, k) of A is at b + batch * (i + M * k)
    plan, (A, B, C) = _batch_matmul_plan(4, 64, 64, 128, layouts=[acc.Layout.LAST_MAJOR, acc.Layout.FIRST_MAJOR,
                                                                   acc.Layout.FIRST_MAJOR], tensorize=False)
    pkg = acc.Package()
    pkg.add(plan, args=(A, B, C), base_name="bmm_lm")
    src = pkg._stub_source("p")
    assert "d.a_stride[0] = INT64_C(4); d.a_stride[1] = INT64_C(256);" in src
    assert "accb_gemm_batched(&d, INT64_C(4), INT64_C(1), INT64_C(8192), INT64_C(4096)" in src
    assert "ACCB_COMPUTE_SIMT" in src                   # plain fp32 nest: true fp32 arithmetic

    # B without the batch index is shared by all problems (batch stride 0); A indexed [b, k, i] is transposed
    A = acc.Array(role=acc.Role.INPUT, element_type=acc.ScalarType.float16, shape=(5, 96, 32))
    B = acc.Array(role=acc.Role.INPUT, element_type=acc.ScalarType.float16, shape=(96, 48))
    C = acc.Array(role=acc.Role.INPUT_OUTPUT, element_type=acc.ScalarType.float16, shape=(5, 32, 48))
    nest = acc.Nest(shape=(5, 32, 48, 96))
    b, i, j, k = nest.get_indices()

    @nest.iteration_logic
    def _():
        C[b, i, j] += A[b, k, i] * B[k, j]

    spec = patterns.recognise(nest)
    assert spec.batch == 5 and spec.a_pos == (0, 2, 1) and spec.b_pos == (None, 0, 1)
    pkg = acc.Package()
    pkg.add(nest, args=(A, B, C), base_name="bmm_shared")
    src = pkg._stub_source("p")
    assert "d.a_stride[0] = INT64_C(1); d.a_stride[1] = INT64_C(32);" in src
    assert "accb_gemm_batched(&d, INT64_C(5), INT64_C(3072), INT64_C(0), INT64_C(1536)" in src

    # neither operand carries the batch index: not a batch matmul
    nest2 = acc.Nest(shape=(5, 32, 48, 96))
    b, i, j, k = nest2.get_indices()
    A2 = acc.Array(role=acc.Role.INPUT, element_type=acc.ScalarType.float16, shape=(32, 96))

    @nest2.iteration_logic
    def _():
        C[b, i, j] += A2[i, k] * B[k, j]

    with pytest.raises(patterns.UnsupportedNestError):
        patterns.recognise(nest2)


def test_reader_accepts_the_reference_emitters_formatting(tmp_path):
    """A function table laid out the way the reference's emitter prints it (the sample in
    docs/Tutorials/Optimized_MatMul.md:176-187: single-quoted names, double-quoted enumerations, padded
    arrays `[ 784, 128 ]`, an inline `return` table, unnamed arguments, an 8-hex-digit name suffix) inside
    the header / TOML guard structure of HATEmitter.h:1197-1265, read back with this package's reader."""
    text = """#pragma once
#ifndef __sample_pkg__
#define __sample_pkg__

#ifdef TOML

[description]
comment = ''
author = ''
version = ''
license_url = ''

[functions]

[functions.tiled_mm_py_0badc0de]
name = 'tiled_mm_py_0badc0de'
description = ''
calling_convention = "cdecl"
arguments = [
    {name = '', description = '', logical_type = "affine_array", declared_type = 'float*', element_type = 'float', usage = "input_output", shape = [ 784, 128 ], affine_map = [ 128, 1 ], affine_offset = 0},
    {name = '', description = '', logical_type = "affine_array", declared_type = 'float*', element_type = 'float', usage = "input_output", shape = [ 128, 512 ], affine_map = [ 512, 1 ], affine_offset = 0},
    {name = '', description = '', logical_type = "affine_array", declared_type = 'float*', element_type = 'float', usage = "input_output", shape = [ 784, 512 ], affine_map = [ 512, 1 ], affine_offset = 0}
]
return = {name = '', description = '', logical_type = "void", declared_type = 'void', element_type = 'void', usage = "output"}

[target]

[target.required]
os = "linux"

[target.required.CPU]
architecture = "x86_64"
extensions = [ "AVX2", "FMA3" ]

[dependencies]
link_target = "sample_pkg.a"
deploy_files = [  ]
dynamic = [  ]

[compiled_with]
compiler = ''
flags = ''
crt = ''
libraries = [  ]

[declaration]
code = '''
#endif // TOML

#if defined(__cplusplus)
extern "C"
{
#endif // defined(__cplusplus)

void tiled_mm_py_0badc0de(float*, float*, float*);

#ifndef __tiled_mm_py_DEFINED__
#define __tiled_mm_py_DEFINED__
void (*tiled_mm_py)(float*, float*, float*) = tiled_mm_py_0badc0de;
#endif

#if defined(__cplusplus)
} // extern "C"
#endif // defined(__cplusplus)

#ifdef TOML
'''

#endif // TOML

#endif // __sample_pkg__
"""
    path = tmp_path / "sample_pkg.hat"
    path.write_text(text)
    hf = hat.HATFile.read(str(path))
    assert hf.name == "sample_pkg" and [f.name for f in hf.functions] == ["tiled_mm_py_0badc0de"]
    f = hf.functions[0]
    assert f.calling_convention == "cdecl" and f.return_info.logical_type == "void"
    assert [a.shape for a in f.arguments] == [[784, 128], [128, 512], [784, 512]]
    assert [a.affine_map for a in f.arguments] == [[128, 1], [512, 1], [512, 1]]
    assert all(a.usage == "input_output" and a.declared_type == "float*" and a.element_type == "float" for a in f.arguments)
    assert f.c_declaration().replace(" ", "") == "voidtiled_mm_py_0badc0de(float*,float*,float*);"
    assert hf.dependencies["link_target"] == "sample_pkg.a" and hf.target["required"]["CPU"]["extensions"] == ["AVX2", "FMA3"]
    assert "void (*tiled_mm_py)(float*, float*, float*) = tiled_mm_py_0badc0de;" in hf.declaration_code
    # the C side of the same file: a compiler sees only the declarations
    src = tmp_path / "client.c"
    src.write_text('#include "sample_pkg.hat"\nint main(void) { return tiled_mm_py == 0; }\n'
                   'void tiled_mm_py_0badc0de(float* a, float* b, float* c) { (void)a; (void)b; (void)c; }\n')
    subprocess.run(["gcc", "-c", str(src), "-o", str(tmp_path / "client.o")], check=True)
    # and it survives a rewrite by this package's writer
    out = tmp_path / "rewritten.hat"
    hf.write(str(out))
    again = hat.HATFile.read(str(out))
    assert again.functions[0].arguments == f.arguments and again.dependencies == hf.dependencies


def test_gemm_tile_plan_is_host_only_and_follows_the_cost_model():
    runtime.set_option("reset", 0)
    plan = runtime.gemm_tile_plan
    # the benchmark problem: 256 x 256 pair tiles, 8192 of them on 74 pairs
    assert plan(65536, 8192, 8192) == {"cta_pairs": True, "tile_cols": 256, "tiles": 8192, "rounds": 111}
    assert plan(4096, 4096, 4096)["rounds"] == 4 and plan(4096, 4096, 4096)["tile_cols"] == 256
    # too small to give every SM a 256-column tile: single CTAs, 128 columns
    assert plan(1024, 1024, 1024) == {"cta_pairs": False, "tile_cols": 128, "tiles": 64, "rounds": 1}
    assert plan(256, 256, 256)["tile_cols"] == 128
    # the compute mode fixes the CTA mode; the width is still chosen
    assert plan(4096, 4096, 4096, compute="tensor") == {"cta_pairs": False, "tile_cols": 256, "tiles": 512, "rounds": 4}
    assert plan(1024, 1024, 1024, compute="tensor_2sm")["cta_pairs"] is True
    # 8-bit operands with a row-major B cannot use 128-column pair tiles (a 64-column share is narrower than a box)
    assert plan(1024, 1024, 1024, in_type="int8", b_row_major=True, compute="tensor_2sm")["tile_cols"] == 256
    # a batch multiplies the tiles; fewer SMs or a capped grid lengthen the rounds
    assert plan(1024, 1024, 1024, batch=64) == {"cta_pairs": True, "tile_cols": 256, "tiles": 1024, "rounds": 14}
    assert plan(8192, 8192, 8192, num_sms=132)["rounds"] == 16 and plan(8192, 8192, 8192, max_ctas=64)["rounds"] == 32
    with pytest.raises(runtime.AccbError):
        plan(0, 8, 8)


def test_device_side_failures_are_attributed_to_the_launch_that_had_them():
    # the status words a kernel writes, decoded as the library does (no GPU involved).  Words: [0] gather count,
    # [1] GEMM site << 24 | block, [2] step, [3] id of the failing GEMM launch, [4] waits that ran out, [5] id of the
    # gather launch that met a bad index.
    ALL, GEMM, GATHER = 0, 1, 2
    timeout = [0, (4 << 24) | 3, 7, 55, 2, 0, 0, 0]
    code, msg = runtime.decode_status(timeout, GEMM, 55)
    assert code == runtime.ERR_TIMEOUT and "epilogue waiting for the accumulator" in msg and "block 3, step 7" in msg and "launch 55" in msg
    assert runtime.decode_status(timeout, GEMM, 56) == (0, "")          # a later GEMM call does not inherit it
    assert runtime.decode_status(timeout, GATHER, 56) == (0, "")        # nor does a gather
    assert runtime.decode_status(timeout, ALL, 0)[0] == runtime.ERR_TIMEOUT   # accb_synchronize reports it
    code, msg = runtime.decode_status([0, (5 << 24) | 140, 12, 9, 1, 0, 0, 0], ALL)
    assert code == runtime.ERR_TIMEOUT and "forwarding CTA waiting for a tile" in msg
    bad_index = [3, 0, 0, 0, 0, 9, 0, 0]
    assert runtime.decode_status(bad_index, GEMM, 10) == (0, "")        # a host-pointer GEMM is not blamed for an old gather
    assert runtime.decode_status(bad_index, GATHER, 10) == (0, "")      # nor a later, clean gather
    code, msg = runtime.decode_status(bad_index, GATHER, 9)
    assert code == runtime.ERR_INDEX and "3 index value(s)" in msg
    assert runtime.decode_status(bad_index, ALL)[0] == runtime.ERR_INDEX
    assert runtime.decode_status([0] * 8, ALL) == (0, "")
    # both recorded: the time-out is reported first, the index error stays for the next collection
    both = [2, (1 << 24), 0, 4, 1, 6, 0, 0]
    assert runtime.decode_status(both, ALL)[0] == runtime.ERR_TIMEOUT


def test_options_are_validated_and_reset():
    runtime.set_option("reset", 0)
    assert runtime.gemm_tile_plan(4096, 4096, 4096)["tile_cols"] == 256
    with runtime.options(**{"gemm.tile_cols": 128}):
        assert runtime.gemm_tile_plan(4096, 4096, 4096)["tile_cols"] == 128
    assert runtime.gemm_tile_plan(4096, 4096, 4096)["tile_cols"] == 256
    for name, value in (("gemm.tile_cols", 192), ("gemm.pace_pct", 101), ("gemm.copy_ctas", 500), ("no.such.option", 1),
                        ("gemm.wait_limit_us", -5), ("host_gemm.stage_chunks", 1000)):
        with pytest.raises(runtime.AccbError):
            runtime.set_option(name, value)
    assert runtime.selected_device() == -1


def test_launch_geometry_follows_the_epilogue_the_launch_will_use():
    """accb_gemm_launch_geometry reports the block the launch code really uses: 320 threads (eight epilogue warps) where
    the K loop is short enough for the epilogue to show - up to 32 slabs of 128 bytes, or 64 when every CTA has one
    tile - and 192 otherwise."""
    runtime.set_option("reset", 0)
    g = runtime.gemm_launch_geometry
    assert g(1024, 1024, 1024)["block"] == [320, 1, 1]             # 16 slabs
    assert g(4096, 4096, 2048)["block"] == [320, 1, 1]             # 32 slabs, several tiles per CTA
    assert g(4096, 4096, 4096)["block"] == [192, 1, 1]             # 64 slabs, 3.5 rounds of tiles
    assert g(1024, 4096, 4096)["block"] == [320, 1, 1]             # 64 slabs, one tile per CTA pair
    assert g(65536, 8192, 8192)["block"] == [192, 1, 1]            # the benchmark's launch
    assert g(8192, 8192, 8192, in_type="int8")["block"] == [192, 1, 1]     # 64 slabs of 128 int8, 14 rounds
    assert g(2048, 2048, 2048, in_type="int8")["block"] == [320, 1, 1]     # 16 slabs
    assert g(1024, 1000, 1024)["block"] == [320, 1, 1]             # rows of 2000 bytes end on a 16-byte boundary
    assert g(1024, 1004, 1024)["block"] == [192, 1, 1]             # rows of 2008 bytes do not: TMA-stored boxes
    for name, value in (("gemm.epi_warps", 4), ("gemm.epi_warps", 8), ("gemm.split_k", 0), ("gemm.split_k", 4), ("gemm.c_in", 0),
                        ("gemm.staged_store", 2), ("stream_kernels.pdl", 0)):
        runtime.set_option(name, value)                              # accepted
    runtime.set_option("reset", 0)
