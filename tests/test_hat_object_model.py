"""The object model the reference drives `.hat` files through, replayed on CPU.

The reference does not parse `.hat` files itself: it calls the third-party hatlib (hatlib==0.0.39; not part of
the reference tree, not installable here, so nothing below is checked against hatlib itself).  These tests replay
the reference's own statements - the post-processing in accera/python/accera/Package.py:678-784 and the assertions
of accera/python/accera/test/dsl_tests.py:5787-5842 and 6398-6449 - against accera_b200.hat, with `hat` standing
where the reference says `hat` / `hatlib`.
"""
import os
import pathlib
import shutil
import subprocess

import pytest

import accera_b200 as acc
from accera_b200 import hat

from test_host_layer import quickstart_package


def _object_package(tmp_path, name="pkg", prefix=""):
    """A .hat as the reference's C++ layer leaves it (function tables + declarations) beside a compiled object file."""
    src = tmp_path / f"{name}.cpp"
    src.write_text('#include <cstdint>\nextern "C" void f_0123(float* a, float* b) { b[0] = a[0] + 1.0f; }\n'
                   'extern "C" void g_4567(int64_t n, int64_t* out) { *out = n * 2; }\n'.replace("f_0123", prefix + "f_0123")
                   .replace("g_4567", prefix + "g_4567"))
    subprocess.run(["g++", "-O1", "-fPIC", "-c", str(src), "-o", str(tmp_path / f"{name}.o")], check=True)
    hf = hat.HATFile(name=name)
    arr = hat.Parameter(logical_type="affine_array", declared_type="float*", element_type="float", usage="input_output",
                        shape=[4], affine_map=[1], affine_offset=0)
    hf.function_map[prefix + "f_0123"] = hat.Function(name=prefix + "f_0123", arguments=[arr, arr])
    hf.function_map[prefix + "g_4567"] = hat.Function(name=prefix + "g_4567", arguments=[
        hat.Parameter(name="n", logical_type="element", declared_type="int64_t", element_type="int64_t", usage="input"),
        hat.Parameter(name="out", logical_type="element", declared_type="int64_t*", element_type="int64_t", usage="output")])
    hf.declaration.code = f"void {prefix}f_0123(float*, float*);\nvoid {prefix}g_4567(int64_t, int64_t*);\n"
    path = tmp_path / f"{name}.hat"
    hf.Serialize(str(path))
    return path


def test_reference_post_processing_statements_run_unchanged(tmp_path):
    """Package.py:678-764, statement by statement."""
    header_path = _object_package(tmp_path, "main")
    support_path = _object_package(tmp_path, "support", prefix="s_")
    output_dir = str(tmp_path)

    hat_file = hat.HATFile.Deserialize(header_path)                                   # :678
    hat_file.dependencies.link_target = os.path.basename(str(tmp_path / "main.o"))    # :681

    supporting_hats = map(hat.HATFile.Deserialize, [support_path])                    # :683
    supporting_objs = []
    supporting_decls = []
    for support in supporting_hats:                                                   # :686-699
        path = os.path
        support.dependencies.link_target = "support.o"
        dependency_path = path.abspath(path.join(output_dir, support.dependencies.link_target))
        supporting_objs.append(hat.LibraryReference(target_file=dependency_path))
        supporting_decls.append(support.declaration.code)
        hat_file._function_table.function_map.update(support._function_table.function_map)         # :699

    dynamic_dependencies = []
    decl_code = hat_file.declaration.code                                             # :700
    hat_file.dependencies.dynamic = dynamic_dependencies + supporting_objs             # :701
    hat_file.declaration.code = decl_code._new("\n".join(map(str, ["", decl_code] + supporting_decls)))   # :702

    hat_func = hat_file.function_map.get("f_0123")                                    # :708
    assert hat_func is not None and hat_file.function_map.get("nope") is None
    hat_func.auxiliary = {"accera": {"parameters": {"P0": 8}}}                        # :712

    gpu_device_func = "f_0123" + "__gpu__"                                            # :717
    hat_target = hat_file.target                                                      # :726
    hat_target.required.gpu.runtime = "CUDA"                                          # :727
    hat_target.required.gpu.model = "NVidia B200"                                     # :728
    hat_func.runtime = "CUDA"                                                         # :730
    hat_func.launches = gpu_device_func                                               # :731
    hat_file.device_function_map[gpu_device_func] = hat.Function(                     # :733-743
        name=gpu_device_func,
        description=f"Device function launched by f_0123",
        calling_convention=hat.CallingConventionType.Device,
        arguments=hat_func.arguments,
        return_info=hat_func.return_info,
        launch_parameters=[64, 64, 1, 128, 4, 1],
        dynamic_shared_mem_bytes=0,
        provider="main.cu",
        runtime="CUDA",
    )

    hat_os = hat.OperatingSystem.Linux                                                # :745-750
    hat_file.target.required.os = hat_os                                              # :751
    hat_file.target.required.cpu.architecture = "x86_64"                              # :752
    hat_file.target.required.cpu.extensions = "AVX2,FMA3".split(",")                  # :756

    description = {"author": "Microsoft Research", "version": "2.0", "license": "https://mit-license.org",
                   "auxiliary": {"Dependencies": ["numpy"]}}
    hat_file.description.author = description.get("author", "")                       # :758
    hat_file.description.version = description.get("version", "")                     # :759
    hat_file.description.license_url = description.get("license", "")                 # :760
    if "auxiliary" in description:
        hat_file.description.auxiliary = description["auxiliary"]                     # :762

    hat_file.Serialize(header_path)                                                   # :764

    # what was written is what was said, in the emitter's key spelling
    back = hat.HATFile.Deserialize(header_path)
    assert back.dependencies.link_target == "main.o"
    assert back.dependencies.dynamic == [{"name": "", "version": "", "target_file": str(tmp_path / "support.o")}]
    assert back.dependencies.dynamic[0].target_file.endswith("support.o")
    assert "void f_0123(float*, float*);" in back.declaration.code and back.declaration.code.count("g_4567") == 2
    assert set(back.function_map) == {"f_0123", "g_4567", "s_f_0123", "s_g_4567"}
    f = back.function_map["f_0123"]
    assert f.auxiliary == {"accera": {"parameters": {"P0": 8}}} and f.launches == gpu_device_func and f.runtime == "CUDA"
    dev = back.device_function_map[gpu_device_func]
    assert dev.calling_convention == hat.CallingConventionType.Device == "device"
    assert dev.launch_parameters == [64, 64, 1, 128, 4, 1] and dev.provider == "main.cu" and dev.arguments == f.arguments
    assert back.target.required.os == hat.OperatingSystem.Linux == "linux"
    assert back.target["required"]["CPU"] == {"architecture": "x86_64", "extensions": ["AVX2", "FMA3"]}
    assert back.target.required.gpu.runtime == "CUDA" and back.target["required"]["GPU"]["model"] == "NVidia B200"
    assert back.description.author == "Microsoft Research" and back.description.license_url == "https://mit-license.org"
    text = pathlib.Path(header_path).read_text()
    assert "[target.required.CPU]" in text and "[target.required.GPU]" in text and 'calling_convention = "device"' in text
    # the file is still a C header
    client = tmp_path / "client.c"
    client.write_text(f'#include <stdint.h>\n#include "main.hat"\nint main(void) {{ return 0; }}\n')
    subprocess.run(["gcc", "-c", str(client), "-I", str(tmp_path), "-o", str(tmp_path / "client.o")], check=True)


def test_static_and_dynamic_packaging_steps(tmp_path):
    """Package.py:766-784: create_static_package / create_dynamic_package, the auxiliary entry, the move."""
    header_path = str(_object_package(tmp_path, "P"))
    path_root = os.path.join(str(tmp_path), "P")
    extension = ".hat"
    hat_file = hat.HATFile.Deserialize(header_path)
    hat_file.dependencies.link_target = "P.o"
    hat_file.Serialize(header_path)

    lib_hat_path = f"{path_root}_lib{extension}"                                      # :767
    hat.create_static_package(header_path, lib_hat_path)                              # :768
    lib_hat_file = hat_file.Deserialize(lib_hat_path)                                 # :770 (called on an instance)
    lib_hat_file.dependencies.auxiliary["static"] = lib_hat_file.dependencies.link_target   # :771
    lib_hat_file.Serialize()                                                          # :772 (no path: back to its own file)
    assert lib_hat_file.dependencies.link_target == "P_lib.a" and os.path.exists(f"{path_root}_lib.a")
    members = subprocess.run(["ar", "t", f"{path_root}_lib.a"], capture_output=True, text=True, check=True).stdout.split()
    assert members == ["P.o"]

    dyn_hat_path = f"{path_root}_dyn{extension}"                                      # :777
    hat.create_dynamic_package(header_path, dyn_hat_path)                             # :778
    dyn_hat_file = hat_file.Deserialize(dyn_hat_path)                                 # :780
    dyn_hat_file.dependencies.auxiliary["dynamic"] = dyn_hat_file.dependencies.link_target   # :781
    dyn_hat_file.Serialize()                                                          # :782
    shutil.move(dyn_hat_path, header_path)                                            # :784
    final = hat.HATFile.Deserialize(header_path)
    assert final.dependencies.link_target == "P_dyn.so" and final.dependencies.auxiliary == {"dynamic": "P_dyn.so"}
    # the dynamic package loads and its functions run (plain host code in this fixture)
    import numpy as np
    _, fns = hat.load(header_path)
    a, b = np.array([1, 2, 3, 4], np.float32), np.zeros(4, np.float32)
    fns["f_0123"](a, b)
    assert b[0] == 2.0
    out = np.zeros(1, np.int64)
    fns["g_4567"](21, out)
    assert out[0] == 42
    # an input whose link target is not an object file is refused
    with pytest.raises(ValueError):
        hat.create_static_package(header_path, f"{path_root}_again.hat")


def test_add_description_round_trip_as_the_reference_checks_it(tmp_path):
    """dsl_tests.py:6398-6449 (test_add_description), with this package's DSL in place of accera."""
    package = quickstart_package()
    description1 = {
        "Dependencies": ["numpy", "onnx", "scipy"],
        "Documentation": "https://docs.readthedocs.io.",
        "SHA": "0bb913ce84afa28127ea3fd2a9995e219dad322a",
    }
    package.add_description(other=description1, version="1.0", author="Microsoft Research", license="https://mit-license.org")
    description2 = {
        "Documentation": "",    # clearing a value
        "SHA": None,    # removing a value
        "Release Notes": "https://stackoverflow.com",    # adding an entry
    }
    package.add_description(other=description2)
    package.add_description(version="2.0")
    package.build("MyPackage", format=acc.Package.Format.HAT_DYNAMIC, output_dir=str(tmp_path))

    hat_file = hat.HATFile.Deserialize(pathlib.Path(tmp_path) / "MyPackage.hat")
    hat_description = hat_file.description.auxiliary
    assert hat_description["Dependencies"] == description1["Dependencies"]
    assert hat_description["Documentation"] == description2["Documentation"]
    assert "SHA" not in hat_description
    assert hat_description["Release Notes"] == description2["Release Notes"]
    assert hat_file.description.version == "2.0"
    assert hat_file.description.author == "Microsoft Research"
    assert hat_file.description.license_url == "https://mit-license.org"


def test_parameter_auxiliary_data_as_the_reference_reads_it(tmp_path):
    """dsl_tests.py:5787-5842 (test_parameterization_auxiliary_data): HATPackage(path).get_functions()[i]
    .auxiliary["accera"]["parameters"].  Parameter grids are expanded by the caller here (one add per point)."""
    package = acc.Package()
    grid = [(p0, p1, p3) for p0 in (8, 16) for p1 in (16, 32) for p3 in (1.0, 2.0)]
    for p0, p1, p3 in grid:
        A = acc.Array(role=acc.Role.INPUT, element_type=acc.ScalarType.float32, shape=(p0, 16))
        B = acc.Array(role=acc.Role.INPUT, element_type=acc.ScalarType.float32, shape=(16, p1))
        C = acc.Array(role=acc.Role.INPUT_OUTPUT, element_type=acc.ScalarType.float32, shape=(p0, p1))
        nest = acc.Nest(shape=(p0, p1, 16))
        i, j, k = nest.get_indices()

        @nest.iteration_logic
        def _():
            C[i, j] += A[i, k] * B[k, j]
        package.add(nest, args=(A, B, C), base_name="matmul", parameters={"P0": p0, "P1": p1, "P2": 16, "P3": p3})
    package_name = "test_parameterization_auxiliary_data"
    package.build(name=package_name, format=acc.Package.Format.HAT_DYNAMIC, output_dir=str(tmp_path))

    hat_package = hat.HATPackage(pathlib.Path(tmp_path) / f"{package_name}.hat")
    functions = [fn for fn in hat_package.get_functions()]
    assert len(functions) == len(grid)
    for function in functions:
        data_point = function.auxiliary["accera"]["parameters"]
        assert data_point
        assert int(data_point["P0"]) in [8, 16]
        assert int(data_point["P1"]) in [16, 32]
        assert int(data_point["P2"]) in [16]
        assert float(data_point["P3"]) in [1.0, 2.0]


def test_built_packages_follow_the_reference_build_order(tmp_path):
    """Package.build goes through the same steps as the reference: object file + header, post-processing, then
    create_*_package, the auxiliary entry and the move over the original .hat (Package.py:669-784)."""
    files = quickstart_package().build("both", format=acc.Package.Format.HAT_DYNAMIC | acc.Package.Format.STATIC_LIBRARY,
                                       output_dir=str(tmp_path))
    assert sorted(os.path.basename(f) for f in files) == ["both.a", "both.hat", "both.so"]
    assert sorted(os.listdir(tmp_path)) == ["both.a", "both.hat", "both.so"]          # no _lib / _dyn / .o left behind
    hf = hat.HATFile.Deserialize(files[0])
    assert hf.dependencies.link_target == "both.so"
    assert hf.dependencies.auxiliary == {"dynamic": "both.so", "static": "both.a"}
    assert [d.target_file for d in hf.dependencies.dynamic] == ["libaccera_b200.so"]
    assert hf.target.required.os == hat.OperatingSystem.host() and hf.target.required.gpu.instruction_set_version == "sm_100a"
    for f in hf.functions:
        assert f.launches is None and f.auxiliary["accera"] == {"parameters": {}}
    only_static = quickstart_package().build("st", format=acc.Package.Format.HAT_STATIC, output_dir=str(tmp_path / "s"))
    hs = hat.HATFile.Deserialize(only_static[0])
    assert hs.dependencies.link_target == "st.a" and hs.dependencies.auxiliary == {"static": "st.a"}
