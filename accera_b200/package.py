"""`Package`: collects functions and builds a HAT package whose functions run on the B200 kernels.

Mirrors accera/python/accera/Package.py: `add` (:203-432, naming by md5 :310-335, dynamic-size
references :337-360, single-target rule :302-308), `build` (:551-788, format resolution :592-603,
HAT post-processing :672-784).  What differs is what happens between add and the artefacts: instead
of emitting MLIR and driving acc-opt / acc-translate / llc, `build` writes one small C++ stub per
function that forwards into libaccera_b200.so (the C ABI over the hand-written sm_100a kernels),
compiles the stubs with the host C++ compiler and writes the `.hat` descriptor beside the library.

Artefacts of `build("P", format=HAT_DYNAMIC)`:  P.hat, P.so   (P.so depends on libaccera_b200.so)
            `build("P", format=HAT_STATIC)`:   P.hat, P.a    (link with libaccera_b200.so)
            `| Format.SOURCE`:                 P.cpp (the stub source) is kept
"""
from __future__ import annotations

import enum
import hashlib
import json
import os
import platform as _platform
import secrets
import shutil
import subprocess
from collections import OrderedDict
from typing import Any, Dict, List, Optional, Sequence, Tuple

from . import lang, patterns
from .hat import hat_file
from .lang import Array, Dimension, Role, Scalar, ScalarType, Target

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
_INCLUDE_DIR = os.path.join(os.path.dirname(_PKG_DIR), "include")

_ACCB_TYPE = {ScalarType.float32: "ACCB_F32", ScalarType.float16: "ACCB_F16", ScalarType.bfloat16: "ACCB_BF16",
              ScalarType.int8: "ACCB_S8", ScalarType.int32: "ACCB_S32", ScalarType.uint8: "ACCB_U8"}
_COMPUTE = {"auto": "ACCB_COMPUTE_AUTO", "simt": "ACCB_COMPUTE_SIMT", "tensor": "ACCB_COMPUTE_TENSOR_PREFERRED"}


class _PackagedFunction:
    def __init__(self, name, base_name, spec, args, target, auxiliary):
        self.name = name
        self.base_name = base_name
        self.spec = spec
        self.args = list(args)
        self.target = target
        self.auxiliary = auxiliary


class Package:
    "A package of functions that can be built and linked with client code."

    class Format(enum.Flag):
        DYNAMIC_LIBRARY = enum.auto()
        STATIC_LIBRARY = enum.auto()
        HAT_PACKAGE = enum.auto()
        MLIR = enum.auto()
        MLIR_VERBOSE = enum.auto()
        SOURCE = enum.auto()
        DEFAULT = enum.auto()
        HAT_DYNAMIC = HAT_PACKAGE | DYNAMIC_LIBRARY
        HAT_STATIC = HAT_PACKAGE | STATIC_LIBRARY
        HAT_SOURCE = HAT_PACKAGE | SOURCE
        MLIR_DYNAMIC = HAT_DYNAMIC | MLIR
        MLIR_STATIC = HAT_STATIC | MLIR
        MLIR_SOURCE = HAT_SOURCE | MLIR

    class Mode(enum.Enum):
        RELEASE = "Release"
        DEBUG = "Debug"

    class Platform(enum.Enum):
        HOST = "host"
        LINUX = "linux"

    def __init__(self):
        self._fns: "OrderedDict[str, _PackagedFunction]" = OrderedDict()
        self._description: Dict[str, Any] = {}

    # ------------------------------------------------------------------ add
    def add(self, source, args: Sequence[Any] = None, base_name: str = "", parameters: Optional[dict] = None,
            function_opts: Optional[dict] = None, auxiliary: Optional[dict] = None):
        """Adds one function.  `source` is a Nest, Schedule or Plan describing matmul(+bias)(+ReLU),
        reduce_mean, gather or a dimension function; `args` fixes the C argument order."""
        if args is None:
            raise ValueError("args is required")
        args = list(args)
        for a in args:
            if isinstance(a, Array) and a.role is Role.TEMP:
                raise ValueError("TEMP arrays cannot be function arguments")      # Package.py:231-236
            if isinstance(a, Scalar) and a.role is Role.TEMP:
                raise ValueError("TEMP scalars cannot be function arguments")
            if not isinstance(a, (Array, Dimension, Scalar)):
                raise TypeError("args may contain Arrays, Dimensions and Scalars")
        target = source.target if isinstance(source, lang.Plan) else Target.HOST
        for f in self._fns.values():
            if not target.is_compatible_with(f.target):
                raise NotImplementedError(
                    "Function target being added is currently incompatible with existing functions in package")
        spec = patterns.recognise(source)
        self._check_args(spec, args)
        aux = {"accera": {"parameters": dict(parameters or {})}}
        if auxiliary:
            aux.update(auxiliary)
        name = self._function_name(base_name, target, aux, args)
        if name in self._fns:
            raise ValueError(f"function {name} already in package")
        fn = _PackagedFunction(name, base_name, spec, args, target, aux)
        self._fns[name] = fn
        return fn

    @staticmethod
    def _function_name(base_name: str, target: Target, aux: dict, args) -> str:
        # stable hash of [base_name, target, parameters, argument signatures] (Package.py:310-335)
        sig = [base_name or secrets.token_hex(4), str(target), str(aux["accera"])]
        for a in args:
            if isinstance(a, Array):
                shape = tuple(s.name if isinstance(s, Dimension) else s for s in a.shape)
                sig.append(str((a.role.name, a.element_type.name, shape, str(a.layout))))
            elif isinstance(a, Scalar):
                sig.append(str((a.role.name, a.type.name, "scalar")))
            else:
                sig.append(str((a.name, a.type.name)))
        suffix = hashlib.md5(json.dumps(tuple(sig)).encode("utf-8")).digest().hex()[:16]
        return f"{base_name}_{suffix}" if base_name else f"_{suffix}"

    @staticmethod
    def _check_args(spec, args) -> None:
        def need(*arrays):
            for arr in arrays:
                if arr is not None and not any(a is arr for a in args):
                    raise ValueError(f"array {arr!r} is used by the nest but missing from args")
            for arr in arrays:
                if arr is None:
                    continue
                for s in arr.shape:
                    if isinstance(s, Dimension) and not any(a is s for a in args):
                        raise ValueError(f"dimension {s!r} sizes {arr!r} but is missing from args")
        if spec.kind == "gemm":
            need(spec.a, spec.b, spec.c, spec.bias)
            if spec.batch is not None and (spec.a.is_dynamic or spec.b.is_dynamic or spec.c.is_dynamic):
                raise patterns.UnsupportedNestError("batch matmul is implemented for statically shaped arrays")
            if spec.c.role is not Role.INPUT_OUTPUT and spec.c.role is not Role.OUTPUT:
                raise ValueError("the GEMM result array must be INPUT_OUTPUT")
            key = (spec.a.element_type, spec.b.element_type, spec.c.element_type)
            ok = {(ScalarType.float32,) * 3, (ScalarType.float16, ScalarType.float16, ScalarType.float32),
                  (ScalarType.float16,) * 3, (ScalarType.bfloat16, ScalarType.bfloat16, ScalarType.float32),
                  (ScalarType.bfloat16,) * 3, (ScalarType.int8, ScalarType.int8, ScalarType.int32),
                  (ScalarType.uint8, ScalarType.uint8, ScalarType.int32)}
            if key not in ok:
                raise patterns.UnsupportedNestError(f"unsupported GEMM element types {[k.name for k in key]}")
            if spec.bias is not None and spec.bias.element_type is not ScalarType.float32:
                raise patterns.UnsupportedNestError("bias must be float32")
        elif spec.kind == "reduce_mean":
            need(spec.data, spec.reduced)
            if spec.data.element_type is not ScalarType.float32 or spec.reduced.element_type is not ScalarType.float32:
                raise patterns.UnsupportedNestError("reduce_mean is implemented for float32")
            if len(spec.data.shape) > 3:
                raise patterns.UnsupportedNestError("reduce_mean is implemented for rank <= 3")
        elif spec.kind == "gather":
            need(spec.data, spec.indices, spec.output)
            if spec.indices.element_type not in (ScalarType.index, ScalarType.int64):
                raise patterns.UnsupportedNestError("gather indices must be index / int64")
            if spec.data.element_type is not spec.output.element_type:
                raise patterns.UnsupportedNestError("gather output must have the data's element type")
        elif spec.kind == "range_size":
            for sc in (spec.start, spec.limit, spec.delta):
                if not any(a is sc for a in args):
                    raise ValueError(f"scalar {sc!r} is used by the nest but missing from args")
                if sc.type is not ScalarType.float32 or sc.role is not Role.INPUT:
                    raise patterns.UnsupportedNestError("range: start, limit and delta must be float32 input scalars")
            if not any(a is spec.size for a in args) or spec.size.role is Role.INPUT:
                raise ValueError("range size: the output Dimension must be an argument with Role.OUTPUT")
        elif spec.kind == "range":
            need(spec.output)
            for sc in (spec.running, spec.delta):
                if not any(a is sc for a in args):
                    raise ValueError(f"scalar {sc!r} is used by the nest but missing from args")
            if spec.output.element_type is not ScalarType.float32 or spec.running.type is not ScalarType.float32 \
                    or spec.delta.type is not ScalarType.float32:
                raise patterns.UnsupportedNestError("range is implemented for float32")
            if spec.running.role is not Role.INPUT_OUTPUT or spec.delta.role is not Role.INPUT:
                raise patterns.UnsupportedNestError("range: the running scalar must be INPUT_OUTPUT and delta INPUT")
            if len(spec.output.shape) != 1:
                raise patterns.UnsupportedNestError("range fills a one-dimensional array")
        elif spec.kind == "dims":
            for out, src in spec.assignments:
                for d in (out, src):
                    if isinstance(d, Dimension) and not any(a is d for a in args):
                        raise ValueError(f"dimension {d!r} is missing from args")

    # ---------------------------------------------------------------- build
    def add_description(self, author: str = None, license: str = None, other: dict = None, version: str = None):
        """Package-level metadata written into [description] (Package.py:789-838)."""
        if other is None:
            other = {}
        if "auxiliary" not in self._description:
            self._description["auxiliary"] = other
        else:
            self._description["auxiliary"].update(other)
        for k in [k for k, v in self._description["auxiliary"].items() if v is None]:
            del self._description["auxiliary"][k]
        if version is not None:
            self._description["version"] = version
        if author is not None:
            self._description["author"] = author
        if license is not None:
            self._description["license"] = license

    def build(self, name: str, format: "Package.Format" = None, mode: "Package.Mode" = None,
              platform: "Package.Platform" = None, tolerance: float = 1e-5, output_dir: str = None,
              fail_on_error: bool = False, **kwargs) -> List[str]:
        """Writes `name`.hat and the library next to it; returns the paths of the files written."""
        format = format if format is not None else Package.Format.DEFAULT
        mode = mode or Package.Mode.RELEASE
        if mode is Package.Mode.DEBUG:
            raise NotImplementedError("Debug mode is not supported for GPU targets")       # Package.py:587-588
        if format & Package.Format.DEFAULT:
            format = Package.Format.HAT_DYNAMIC
        if not (format & Package.Format.HAT_PACKAGE):
            raise NotImplementedError("only HAT package formats are produced")
        if not name.isidentifier():
            raise ValueError("package name must be a valid C identifier")
        output_dir = os.path.abspath(output_dir or os.getcwd())
        os.makedirs(output_dir, exist_ok=True)

        dynamic = bool(format & Package.Format.DYNAMIC_LIBRARY)
        static = bool(format & Package.Format.STATIC_LIBRARY)
        if not dynamic and not static:
            dynamic = True
        keep_source = bool(format & Package.Format.SOURCE)

        src_path = os.path.join(output_dir, f"{name}.cpp")
        with open(src_path, "w") as f:
            f.write(self._stub_source(name))
        written = []
        lib_name = ""
        cxx = shutil.which("g++") or shutil.which("c++")
        if cxx is None:
            raise RuntimeError("a host C++ compiler (g++) is required to build a package")
        core_lib = os.path.join(_PKG_DIR, "libaccera_b200.so")
        if not os.path.exists(core_lib):
            from . import build as _build
            _build.build()
        common = [cxx, "-O2", "-fPIC", "-std=c++17", f"-I{_INCLUDE_DIR}"]
        if dynamic:
            lib_name = f"{name}.so"
            cmd = common + ["-shared", src_path, "-o", os.path.join(output_dir, lib_name), f"-L{_PKG_DIR}",
                            "-laccera_b200", f"-Wl,-rpath,{_PKG_DIR}", "-Wl,-rpath,$ORIGIN"]
            self._run(cmd)
            written.append(os.path.join(output_dir, lib_name))
        if static:
            obj = os.path.join(output_dir, f"{name}.o")
            self._run(common + ["-c", src_path, "-o", obj])
            lib_a = os.path.join(output_dir, f"{name}.a")
            if os.path.exists(lib_a):
                os.remove(lib_a)
            self._run(["ar", "rcs", lib_a, obj])
            os.remove(obj)
            written.append(lib_a)
            if not dynamic:
                lib_name = f"{name}.a"
        if keep_source:
            written.append(src_path)
        else:
            os.remove(src_path)

        hat_path = os.path.join(output_dir, f"{name}.hat")
        self._hat_file(name, lib_name, dynamic).write(hat_path)
        written.insert(0, hat_path)
        return written

    @staticmethod
    def _run(cmd: List[str]) -> None:
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"{' '.join(cmd)} failed:\n{r.stdout}\n{r.stderr}")

    # -------------------------------------------------------- .hat emission
    def _hat_file(self, name: str, lib_name: str, dynamic: bool) -> hat_file.HATFile:
        hf = hat_file.HATFile(name=name)
        desc = {"comment": "", "author": self._description.get("author", ""),
                "version": self._description.get("version", ""), "license_url": self._description.get("license", "")}
        if self._description.get("auxiliary"):
            desc["auxiliary"] = self._description["auxiliary"]
        hf.description = desc
        decl = [hat_file.header_prologue(name)]
        seen_alias = set()
        for fn in self._fns.values():
            hfn = hat_file.Function(name=fn.name, description="", calling_convention="cdecl",
                                    arguments=[self._parameter(fn, a) for a in fn.args],
                                    auxiliary=dict(fn.auxiliary))
            hfn.auxiliary["accera_b200"] = self._kernel_metadata(fn)
            hf.functions.append(hfn)
            if fn.target.category is Target.Category.GPU and fn.spec.kind == "gemm" and fn.spec.compute == "tensor":
                # GPU targets: the host entry names the kernel it launches and a device-function entry carries
                # the launch geometry (Package.py:726-743); here that kernel is the persistent tcgen05 GEMM
                # precompiled in the core library: one 192-thread CTA per SM, ~193 KiB of dynamic shared memory
                hfn.launches = fn.name + "__gpu__"
                hfn.runtime = "CUDA"
                hf.device_functions.append(hat_file.Function(
                    name=fn.name + "__gpu__", description="", calling_convention="device",
                    arguments=[self._parameter(fn, a) for a in fn.args], launch_parameters=[148, 1, 1, 192, 1, 1],
                    dynamic_shared_mem_bytes=197888, provider="libaccera_b200.so", runtime="CUDA"))
            decl.append(hfn.c_declaration() + "\n\n")
            if fn.base_name and fn.base_name not in seen_alias:
                seen_alias.add(fn.base_name)
                decl.append(hfn.c_alias(fn.base_name) + "\n")
        decl.append(hat_file.header_epilogue())
        hf.declaration_code = "".join(decl)
        hf.target = {
            "required": {"os": "linux", "CPU": {"architecture": _platform.machine() or "x86_64", "extensions": []},
                         "GPU": {"runtime": "CUDA", "instruction_set_version": "sm_100a", "min_threads": 192,
                                 "min_global_memory_KB": 0, "min_shared_memory_KB": 227, "min_texture_memory_KB": 0}},
            "optimized_for": {"GPU": {"name": "NVIDIA B200", "family": "Blackwell", "cores": 148}},
        }
        hf.dependencies = {"link_target": lib_name, "deploy_files": [],
                           "dynamic": [{"name": "accera_b200", "version": "0.1", "target_file": "libaccera_b200.so"}],
                           "auxiliary": {"dynamic" if dynamic else "static": lib_name}}
        hf.compiled_with = {"compiler": "nvcc + g++", "flags": "-gencode arch=compute_100a,code=sm_100a -O3", "crt": "",
                            "libraries": ["libaccera_b200.so"]}
        return hf

    @staticmethod
    def _parameter(fn: _PackagedFunction, a) -> hat_file.Parameter:
        if isinstance(a, Dimension):
            ctype = lang.C_TYPE[ScalarType.index]
            usage = "input" if a.role is Role.INPUT else "output"
            return hat_file.Parameter(name=a.name, logical_type="element", usage=usage, element_type=ctype,
                                      declared_type=ctype + ("" if usage == "input" else "*"))
        ctype = lang.C_TYPE[a.element_type]
        usage = {Role.INPUT: "input", Role.INPUT_OUTPUT: "input_output", Role.OUTPUT: "output"}[a.role]
        if isinstance(a, Scalar):
            # element arguments that are not inputs are passed by pointer (HATEmitter.h:392-400)
            return hat_file.Parameter(name=a.name, logical_type="element", usage=usage, element_type=ctype,
                                      declared_type=ctype + ("" if usage == "input" else "*"))
        if a.is_dynamic:
            size = "*".join(s.name if isinstance(s, Dimension) else str(s) for s in a.shape)
            return hat_file.Parameter(name=a.name, logical_type="runtime_array", usage=usage, element_type=ctype,
                                      declared_type=ctype + "*", size=size)
        return hat_file.Parameter(name=a.name, logical_type="affine_array", usage=usage, element_type=ctype,
                                  declared_type=ctype + "*", shape=list(a.shape), affine_map=list(a.strides()),
                                  affine_offset=a.offset)

    @staticmethod
    def _kernel_metadata(fn: _PackagedFunction) -> Dict[str, Any]:
        s = fn.spec
        if s.kind == "gemm":
            return {"op": "gemm", "compute": s.compute, "relu": s.relu, "bias": s.bias is not None,
                    "alpha": float(s.alpha), "beta": float(s.beta)}
        if s.kind == "reduce_mean":
            return {"op": "reduce_mean", "axes": list(s.axes), "keepdims": int(s.keepdims)}
        if s.kind == "gather":
            return {"op": "gather", "axis": int(s.axis)}
        if s.kind in ("range", "range_size"):
            return {"op": s.kind}
        return {"op": "dims"}

    # ------------------------------------------------------ stub generation
    def _stub_source(self, name: str) -> str:
        out = [f"// Generated by accera_b200.Package for package {name}: thin forwards into the C ABI of\n"
               "// libaccera_b200.so (include/accera_b200.h).  The exported prototypes are the HAT prototypes.\n"
               "#include <cstdint>\n#include <cstdio>\n#include \"accera_b200.h\"\n\n"
               "typedef uint16_t float16_t;\ntypedef uint16_t bfloat16_t;\n\n"
               "static void report(const char* fn, int rc)\n{\n"
               "    // HAT functions return void: errors go to stderr, like the reference's debug-mode prints\n"
               "    if (rc < 0) std::fprintf(stderr, \"%s: error %d: %s\\n\", fn, rc, accb_last_error());\n}\n\n"
               "extern \"C\" {\n\n"]
        for fn in self._fns.values():
            out.append(self._stub_function(fn))
        out.append("}  // extern \"C\"\n")
        return "".join(out)

    def _stub_function(self, fn: _PackagedFunction) -> str:
        arg_name: Dict[int, str] = {}
        params = []
        for pos, a in enumerate(fn.args):
            arg_name[id(a)] = f"a{pos}"
            if isinstance(a, Dimension):
                params.append(f"int64_t{'' if a.role is Role.INPUT else '*'} a{pos}")
            elif isinstance(a, Scalar):
                params.append(f"{lang.C_TYPE[a.element_type]}{'' if a.role is Role.INPUT else '*'} a{pos}")
            else:
                params.append(f"{lang.C_TYPE[a.element_type]}* a{pos}")

        def dim(v) -> str:
            if isinstance(v, Dimension):
                return arg_name[id(v)]
            return f"INT64_C({int(v)})"

        def strides(arr: Array, transposed: bool = False) -> List[str]:
            if arr.is_dynamic:                      # dense first-major from the dimension arguments
                st = [dim(arr.shape[1]), "INT64_C(1)"]
            else:
                st = [f"INT64_C({s})" for s in arr.strides()]
            return st[::-1] if transposed else st

        body: List[str] = []
        s = fn.spec
        batched = s.kind == "gemm" and s.batch is not None
        if batched:
            def split(arr: Array, pos) -> Tuple[List[str], str]:
                st = arr.strides()
                return ([f"INT64_C({st[pos[1]]})", f"INT64_C({st[pos[2]]})"],
                        f"INT64_C({st[pos[0]] if pos[0] is not None else 0})")
            (sa, a_bs), (sb, b_bs), (sc, c_bs) = split(s.a, s.a_pos), split(s.b, s.b_pos), split(s.c, s.c_pos)
            call = (f"accb_gemm_batched(&d, {dim(s.batch)}, {a_bs}, {b_bs}, {c_bs}, {arg_name[id(s.a)]}, "
                    f"{arg_name[id(s.b)]}, {arg_name[id(s.c)]}, nullptr)")
        elif s.kind == "gemm":
            sa, sb, sc = strides(s.a, s.a_transposed), strides(s.b, s.b_transposed), strides(s.c)
            call = (f"accb_gemm(&d, {arg_name[id(s.a)]}, {arg_name[id(s.b)]}, {arg_name[id(s.c)]}, "
                    f"{arg_name[id(s.bias)] if s.bias is not None else 'nullptr'})")
        if s.kind == "gemm":
            body += [
                "    accb_gemm_desc d = {};",
                f"    d.m = {dim(s.m)}; d.n = {dim(s.n)}; d.k = {dim(s.k)};",
                f"    d.a_type = {_ACCB_TYPE[s.a.element_type]}; d.b_type = {_ACCB_TYPE[s.b.element_type]}; "
                f"d.c_type = {_ACCB_TYPE[s.c.element_type]};",
                f"    d.compute = {_COMPUTE[s.compute]};",
                f"    d.a_stride[0] = {sa[0]}; d.a_stride[1] = {sa[1]};",
                f"    d.b_stride[0] = {sb[0]}; d.b_stride[1] = {sb[1]};",
                f"    d.c_stride[0] = {sc[0]}; d.c_stride[1] = {sc[1]};",
                f"    d.alpha = {float(s.alpha)!r}f; d.beta = {float(s.beta)!r}f;",
                f"    d.epilogue = {'ACCB_EPI_RELU' if s.relu else 'ACCB_EPI_NONE'};",
                f"    report(\"{fn.name}\", {call});",
            ]
        elif s.kind == "reduce_mean":
            shape = list(s.data.shape)
            pad = 3 - len(shape)
            dims3 = ["INT64_C(1)"] * pad + [dim(v) for v in shape]
            mask = 0
            for ax in s.axes:
                mask |= 1 << (ax + pad)
            body.append(f"    report(\"{fn.name}\", accb_reduce_mean_rank3({arg_name[id(s.data)]}, {dims3[0]}, {dims3[1]}, "
                        f"{dims3[2]}, {arg_name[id(s.reduced)]}, {mask}));")
        elif s.kind == "gather":
            d0, d1 = (dim(v) for v in s.data.shape)
            i0, i1 = (dim(v) for v in s.indices.shape)
            body.append(f"    report(\"{fn.name}\", accb_gather_rank2({arg_name[id(s.data)]}, {d0}, {d1}, "
                        f"{arg_name[id(s.indices)]}, {i0}, {i1}, {arg_name[id(s.output)]}, {int(s.axis)}, "
                        f"{lang.TYPE_BYTES[s.data.element_type]}));")
        elif s.kind == "range_size":
            body.append(f"    *{arg_name[id(s.size)]} = accb_range_count_f32({arg_name[id(s.start)]}, {arg_name[id(s.limit)]}, "
                        f"{arg_name[id(s.delta)]});")
        elif s.kind == "range":
            body.append(f"    report(\"{fn.name}\", accb_range_f32({dim(s.n)}, {arg_name[id(s.output)]}, "
                        f"{arg_name[id(s.running)]}, {arg_name[id(s.delta)]}));")
        else:
            for out_dim, src in s.assignments:
                body.append(f"    *{arg_name[id(out_dim)]} = {dim(src)};")
        return f"void {fn.name}({', '.join(params)})\n{{\n" + "\n".join(body) + "\n}\n\n"
