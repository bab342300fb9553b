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
from .hat import hat_file, packaging
from .lang import Array, Dimension, Role, Scalar, ScalarType, Target

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
_INCLUDE_DIR = os.path.join(os.path.dirname(_PKG_DIR), "include")

_ACCB_TYPE = {ScalarType.float32: "ACCB_F32", ScalarType.float16: "ACCB_F16", ScalarType.bfloat16: "ACCB_BF16",
              ScalarType.int8: "ACCB_S8", ScalarType.int32: "ACCB_S32", ScalarType.uint8: "ACCB_U8", ScalarType.int16: "ACCB_S16"}
_COMPUTE = {"auto": "ACCB_COMPUTE_AUTO", "simt": "ACCB_COMPUTE_SIMT", "tensor": "ACCB_COMPUTE_TENSOR_PREFERRED"}


class _PackagedFunction:
    def __init__(self, name, base_name, spec, args, target, auxiliary):
        self.name = name
        self.base_name = base_name
        self.spec = spec
        self.args = list(args)
        self.target = target
        self.auxiliary = auxiliary
        self.launch_request = None      # (block, grid) a bound GPU plan asked for


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
            if isinstance(a, Array) and not a.is_dynamic and getattr(a, "offset", 0):
                # the exported functions take the array's first element; an affine_offset in the descriptor would
                # promise something the stub does not do
                raise patterns.UnsupportedNestError("arrays with a non-zero offset are not supported as function arguments")
        target = source.target if isinstance(source, lang.Plan) else Target.HOST
        if isinstance(source, lang.Plan):
            source.check_launch_request()           # an impossible block is rejected here, as in lang/Plan.py:989-1004
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
        if isinstance(source, lang.Plan) and target.category is Target.Category.GPU:
            try:
                fn.launch_request = source.launch_request()
            except ValueError:
                fn.launch_request = None
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
                  (ScalarType.uint8, ScalarType.uint8, ScalarType.int32), (ScalarType.int16, ScalarType.int16, ScalarType.int32)}
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
        cxx = shutil.which("g++") or shutil.which("c++")
        if cxx is None:
            raise RuntimeError("a host C++ compiler (g++) is required to build a package")
        core_lib = os.path.join(_PKG_DIR, packaging.CORE_LIBRARY)
        if not os.path.exists(core_lib):
            from . import build as _build
            _build.build()

        # 1. the object file, and a .hat that names it as its link target (Package.py:669-681)
        obj_path = os.path.join(output_dir, f"{name}.o")
        self._run([cxx, "-O2", "-fPIC", "-std=c++17", f"-I{_INCLUDE_DIR}", "-c", src_path, "-o", obj_path])
        hat_path = os.path.join(output_dir, f"{name}.hat")
        self._emit_header(name).Serialize(hat_path)

        # 2. completed with what this layer knows, through the same calls the reference makes on hatlib's
        #    HATFile (Package.py:678-764)
        hf = hat_file.HATFile.Deserialize(hat_path)
        hf.dependencies.link_target = os.path.basename(obj_path)
        hf.dependencies.dynamic = [hat_file.LibraryReference(name="accera_b200", version="0.1", target_file=packaging.CORE_LIBRARY)]
        for fn in self._fns.values():
            hat_func = hf.function_map.get(fn.name)
            if hat_func is None:
                raise ValueError(f"Couldn't find header-declared function {fn.name} in emitted HAT file")
            hat_func.auxiliary = dict(fn.auxiliary)
            hat_func.auxiliary["accera_b200"] = self._kernel_metadata(fn)
            if fn.target.category is Target.Category.GPU:
                hf.target.required.gpu.model = fn.target.name
        hf.target.required.os = hat_file.OperatingSystem.host()
        hf.target.required.cpu.architecture = _platform.machine() or "x86_64"
        hf.target.required.cpu.extensions = []
        gpu = hf.target.required.gpu
        gpu.runtime = "CUDA"
        gpu.instruction_set_version = "sm_100a"
        gpu.min_threads = 192
        gpu.min_global_memory_KB = 0
        gpu.min_shared_memory_KB = 227
        gpu.min_texture_memory_KB = 0
        hf.target.optimized_for.gpu.name = "NVIDIA B200"
        hf.target.optimized_for.gpu.family = "Blackwell"
        hf.target.optimized_for.gpu.cores = 148
        hf.compiled_with.compiler = "nvcc + g++"
        hf.compiled_with.flags = "-gencode arch=compute_100a,code=sm_100a -O3"
        hf.compiled_with.libraries = [packaging.CORE_LIBRARY]
        hf.description.author = self._description.get("author", "")
        hf.description.version = self._description.get("version", "")
        hf.description.license_url = self._description.get("license", "")
        if self._description.get("auxiliary"):
            hf.description.auxiliary = self._description["auxiliary"]
        hf.Serialize(hat_path)

        # 3. the library, and the .hat that points at it (Package.py:766-784)
        written = [hat_path]
        path_root = os.path.join(output_dir, name)
        if static:
            lib_hat_path = f"{path_root}_lib.hat"
            packaging.create_static_package(hat_path, lib_hat_path)
            os.replace(f"{path_root}_lib.a", f"{path_root}.a")
            lib_hat_file = hat_file.HATFile.Deserialize(lib_hat_path)
            lib_hat_file.dependencies.link_target = f"{name}.a"
            lib_hat_file.dependencies.auxiliary["static"] = lib_hat_file.dependencies.link_target
            lib_hat_file.Serialize()
            static_hat = lib_hat_file
            written.append(f"{path_root}.a")
        if dynamic:
            dyn_hat_path = f"{path_root}_dyn.hat"
            packaging.create_dynamic_package(hat_path, dyn_hat_path)
            os.replace(f"{path_root}_dyn.so", f"{path_root}.so")
            dyn_hat_file = hat_file.HATFile.Deserialize(dyn_hat_path)
            dyn_hat_file.dependencies.link_target = f"{name}.so"
            dyn_hat_file.dependencies.auxiliary["dynamic"] = dyn_hat_file.dependencies.link_target
            if static:
                dyn_hat_file.dependencies.auxiliary["static"] = f"{name}.a"
            dyn_hat_file.Serialize()
            written.insert(1, f"{path_root}.so")
        # the .hat a loader sees points at the dynamic library when there is one (Package.py:775-786 moves the
        # static one over the original first, then the dynamic one)
        if static:
            shutil.move(f"{path_root}_lib.hat", hat_path)
        if dynamic:
            shutil.move(f"{path_root}_dyn.hat", hat_path)
        os.remove(obj_path)
        if keep_source:
            written.append(src_path)
        else:
            os.remove(src_path)
        return written

    @staticmethod
    def _run(cmd: List[str]) -> None:
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"{' '.join(cmd)} failed:\n{r.stdout}\n{r.stderr}")

    # -------------------------------------------------------- .hat emission
    def _emit_header(self, name: str) -> hat_file.HATFile:
        """The part of the .hat the reference's C++ layer writes (package_module.WriteHeader, Package.py:674-675;
        TranslateToHeader.cpp:165-201, 402-506): one function table per public function and the C declarations."""
        hf = hat_file.HATFile(name=name)
        decl = [hat_file.header_prologue(name)]
        seen_alias = set()
        for fn in self._fns.values():
            hfn = hat_file.Function(name=fn.name, description="", calling_convention=hat_file.CallingConventionType.CDecl,
                                    arguments=[self._parameter(fn, a) for a in fn.args])
            hf.function_map[fn.name] = hfn
            decl.append(hfn.c_declaration() + "\n\n")
            if fn.base_name and fn.base_name not in seen_alias:
                seen_alias.add(fn.base_name)
                decl.append(hfn.c_alias(fn.base_name) + "\n")
        decl.append(hat_file.header_epilogue())
        hf.declaration.code = "".join(decl)
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
        """What runs behind the exported function, for tools and readers; no loader needs it.

        The reference lists a GPU function's kernel as a device function with `launches`, `launch_parameters` and
        `dynamic_shared_mem_bytes`, and its loader compiles the `.cu` provider and launches that kernel itself
        (Package.py:714-743).  The functions of this package are HOST-callable stubs over a prebuilt library: a
        loader must call them like any CPU function (host arrays are staged through the GPU), so they carry no
        `launches` link.  The geometry of the kernel the stub ends up launching is recorded here instead - the
        true one for the tensor-core GEMM on the target's SM count (accb_gemm_launch_geometry), next to what a
        bound plan asked for."""
        s = fn.spec
        gpu_target = fn.target.category is Target.Category.GPU
        if s.kind == "gemm":
            meta: Dict[str, Any] = {"op": "gemm", "compute": s.compute, "relu": s.relu, "bias": s.bias is not None,
                                    "alpha": float(s.alpha), "beta": float(s.beta)}
            static = all(isinstance(v, int) for v in (s.m, s.n, s.k)) and s.batch is None
            if s.compute == "tensor" and static:
                from . import runtime
                in_type = s.a.element_type.name
                try:
                    sms = fn.target.num_sms or 148
                    geo = runtime.gemm_launch_geometry(int(s.m), int(s.n), int(s.k), in_type=in_type, compute="tensor_preferred",
                                                       num_sms=sms, b_row_major=not s.b_transposed and s.b.strides()[1] == 1)
                    plan = runtime.gemm_tile_plan(int(s.m), int(s.n), int(s.k), in_type=in_type, compute="tensor_preferred",
                                                  num_sms=sms, b_row_major=not s.b_transposed and s.b.strides()[1] == 1)
                    meta.update({"kernel": "gemm_umma_kernel", "device_function": fn.name + "__gpu__",
                                 "launch_parameters": geo["grid"] + geo["block"],
                                 "dynamic_shared_mem_bytes": geo["dynamic_shared_mem_bytes"], "num_sms": sms,
                                 "cta_pairs": plan["cta_pairs"], "tile_cols": plan["tile_cols"], "tiles": plan["tiles"]})
                except Exception:            # the library is not built yet: the metadata is optional
                    pass
            if gpu_target and fn.launch_request is not None:
                block, grid = fn.launch_request
                meta["requested_launch_parameters"] = list(grid) + list(block)
            if gpu_target:
                meta["runtime"] = "CUDA"
            return meta
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
