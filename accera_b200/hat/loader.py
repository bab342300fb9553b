"""Loads a HAT package and calls / benchmarks its functions, with the call shape of the third-party
`hatlib` the reference's tests and tools use (it is not part of the reference tree):

    package, functions = load("P.hat")              # verifiers.py:18-38
    functions.names                                  # verifiers.py:27
    functions["matmul_relu_<hash>"](A, B, C)         # numpy arrays, mutated in place
    functions.matmul_relu                            # base-name alias (first function with that base name)
    run_benchmark("P.hat", batch_size=5, min_time_in_sec=5)   # README.md:136, accera_gemm.py:612-626

Arguments are checked against the descriptor before the call: element type, shape and element strides
of every affine_array (a column-major B must be passed Fortran-ordered, mfma_tests.py:184-192), element
count of every runtime_array (evaluated from the dimension arguments).

Array arguments may also be torch CUDA tensors: they are used in place on torch's current stream and the
call does not synchronise.  `run_benchmark(..., device_resident=True)` times functions that way, with CUDA
events around batches of launches on buffers that already live on the GPU - what hatlib does for GPU
functions and what the reference's GEMM benchmarker reads its TFLOP/s from (accera_gemm.py:612-660).
"""
from __future__ import annotations

import ctypes
import dataclasses
import os
import re
import statistics
import time
from typing import Any, Dict, List, Optional

import numpy as np

from .hat_file import Function, HATFile

_NP_OF_C = {
    "float": np.float32, "double": np.float64, "float16_t": np.float16, "bfloat16_t": np.uint16,
    "int8_t": np.int8, "int16_t": np.int16, "int32_t": np.int32, "int64_t": np.int64,
    "uint8_t": np.uint8, "uint16_t": np.uint16, "uint32_t": np.uint32, "uint64_t": np.uint64, "bool": np.bool_,
}
_TORCH_OF_C = {
    "float": "float32", "double": "float64", "float16_t": "float16", "bfloat16_t": "bfloat16", "int8_t": "int8",
    "int16_t": "int16", "int32_t": "int32", "int64_t": "int64", "uint8_t": "uint8", "bool": "bool",
}


def _is_torch(x) -> bool:
    return type(x).__module__.split(".")[0] == "torch"


_CTYPES_OF_C = {
    "int8_t": ctypes.c_int8, "int16_t": ctypes.c_int16, "int32_t": ctypes.c_int32, "int64_t": ctypes.c_int64,
    "uint8_t": ctypes.c_uint8, "uint16_t": ctypes.c_uint16, "uint32_t": ctypes.c_uint32, "uint64_t": ctypes.c_uint64,
    "float": ctypes.c_float, "double": ctypes.c_double, "bool": ctypes.c_bool,
}


class HATFunction:
    """A callable bound to one exported symbol, checked against its descriptor."""

    def __init__(self, desc: Function, symbol):
        self.desc = desc
        self.name = desc.name
        self._symbol = symbol
        self._symbol.restype = None

    def _marshal(self, args):
        params = self.desc.arguments
        if len(args) != len(params):
            raise ValueError(f"{self.name}: expected {len(params)} arguments, got {len(args)}")
        values: Dict[str, int] = {}
        c_args = []
        keep = []
        for p, a in zip(params, args):
            if p.logical_type == "element":
                ct = _CTYPES_OF_C.get(p.element_type)
                if ct is None:
                    raise TypeError(f"{self.name}: unsupported element type {p.element_type}")
                if p.usage == "input":
                    values[p.name] = int(a) if "int" in p.element_type else a
                    c_args.append(ct(a))
                else:
                    # output / in-out scalar: pass a 1-element numpy array or a ctypes instance
                    if isinstance(a, np.ndarray):
                        if a.dtype != _NP_OF_C[p.element_type] or a.size != 1:
                            raise TypeError(f"{self.name}: argument {p.name!r} must be a 1-element {p.element_type} array")
                        c_args.append(ctypes.c_void_p(a.ctypes.data))
                    else:
                        c_args.append(ctypes.byref(a))
                    keep.append(a)
        # arrays second, once the dimension values are known
        it = iter(c_args)
        out = []
        for p, a in zip(params, args):
            if p.logical_type == "element":
                out.append(next(it))
                continue
            if _is_torch(a):
                # a device tensor: same checks, element strides straight from the tensor
                if str(a.dtype).replace("torch.", "") != _TORCH_OF_C.get(p.element_type):
                    raise TypeError(f"{self.name}: argument {p.name!r} has dtype {a.dtype}, descriptor says {p.element_type}")
                if not a.is_cuda:
                    raise TypeError(f"{self.name}: torch arguments must be CUDA tensors (pass host data as numpy arrays)")
                if p.logical_type == "affine_array":
                    if list(a.shape) != list(p.shape):
                        raise ValueError(f"{self.name}: argument {p.name!r} has shape {tuple(a.shape)}, descriptor says {p.shape}")
                    for dim, st, ws in zip(a.shape, a.stride(), p.affine_map):
                        if dim > 1 and st != ws:
                            raise ValueError(f"{self.name}: argument {p.name!r} has element strides {list(a.stride())}, "
                                             f"descriptor says {p.affine_map}")
                else:
                    n = _eval_size(p.size or "", values)
                    if a.numel() != n or not a.is_contiguous():
                        raise ValueError(f"{self.name}: argument {p.name!r} must be a dense tensor of {n} elements ({p.size})")
                out.append(ctypes.c_void_p(a.data_ptr()))
                keep.append(a)
                continue
            if not isinstance(a, np.ndarray):
                raise TypeError(f"{self.name}: argument {p.name!r} must be a numpy array or a torch CUDA tensor")
            want = _NP_OF_C.get(p.element_type)
            if want is None or a.dtype != want:
                raise TypeError(f"{self.name}: argument {p.name!r} has dtype {a.dtype}, descriptor says {p.element_type}")
            if p.logical_type == "affine_array":
                if list(a.shape) != list(p.shape):
                    raise ValueError(f"{self.name}: argument {p.name!r} has shape {a.shape}, descriptor says {p.shape}")
                strides = [s // a.itemsize for s in a.strides]
                for dim, st, ws in zip(a.shape, strides, p.affine_map):
                    if dim > 1 and st != ws:
                        raise ValueError(f"{self.name}: argument {p.name!r} has element strides {strides}, descriptor "
                                         f"says {p.affine_map} (pass column-major arrays with order='F')")
            else:
                n = _eval_size(p.size or "", values)
                if a.size != n or not a.flags.c_contiguous:
                    raise ValueError(f"{self.name}: argument {p.name!r} must be a dense array of {n} elements ({p.size})")
            out.append(ctypes.c_void_p(a.ctypes.data))
        return out, keep

    def __call__(self, *args, device_id: Optional[int] = None):
        c_args, keep = self._marshal(args)
        tensors = [a for a in keep if _is_torch(a)]
        from .. import runtime
        if tensors:
            # device buffers: the kernels go to torch's current stream of that device
            runtime._sync_torch_stream(*tensors)
            self._symbol(*c_args)
            return
        runtime.set_stream(0)                 # host arrays run on the default stream, whatever was selected before
        if device_id is None:
            self._symbol(*c_args)
            return
        # host arrays: staged through, and computed on, the GPU the caller names (hatlib's device_id argument,
        # tools/benchmarkers/accera_gemm.py:614) - for this call only: the thread's selection and the CUDA
        # runtime's current device are put back afterwards
        selected, current = runtime.selected_device(), runtime.current_device()
        runtime.set_device(int(device_id))
        try:
            self._symbol(*c_args)
        finally:
            runtime.set_device(current)
            if selected < 0:
                runtime.set_device(-1)

    def bind(self, *args):
        """-> zero-argument callable repeating this call on the same arguments (marshalled and checked once)."""
        c_args, keep = self._marshal(args)
        tensors = [a for a in keep if _is_torch(a)]
        from .. import runtime
        dev, stream = runtime._captured_selection(*tensors)
        L = runtime.lib()
        set_dev, set_str = L.accb_set_device, L.accb_set_stream
        symbol = self._symbol

        def call() -> None:
            # the device and stream of the arguments, re-selected: another call may have changed them in between
            if dev is not None:
                set_dev(dev)
            set_str(stream)
            symbol(*c_args)
        call.keep_alive = (keep, args)
        return call


def _eval_size(expr: str, values: Dict[str, int]) -> int:
    n = 1
    for tok in filter(None, (t.strip() for t in expr.split("*"))):
        n *= int(tok) if re.fullmatch(r"\d+", tok) else int(values[tok])
    return n


class FunctionMap:
    def __init__(self, functions: Dict[str, HATFunction], aliases: Dict[str, str]):
        self._functions = functions
        self._aliases = aliases

    @property
    def names(self) -> List[str]:
        return list(self._functions)

    def _resolve(self, name: str) -> HATFunction:
        if name in self._functions:
            return self._functions[name]
        if name in self._aliases:
            return self._functions[self._aliases[name]]
        raise KeyError(name)

    def __getitem__(self, name: str) -> HATFunction:
        return self._resolve(name)

    def __getattr__(self, name: str) -> HATFunction:
        try:
            return self._resolve(name)
        except KeyError:
            raise AttributeError(name) from None

    def __contains__(self, name: str) -> bool:
        return name in self._functions or name in self._aliases

    def __iter__(self):
        return iter(self._functions.values())

    def __len__(self):
        return len(self._functions)


class HATPackage:
    """A `.hat` file and, once loaded, its library.  `HATPackage(path)` only reads the descriptor, which is how
    the reference's tests inspect a built package (dsl_tests.py:5834-5842); `load` returns one with the library."""

    def __init__(self, hat, library: Optional[ctypes.CDLL] = None):
        if not isinstance(hat, HATFile):
            hat = HATFile.Deserialize(str(hat))
        self.hat_file = hat
        self.hat_file_path = hat.path
        self.library = library
        self.name = hat.name

    def get_functions(self) -> List[Function]:
        return list(self.hat_file.functions)

    def get_function(self, name: str) -> Optional[Function]:
        return self.hat_file.function_map.get(name)

    def get_functions_for_base_name(self, base_name: str) -> List[Function]:
        return [f for f in self.hat_file.functions if f.name == base_name or f.name.rsplit("_", 1)[0] == base_name]


def _aliases(hat: HATFile) -> Dict[str, str]:
    out: Dict[str, str] = {}
    for m in re.finditer(r"\(\*(\w+)\)\([^)]*\)\s*=\s*(\w+);", hat.declaration_code):
        out.setdefault(m.group(1), m.group(2))
    return out


def load(hat_path: str, try_dynamic_load: bool = True):
    """-> (HATPackage, FunctionMap).  The package must be dynamically linked (HAT_DYNAMIC)."""
    hat = HATFile.read(hat_path)
    lib_path = hat.link_target_path
    if not lib_path or not lib_path.endswith((".so", ".dll", ".dylib")):
        raise RuntimeError(f"{hat_path}: link_target {hat.dependencies.get('link_target')!r} is not a dynamic library; "
                           "build the package with Format.HAT_DYNAMIC to load it")
    if not os.path.exists(lib_path):
        raise FileNotFoundError(lib_path)
    library = ctypes.CDLL(lib_path)
    functions: Dict[str, HATFunction] = {}
    for f in hat.functions:
        if f.calling_convention == "device":
            continue
        functions[f.name] = HATFunction(f, getattr(library, f.name))
    return HATPackage(hat, library), FunctionMap(functions, _aliases(hat))


# ---------------------------------------------------------------------------
# benchmarking (row fields as printed in docs/Tutorials/GPU/Hello_MatMul_GPU.md:207-209)
# ---------------------------------------------------------------------------

@dataclasses.dataclass
class BenchmarkResult:
    """hatlib's result record (the reference's benchmarker turns it into a dict with dataclasses.asdict and reads
    min_of_means, tools/benchmarkers/accera_gemm.py:640-650).  All times are seconds per call."""
    function_name: str
    mean: float
    median_of_means: float
    mean_of_small_means: float
    robust_mean: float
    min_of_means: float

    @staticmethod
    def from_batch_means(function_name: str, batch_means: List[float]) -> "BenchmarkResult":
        means = sorted(batch_means)
        small = means[: max(1, len(means) // 2)]
        trim = len(means) // 5
        core = means[trim: len(means) - trim] or means
        return BenchmarkResult(function_name=function_name, mean=statistics.mean(means),
                               median_of_means=statistics.median(means), mean_of_small_means=statistics.mean(small),
                               robust_mean=statistics.mean(core), min_of_means=means[0])

    def as_dict(self) -> Dict[str, Any]:
        return dataclasses.asdict(self)


def _index_bound(fn: Function, values: Dict[str, int], dim_value: int) -> int:
    """Upper bound for generated gather indices: the gathered dimension of the data array (so that a benchmark does
    not time the out-of-range path)."""
    op = fn.auxiliary.get("accera_b200", {})
    if op.get("op") != "gather":
        return dim_value
    axis = int(op.get("axis", 0))
    for p in fn.arguments:
        if p.logical_type == "element" or p.usage != "input" or p.element_type == "int64_t":
            continue
        if p.logical_type == "affine_array" and p.shape and len(p.shape) == 2:
            return int(p.shape[axis])
        if p.logical_type == "runtime_array" and p.size:
            names = [t.strip() for t in p.size.split("*")]
            if len(names) == 2:
                tok = names[axis]
                return int(tok) if re.fullmatch(r"\d+", tok) else int(values.get(tok, dim_value))
    return dim_value


def generate_arg_values(fn: Function, rng: np.random.Generator, dim_value: int = 128):
    """Random inputs matching a function's descriptor (dimension arguments get `dim_value`; gather indices stay
    inside the gathered dimension)."""
    values: Dict[str, int] = {}
    for p in fn.arguments:
        if p.logical_type == "element" and p.usage == "input":
            values[p.name] = dim_value
    args = []
    for p in fn.arguments:
        if p.logical_type == "element":
            if p.usage == "input":
                args.append(values[p.name])
            else:
                args.append(np.zeros(1, dtype=_NP_OF_C[p.element_type]))
            continue
        dt = _NP_OF_C[p.element_type]
        if p.logical_type == "affine_array":
            shape = tuple(p.shape)
            fortran = len(shape) > 1 and p.affine_map[0] == 1 and p.affine_map[-1] != 1
        else:
            shape = (_eval_size(p.size or "", values),)
            fortran = False
        if p.element_type == "bfloat16_t":
            a = (rng.standard_normal(shape).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
        elif np.issubdtype(dt, np.floating):
            a = rng.random(shape).astype(dt)
        elif p.usage == "input" and "index" in p.name.lower() or (p.usage == "input" and dt == np.int64):
            a = rng.integers(0, max(1, _index_bound(fn, values, dim_value)), size=shape).astype(dt)       # valid gather indices
        else:
            info = np.iinfo(dt)
            a = rng.integers(max(info.min, -4), min(info.max, 4), size=shape).astype(dt)
        args.append(np.asfortranarray(a) if fortran else np.ascontiguousarray(a))
    return args


def _to_device(args, device):
    """numpy argument values -> torch tensors on `device` with the same shapes and element strides."""
    import torch
    out = []
    for a in args:
        if not isinstance(a, np.ndarray):
            out.append(a)
            continue
        if a.ndim >= 2 and a.flags.f_contiguous and not a.flags.c_contiguous:
            t = torch.from_numpy(np.ascontiguousarray(a.T)).to(device).t()      # keeps the column-major strides
        else:
            t = torch.from_numpy(np.ascontiguousarray(a)).to(device)
        out.append(t)
    return out


def _run_benchmark_on_device(fn: "HATFunction", rng, batch_size: int, min_time_in_sec: float, min_set_mb: int,
                             device_id: int) -> List[float]:
    """Batch means (seconds per call) with the arguments resident on the GPU, timed with CUDA events.  The
    calls rotate over several input sets that together exceed `min_set_mb`, so launches do not find their
    inputs in L2 (hatlib's input_sets_minimum_size_MB)."""
    import torch
    if not torch.cuda.is_available():
        raise RuntimeError("device_resident benchmarking needs a CUDA device")
    device = torch.device("cuda", device_id)
    first = generate_arg_values(fn.desc, rng)
    set_bytes = sum(a.nbytes for a in first if isinstance(a, np.ndarray)) or 1
    n_sets = int(min(8, max(1, -(-min_set_mb * (1 << 20) // set_bytes))))
    calls = []
    for i in range(n_sets):
        host = first if i == 0 else generate_arg_values(fn.desc, rng)
        dev_args = []
        for p, a in zip(fn.desc.arguments, host):
            if p.logical_type == "element":
                dev_args.append(a)                       # dimensions and output scalars stay on the host
            elif p.element_type == "bfloat16_t":
                dev_args.append(_to_device([a.view(np.int16)], device)[0].view(torch.bfloat16))
            else:
                dev_args.append(_to_device([a], device)[0])
        calls.append(fn.bind(*dev_args))
    with torch.cuda.device(device):
        for c in calls:
            c()
        torch.cuda.synchronize()
        batch_means: List[float] = []
        t_end = time.perf_counter() + float(min_time_in_sec)
        k = 0
        while len(batch_means) < 3 or time.perf_counter() < t_end:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(batch_size):
                calls[k % n_sets]()
                k += 1
            e1.record()
            e1.synchronize()
            batch_means.append(e0.elapsed_time(e1) * 1e-3 / batch_size)
            if len(batch_means) >= 100000:
                break
    from .. import runtime
    runtime.synchronize()                                # surfaces deferred device-side errors
    return batch_means


def run_benchmark(hat_path: str, store_in_hat: bool = False, batch_size: int = 10, min_time_in_sec: float = 10,
                  input_sets_minimum_size_MB: int = 50, device_id: int = 0, verbose: bool = False,
                  functions: Optional[List[str]] = None, device_resident: Optional[bool] = None) -> List[BenchmarkResult]:
    """Times every function of the package: batches of `batch_size` calls until `min_time_in_sec` has
    elapsed (at least 3 batches).  device_resident=True times on GPU-resident buffers with CUDA events, False on
    host arrays (each call then includes the library's host<->device staging).  The default follows hatlib: functions
    built for a GPU target are timed on the device, the others on host arrays."""
    _, fmap = load(hat_path)
    rng = np.random.default_rng(0)
    results = []
    for fn in fmap:
        if functions and fn.name not in functions:
            continue
        gpu_function = bool(fn.desc.launches) or fn.desc.auxiliary.get("accera_b200", {}).get("runtime") == "CUDA"
        on_device = device_resident if device_resident is not None else gpu_function
        if on_device:
            r = BenchmarkResult.from_batch_means(fn.name, _run_benchmark_on_device(fn, rng, batch_size, min_time_in_sec,
                                                                  input_sets_minimum_size_MB, device_id))
            if verbose:
                print(r.as_dict())
            results.append(r)
            continue
        args = generate_arg_values(fn.desc, rng)
        fn(*args, device_id=device_id)                 # warm-up (and first-touch of the staging workspace)
        batch_means: List[float] = []
        t_end = time.perf_counter() + float(min_time_in_sec)
        while len(batch_means) < 3 or time.perf_counter() < t_end:
            t0 = time.perf_counter()
            for _ in range(batch_size):
                fn(*args)
            batch_means.append((time.perf_counter() - t0) / batch_size)
            if len(batch_means) >= 100000:
                break
        r = BenchmarkResult.from_batch_means(fn.name, batch_means)
        if verbose:
            print(r.as_dict())
        results.append(r)
    return results
