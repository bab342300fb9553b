"""ctypes binding of libaccera_b200.so (the C ABI declared in include/accera_b200.h).

This is the Python face of the launch layer that replaces the reference's
accera/runtime + acc-gpu-runner + hatlib device plumbing for the GEMM(+ReLU),
reduce_mean and gather functions.  Arrays may be numpy arrays (host memory: the
library stages them through the GPU and the call is synchronous) or torch CUDA
tensors (used in place, enqueued on torch's current stream, not synchronised).

There is no CPU fallback: if the library is missing or no B200 is visible every
compute call raises.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import numpy as np

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libaccera_b200.so")

F32, F16, BF16, S8, S32, U8, S16 = 0, 1, 2, 3, 4, 5, 6
COMPUTE_AUTO, COMPUTE_SIMT, COMPUTE_TENSOR, COMPUTE_TENSOR_2SM, COMPUTE_TENSOR_PREFERRED = 0, 1, 2, 3, 4
EPI_NONE, EPI_RELU = 0, 1
ERR_ARG, ERR_CUDA, ERR_INDEX, ERR_TIMEOUT, ERR_LIMIT = -1, -2, -3, -4, -5

TYPE_BYTES = {F32: 4, F16: 2, BF16: 2, S8: 1, S32: 4, U8: 1, S16: 2}
_NP_TYPE = {"float32": F32, "float16": F16, "int8": S8, "int32": S32, "uint8": U8, "int16": S16}
_COMPUTE = {"auto": COMPUTE_AUTO, "simt": COMPUTE_SIMT, "tensor": COMPUTE_TENSOR, "tensor_2sm": COMPUTE_TENSOR_2SM,
            "tensor_preferred": COMPUTE_TENSOR_PREFERRED}

EXPORTED_SYMBOLS = (
    "accb_gemm", "accb_gemm_batched", "accb_gemm_tile_plan", "accb_gemm_launch_geometry", "accb_gemm_replicated", "accb_reduce_mean_rank3", "accb_reduce_mean_rank3_noalloc", "accb_reduce_mean_rank3_dims", "accb_gather_rank2",
    "accb_gather_rank2_dims", "accb_range_count_f32", "accb_range_f32", "accb_range_plan_f32", "accb_set_device", "accb_get_device", "accb_current_device", "accb_set_stream", "accb_synchronize", "accb_last_error",
    "accb_launch_count", "accb_release_workspace", "accb_device_count", "accb_version", "accb_set_option", "accb_debug_decode_status",
)


class AccbError(RuntimeError):
    """A C-ABI entry point returned a negative status."""

    def __init__(self, code: int, message: str):
        super().__init__(f"[{code}] {message}")
        self.code = code


class GemmDesc(ctypes.Structure):
    _fields_ = [
        ("m", ctypes.c_int64), ("n", ctypes.c_int64), ("k", ctypes.c_int64),
        ("a_type", ctypes.c_int32), ("b_type", ctypes.c_int32), ("c_type", ctypes.c_int32),
        ("compute", ctypes.c_int32),
        ("a_stride", ctypes.c_int64 * 2), ("b_stride", ctypes.c_int64 * 2), ("c_stride", ctypes.c_int64 * 2),
        ("alpha", ctypes.c_float), ("beta", ctypes.c_float),
        ("epilogue", ctypes.c_int32), ("max_ctas", ctypes.c_int32),
    ]


_lib: Optional[ctypes.CDLL] = None


def lib() -> ctypes.CDLL:
    """Loads the library (building it first when the sources are newer and nvcc is present)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        from . import build as _build
        _build.build()
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(f"{LIB_PATH} is missing: run `python -m accera_b200.build` (needs nvcc); there is no CPU fallback")
    L = ctypes.CDLL(LIB_PATH)
    vp, i64, i32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32
    L.accb_gemm.argtypes = [ctypes.POINTER(GemmDesc), vp, vp, vp, vp]
    L.accb_gemm.restype = ctypes.c_int
    L.accb_gemm_batched.argtypes = [ctypes.POINTER(GemmDesc), i64, i64, i64, i64, vp, vp, vp, vp]
    L.accb_gemm_batched.restype = ctypes.c_int
    L.accb_gemm_tile_plan.argtypes = [ctypes.POINTER(GemmDesc), i64, i32, ctypes.POINTER(i32), ctypes.POINTER(i32),
                                      ctypes.POINTER(i64), ctypes.POINTER(i64)]
    L.accb_gemm_tile_plan.restype = ctypes.c_int
    L.accb_gemm_launch_geometry.argtypes = [ctypes.POINTER(GemmDesc), i64, i32, ctypes.POINTER(i32), ctypes.POINTER(i32),
                                            ctypes.POINTER(i32)]
    L.accb_gemm_launch_geometry.restype = ctypes.c_int
    L.accb_gemm_replicated.argtypes = [ctypes.POINTER(GemmDesc), vp, vp, ctypes.POINTER(vp), i32, vp]
    L.accb_gemm_replicated.restype = ctypes.c_int
    L.accb_reduce_mean_rank3.argtypes = [vp, i64, i64, i64, vp, i32]
    L.accb_reduce_mean_rank3.restype = ctypes.c_int
    L.accb_reduce_mean_rank3_noalloc.argtypes = [vp, i64, i64, i64, vp, i32, vp]
    L.accb_reduce_mean_rank3_noalloc.restype = ctypes.c_int
    L.accb_reduce_mean_rank3_dims.argtypes = [i64, i64, i64, i32, i32, ctypes.POINTER(i64)]
    L.accb_reduce_mean_rank3_dims.restype = ctypes.c_int
    L.accb_gather_rank2.argtypes = [vp, i64, i64, vp, i64, i64, vp, i32, i32]
    L.accb_gather_rank2.restype = ctypes.c_int
    L.accb_gather_rank2_dims.argtypes = [i64, i64, i64, i64, i32, ctypes.POINTER(i64)]
    L.accb_gather_rank2_dims.restype = ctypes.c_int
    L.accb_range_count_f32.argtypes = [ctypes.c_float, ctypes.c_float, ctypes.c_float]
    L.accb_range_count_f32.restype = ctypes.c_int64
    L.accb_range_plan_f32.argtypes = [ctypes.c_float, ctypes.c_float, i64, vp, vp, vp, i64, vp]
    L.accb_range_plan_f32.restype = ctypes.c_int64
    L.accb_range_f32.argtypes = [i64, vp, vp, ctypes.c_float]
    L.accb_range_f32.restype = ctypes.c_int
    L.accb_set_device.argtypes = [i32]
    L.accb_set_device.restype = ctypes.c_int
    L.accb_get_device.restype = ctypes.c_int
    L.accb_current_device.restype = ctypes.c_int
    L.accb_set_option.argtypes = [ctypes.c_char_p, i64]
    L.accb_set_option.restype = ctypes.c_int
    L.accb_debug_decode_status.argtypes = [ctypes.POINTER(i32), i32, i32, ctypes.c_char_p, i32]
    L.accb_debug_decode_status.restype = ctypes.c_int
    L.accb_set_stream.argtypes = [vp]
    L.accb_set_stream.restype = ctypes.c_int
    L.accb_synchronize.restype = ctypes.c_int
    L.accb_last_error.restype = ctypes.c_char_p
    L.accb_launch_count.restype = ctypes.c_int64
    L.accb_release_workspace.restype = ctypes.c_int
    L.accb_device_count.restype = ctypes.c_int
    L.accb_version.restype = ctypes.c_char_p
    _lib = L
    return L


def _check(rc: int) -> None:
    if rc < 0:
        raise AccbError(rc, lib().accb_last_error().decode())


def device_count() -> int:
    return int(lib().accb_device_count())


def launch_count() -> int:
    return int(lib().accb_launch_count())


def set_device(device: int) -> None:
    _check(lib().accb_set_device(int(device)))


def selected_device() -> int:
    """The device this thread selected with set_device, -1 if none (calls then follow the current CUDA device)."""
    return int(lib().accb_get_device())


def current_device() -> int:
    """The CUDA runtime's current device of this thread."""
    d = int(lib().accb_current_device())
    if d < 0:
        raise AccbError(d, "no usable CUDA device")
    return d


def set_stream(stream_handle: int) -> None:
    _check(lib().accb_set_stream(ctypes.c_void_p(int(stream_handle) or None)))


def set_option(name: str, value: int) -> None:
    """Per-thread override of a choice the launch code otherwise makes itself (see accb_set_option in
    include/accera_b200.h); set_option("reset", 0) restores every default."""
    _check(lib().accb_set_option(name.encode(), int(value)))


class options:
    """Context manager: `with options(**{"gemm.tile_cols": 128}): ...` sets the overrides and resets ALL of them on exit."""

    def __init__(self, **kv):
        self._kv = kv

    def __enter__(self):
        for k, v in self._kv.items():
            set_option(k.replace("__", "."), v)
        return self

    def __exit__(self, *exc):
        set_option("reset", 0)
        return False


def decode_status(words, what: int = 0, launch_id: int = 0):
    """-> (code, message) the library derives from eight device status words (host only; for tests)."""
    arr = (ctypes.c_int32 * 8)(*[int(w) for w in words])
    buf = ctypes.create_string_buffer(512)
    rc = lib().accb_debug_decode_status(arr, int(what), int(launch_id), buf, 512)
    return int(rc), buf.value.decode()


def synchronize() -> None:
    _check(lib().accb_synchronize())


def release_workspace() -> None:
    _check(lib().accb_release_workspace())


# ---------------------------------------------------------------------------
# array adaptors
# ---------------------------------------------------------------------------

def _is_torch(x) -> bool:
    return type(x).__module__.split(".")[0] == "torch"


def _describe(x, kind: Optional[str] = None):
    """-> (pointer, element type code, shape, element strides, is_device)."""
    if _is_torch(x):
        import torch
        tmap = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16, torch.int8: S8, torch.int32: S32,
                torch.uint8: U8, torch.int16: S16}
        if kind is not None:
            code = {"bfloat16": BF16, "float16": F16, "float32": F32, "int8": S8, "uint8": U8, "int32": S32, "int16": S16}[kind]
        elif x.dtype in tmap:
            code = tmap[x.dtype]
        elif x.dtype == torch.int64:
            code = None
        else:
            raise TypeError(f"unsupported tensor dtype {x.dtype}")
        return x.data_ptr(), code, tuple(x.shape), tuple(x.stride()), x.is_cuda
    a = x
    if not isinstance(a, np.ndarray):
        raise TypeError("expected a numpy array or a torch tensor")
    if kind == "bfloat16":
        if a.dtype != np.uint16:
            raise TypeError("bfloat16 numpy arrays are passed as uint16 bit patterns")
        code = BF16
    elif a.dtype == np.int64:
        code = None
    else:
        code = _NP_TYPE.get(str(a.dtype))
        if code is None:
            raise TypeError(f"unsupported array dtype {a.dtype}")
    return a.ctypes.data, code, a.shape, tuple(s // a.itemsize for s in a.strides), False


def _raw(x):
    """-> (pointer, shape, element size) of a dense first-major array of any element type."""
    if _is_torch(x):
        if not x.is_contiguous():
            raise ValueError("expected a contiguous tensor")
        return x.data_ptr(), tuple(x.shape), x.element_size()
    if not isinstance(x, np.ndarray):
        raise TypeError("expected a numpy array or a torch tensor")
    if not x.flags.c_contiguous:
        raise ValueError("expected a C-contiguous array")
    return x.ctypes.data, x.shape, x.itemsize


def _sync_torch_stream(*arrays) -> None:
    """Device-pointer calls run on torch's current stream of the tensors' device; calls on host arrays run on
    the default stream (a stream selected for an earlier device-pointer call is not carried over: it may
    belong to another device or no longer exist)."""
    for x in arrays:
        if _is_torch(x) and x.is_cuda:
            import torch
            set_device(x.device.index)
            set_stream(torch.cuda.current_stream(x.device).cuda_stream)
            return
    set_stream(0)


def _captured_selection(*arrays):
    """-> (device index or None, stream as c_void_p) for a callable that repeats a call on these arrays later:
    torch's current stream of the tensors' device now; the default stream and no device change for host arrays."""
    for x in arrays:
        if _is_torch(x) and x.is_cuda:
            import torch
            return x.device.index, ctypes.c_void_p(torch.cuda.current_stream(x.device).cuda_stream or None)
    return None, ctypes.c_void_p(None)


# ---------------------------------------------------------------------------
# the three ops
# ---------------------------------------------------------------------------

def _gemm_args(A, B, C, bias, alpha, beta, relu, compute, kind, out_kind, max_ctas):
    pa, ta, sha, sta, da = _describe(A, kind)
    pb, tb, shb, stb, db = _describe(B, kind)
    pc, tc, shc, stc, dc = _describe(C, out_kind)
    if len(sha) != 2 or len(shb) != 2 or len(shc) != 2:
        raise ValueError("gemm operands must be rank 2")
    m, k = sha
    k2, n = shb
    if k2 != k or tuple(shc) != (m, n):
        raise ValueError(f"shape mismatch: A{sha} B{shb} C{shc}")
    pbias = None
    if bias is not None:
        pbias, tbias, shbias, _, _ = _describe(bias)
        if tbias != F32 or tuple(shbias) != (n,):
            raise ValueError("bias must be fp32 of length N")
    d = GemmDesc()
    d.m, d.n, d.k = m, n, k
    d.a_type, d.b_type, d.c_type = ta, tb, tc
    d.compute = _COMPUTE[compute]
    d.a_stride[0], d.a_stride[1] = max(sta[0], 1), max(sta[1], 1)
    d.b_stride[0], d.b_stride[1] = max(stb[0], 1), max(stb[1], 1)
    d.c_stride[0], d.c_stride[1] = max(stc[0], 1), max(stc[1], 1)
    d.alpha, d.beta = alpha, beta
    d.epilogue = EPI_RELU if relu else EPI_NONE
    d.max_ctas = int(max_ctas)
    return d, pa, pb, pc, pbias


def gemm(A, B, C, *, bias=None, alpha: float = 1.0, beta: float = 1.0, relu: bool = False, compute: str = "auto",
         kind: Optional[str] = None, out_kind: Optional[str] = None, max_ctas: int = 0) -> None:
    """C <- epi(alpha * A @ B + beta * C + bias), in place in C.

    A [M,K], B [K,N], C [M,N]; strides are taken from the arrays, so a Fortran-
    ordered B is the reference's LAST_MAJOR layout.  `kind`/`out_kind` = "bfloat16"
    marks uint16 numpy arrays as bf16 bit patterns.  `max_ctas` bounds the tensor-core kernel's persistent
    grid (0 = every SM), to leave SMs for a collective that runs concurrently.
    """
    d, pa, pb, pc, pbias = _gemm_args(A, B, C, bias, alpha, beta, relu, compute, kind, out_kind, max_ctas)
    _sync_torch_stream(A, B, C)
    _check(lib().accb_gemm(ctypes.byref(d), pa, pb, pc, pbias))


def gemm_tile_plan(m: int, n: int, k: int, *, in_type: str = "bfloat16", compute: str = "auto", batch: int = 1,
                   num_sms: int = 148, b_row_major: bool = False, max_ctas: int = 0) -> dict:
    """The tile shape the tensor-core path picks for an M x N x K problem (host only, no GPU needed):
    {"cta_pairs", "tile_cols", "tiles", "rounds"}."""
    d = GemmDesc()
    d.m, d.n, d.k = m, n, k
    t = {"bfloat16": BF16, "float16": F16, "float32": F32, "int8": S8, "uint8": U8}[in_type]
    d.a_type = d.b_type = t
    d.c_type = S32 if t in (S8, U8) else t
    d.compute = _COMPUTE[compute]
    d.a_stride[0], d.a_stride[1] = k, 1
    d.b_stride[0], d.b_stride[1] = (n, 1) if b_row_major else (1, k)
    d.c_stride[0], d.c_stride[1] = n, 1
    d.alpha, d.beta, d.epilogue, d.max_ctas = 1.0, 0.0, EPI_NONE, int(max_ctas)
    pairs, cols = ctypes.c_int32(), ctypes.c_int32()
    tiles, rounds = ctypes.c_int64(), ctypes.c_int64()
    _check(lib().accb_gemm_tile_plan(ctypes.byref(d), int(batch), int(num_sms), ctypes.byref(pairs), ctypes.byref(cols),
                                     ctypes.byref(tiles), ctypes.byref(rounds)))
    return {"cta_pairs": bool(pairs.value), "tile_cols": cols.value, "tiles": tiles.value, "rounds": rounds.value}


def gemm_launch_geometry(m: int, n: int, k: int, *, in_type: str = "bfloat16", compute: str = "auto", batch: int = 1,
                         num_sms: int = 148, b_row_major: bool = False, max_ctas: int = 0) -> dict:
    """Grid, block and dynamic shared memory of the tensor-core launch for an M x N x K problem (host only):
    {"grid": [x, y, z], "block": [x, y, z], "dynamic_shared_mem_bytes"}."""
    d = GemmDesc()
    d.m, d.n, d.k = m, n, k
    t = {"bfloat16": BF16, "float16": F16, "float32": F32, "int8": S8, "uint8": U8}[in_type]
    d.a_type = d.b_type = t
    d.c_type = S32 if t in (S8, U8) else t
    d.compute = _COMPUTE[compute]
    d.a_stride[0], d.a_stride[1] = k, 1
    d.b_stride[0], d.b_stride[1] = (n, 1) if b_row_major else (1, k)
    d.c_stride[0], d.c_stride[1] = n, 1
    d.alpha, d.beta, d.epilogue, d.max_ctas = 1.0, 0.0, EPI_NONE, int(max_ctas)
    grid, block = (ctypes.c_int32 * 3)(), (ctypes.c_int32 * 3)()
    smem = ctypes.c_int32()
    _check(lib().accb_gemm_launch_geometry(ctypes.byref(d), int(batch), int(num_sms), grid, block, ctypes.byref(smem)))
    return {"grid": list(grid), "block": list(block), "dynamic_shared_mem_bytes": smem.value}


def gemm_call(A, B, C, *, bias=None, alpha: float = 1.0, beta: float = 1.0, relu: bool = False, compute: str = "auto",
              kind: Optional[str] = None, out_kind: Optional[str] = None, max_ctas: int = 0):
    """-> a zero-argument callable that repeats this GEMM on the same arrays.

    The descriptor is filled and the device / stream selected once, now; each later call is only the C-ABI call,
    which is what a compiled HAT stub does (its descriptor is a constant).  For timing loops and for callers
    that issue the same GEMM many times.  The arrays must stay alive and in place; for device tensors the stream
    is torch's current stream at the time of THIS call (it is re-selected before every repeat).
    """
    d, pa, pb, pc, pbias = _gemm_args(A, B, C, bias, alpha, beta, relu, compute, kind, out_kind, max_ctas)
    dev, stream = _captured_selection(A, B, C)
    L = lib()
    fn = L.accb_gemm
    set_dev, set_str = L.accb_set_device, L.accb_set_stream
    ref = ctypes.byref(d)
    keep = (A, B, C, bias, d)

    def call() -> None:
        # another call of this thread may have selected a different device or stream in between
        if dev is not None:
            set_dev(dev)
        set_str(stream)
        rc = fn(ref, pa, pb, pc, pbias)
        if rc < 0:
            _check(rc)
    call.keep_alive = keep
    return call


def gemm_batched(A, B, C, *, bias=None, alpha: float = 1.0, beta: float = 1.0, relu: bool = False,
                 compute: str = "auto", kind: Optional[str] = None, out_kind: Optional[str] = None,
                 max_ctas: int = 0) -> None:
    """C[b] <- epi(alpha * A[b] @ B[b] + beta * C[b] + bias) for every b, in place in C.

    A [batch, M, K], B [batch, K, N], C [batch, M, N]: rank-3 arrays whose first stride is the batch
    stride; the other two are the matrix strides, as for `gemm`.  A or B may also be rank 2 (or have
    batch stride 0, e.g. an expanded tensor): that operand is shared by all problems.
    """
    pa, ta, sha, sta, _ = _describe(A, kind)
    pb, tb, shb, stb, _ = _describe(B, kind)
    pc, tc, shc, stc, _ = _describe(C, out_kind)
    if len(shc) != 3 or len(sha) not in (2, 3) or len(shb) not in (2, 3):
        raise ValueError("gemm_batched: C must be rank 3, A and B rank 2 or 3")
    batch, m, n = shc
    if len(sha) == 2:
        sha, sta = (batch,) + tuple(sha), (0,) + tuple(sta)
    if len(shb) == 2:
        shb, stb = (batch,) + tuple(shb), (0,) + tuple(stb)
    k = sha[2]
    if tuple(sha) != (batch, m, k) or tuple(shb) != (batch, k, n):
        raise ValueError(f"shape mismatch: A{tuple(sha)} B{tuple(shb)} C{tuple(shc)}")
    pbias = None
    if bias is not None:
        pbias, tbias, shbias, _, _ = _describe(bias)
        if tbias != F32 or tuple(shbias) != (n,):
            raise ValueError("bias must be fp32 of length N")
    d = GemmDesc()
    d.m, d.n, d.k = m, n, k
    d.a_type, d.b_type, d.c_type = ta, tb, tc
    d.compute = _COMPUTE[compute]
    d.a_stride[0], d.a_stride[1] = max(sta[1], 1), max(sta[2], 1)
    d.b_stride[0], d.b_stride[1] = max(stb[1], 1), max(stb[2], 1)
    d.c_stride[0], d.c_stride[1] = max(stc[1], 1), max(stc[2], 1)
    d.alpha, d.beta = alpha, beta
    d.epilogue = EPI_RELU if relu else EPI_NONE
    d.max_ctas = int(max_ctas)
    # a batch of one problem has no meaningful batch stride (torch reports any value for a size-1 dimension)
    a_bs, b_bs, c_bs = (0, 0, 0) if batch <= 1 else (sta[0], stb[0], stc[0])
    _sync_torch_stream(A, B, C)
    _check(lib().accb_gemm_batched(ctypes.byref(d), batch, a_bs, b_bs, c_bs, pa, pb, pc, pbias))


def gemm_replicated(A, B, C_replicas, *, bias=None, alpha: float = 1.0, beta: float = 1.0, relu: bool = False,
                    compute: str = "tensor_2sm", max_ctas: int = 0) -> None:
    """Tensor-core GEMM whose result is stored to every tensor of `C_replicas` (torch CUDA tensors with
    identical shape and strides; replica 0 is the local C and is read when beta != 0, the others may be
    peer / symmetric memory of other GPUs and are only written)."""
    pa, ta, sha, sta, _ = _describe(A)
    pb, tb, shb, stb, _ = _describe(B)
    c0 = C_replicas[0]
    pc, tc, shc, stc, _ = _describe(c0)
    m, k = sha
    k2, n = shb
    if k2 != k or tuple(shc) != (m, n):
        raise ValueError(f"shape mismatch: A{sha} B{shb} C{shc}")
    ptrs = (ctypes.c_void_p * len(C_replicas))()
    for i, c in enumerate(C_replicas):
        if tuple(c.shape) != (m, n) or tuple(c.stride()) != tuple(c0.stride()) or c.dtype != c0.dtype:
            raise ValueError("all C replicas must have the same shape, strides and dtype")
        ptrs[i] = c.data_ptr()
    pbias = None
    if bias is not None:
        pbias, tbias, shbias, _, _ = _describe(bias)
        if tbias != F32 or tuple(shbias) != (n,):
            raise ValueError("bias must be fp32 of length N")
    d = GemmDesc()
    d.m, d.n, d.k = m, n, k
    d.a_type, d.b_type, d.c_type = ta, tb, tc
    d.compute = _COMPUTE[compute]
    d.a_stride[0], d.a_stride[1] = max(sta[0], 1), max(sta[1], 1)
    d.b_stride[0], d.b_stride[1] = max(stb[0], 1), max(stb[1], 1)
    d.c_stride[0], d.c_stride[1] = max(stc[0], 1), max(stc[1], 1)
    d.alpha, d.beta = alpha, beta
    d.epilogue = EPI_RELU if relu else EPI_NONE
    d.max_ctas = int(max_ctas)
    _sync_torch_stream(A, B, c0)
    _check(lib().accb_gemm_replicated(ctypes.byref(d), pa, pb, ptrs, len(C_replicas), pbias))


def reduce_mean_rank3_dims(d0: int, d1: int, d2: int, axes, keepdims: int = 1):
    axes = list(range(3)) if not axes else [a % 3 for a in axes]
    mask = sum(1 << a for a in set(axes))
    out = (ctypes.c_int64 * 3)()
    n = lib().accb_reduce_mean_rank3_dims(d0, d1, d2, mask, int(keepdims), out)
    _check(n)
    return tuple(out[i] for i in range(n)), mask


def reduce_mean_rank3(data, reduced, axes) -> None:
    """reduced <- mean of rank-3 fp32 `data` over `axes` (ONNX ReduceMean; empty axes = all)."""
    pd, td, shd, std_, dd = _describe(data)
    pr, tr, shr, str_, dr = _describe(reduced)
    if td != F32 or tr != F32 or len(shd) != 3:
        raise ValueError("reduce_mean_rank3 takes a rank-3 fp32 array")
    axes = list(range(3)) if not axes else [a % 3 for a in axes]
    mask = sum(1 << a for a in set(axes))
    _sync_torch_stream(data, reduced)
    _check(lib().accb_reduce_mean_rank3(pd, shd[0], shd[1], shd[2], pr, mask))


def reduce_mean_rank3_noalloc(data, reduced, axes, stream_handle: Optional[int] = None) -> None:
    """Like reduce_mean_rank3 for torch CUDA tensors, through the entry point that never allocates device
    memory (partial sums go to a 256 KiB array built into the library).  For hosts that own all device
    memory themselves.  Shapes that would need more scratch raise AccbError(ERR_LIMIT); calls that overlap
    on the GPU race on the shared array.  Enqueued on `stream_handle` (default: torch's current stream)."""
    pd, td, shd, _, dd = _describe(data)
    pr, tr, _, _, dr = _describe(reduced)
    if td != F32 or tr != F32 or len(shd) != 3:
        raise ValueError("reduce_mean_rank3_noalloc takes a rank-3 fp32 array")
    axes = list(range(3)) if not axes else [a % 3 for a in axes]
    mask = sum(1 << a for a in set(axes))
    if stream_handle is None and _is_torch(data) and data.is_cuda:
        import torch
        set_device(data.device.index)
        stream_handle = torch.cuda.current_stream(data.device).cuda_stream
    _check(lib().accb_reduce_mean_rank3_noalloc(pd, shd[0], shd[1], shd[2], pr, mask,
                                                ctypes.c_void_p(int(stream_handle or 0) or None)))


def gather_rank2(data, indices, output, axis: int = 0) -> None:
    """output <- gather(data, indices, axis) for rank-2 data and rank-2 int64 indices."""
    pd, shd, esize = _raw(data)
    pi, shi, isize = _raw(indices)
    po, sho, osize = _raw(output)
    idx_dtype = str(indices.dtype)
    if "int64" not in idx_dtype:
        raise TypeError("indices must be int64")
    if len(shd) != 2 or len(shi) != 2:
        raise ValueError("gather_rank2 takes rank-2 data and rank-2 indices")
    if osize != esize:
        raise TypeError("output element size differs from data element size")
    _sync_torch_stream(data, indices, output)
    _check(lib().accb_gather_rank2(pd, shd[0], shd[1], pi, shi[0], shi[1], po, int(axis), int(esize)))


def range_count(start, limit, delta) -> int:
    """Number of elements of Range(start, limit, delta): floor((limit - start) / delta) in fp32 (host only)."""
    return int(lib().accb_range_count_f32(float(np.float32(start)), float(np.float32(limit)), float(np.float32(delta))))


def range_plan(start, delta, n: int):
    """-> (first[int64], bits[uint32], step[int32], final fp32): the segments of constant bit-pattern step that
    the range kernel fills (host only; no GPU needed)."""
    s, d = float(np.float32(start)), float(np.float32(delta))
    final = np.zeros(1, dtype=np.float32)
    count = int(lib().accb_range_plan_f32(s, d, int(n), None, None, None, 0, final.ctypes.data))
    first = np.zeros(count, dtype=np.int64)
    bits = np.zeros(count, dtype=np.uint32)
    step = np.zeros(count, dtype=np.int32)
    lib().accb_range_plan_f32(s, d, int(n), first.ctypes.data, bits.ctypes.data, step.ctypes.data, count, final.ctypes.data)
    return first, bits, step, np.float32(final[0])


def range_f32(output, start, delta) -> np.float32:
    """Fills the 1-D fp32 `output` (numpy array or torch CUDA tensor) with start, start + delta, ... where every
    addition is rounded to fp32 in index order; returns the running value after the last addition."""
    ptr, shape, es = _raw(output)
    if es != 4 or len(shape) != 1:
        raise ValueError("range_f32 fills a one-dimensional fp32 array")
    s = np.array([start], dtype=np.float32)
    _sync_torch_stream(output)
    _check(lib().accb_range_f32(int(shape[0]), ptr, s.ctypes.data, float(np.float32(delta))))
    return np.float32(s[0])


def gather_rank2_dims(d0: int, d1: int, i0: int, i1: int, axis: int):
    out = (ctypes.c_int64 * 3)()
    _check(lib().accb_gather_rank2_dims(d0, d1, i0, i1, int(axis), out))
    return tuple(out)
