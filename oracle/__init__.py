"""CPU oracle for the HAT GEMM(+ReLU) / reduce_mean / gather / range path.

TEST INFRASTRUCTURE ONLY: tests, the smoke check and the timed CPU baseline of
the benchmark use it as the checker; the product never imports it.

`hat_oracle.c` restates the reference's HOST-target loop nests in plain C (each
function cites the reference file:line it follows); this module binds it with
ctypes and adds the seeded input generators shared by the tests and the
benchmark so that the oracle and the GPU see identical bytes.

Parity status: pinned against the vectors in tests/golden/ (produced by the
reference's own numpy gather / range loops and by executing the reference's nest
definitions under a loop-nest interpreter) and against the two outputs of compiled
reference packages that its tutorials print (768.419983 and 1536.419922, which fix
the accumulation order of the fp32 matmul).  Beyond those two values, parity with
the reference's *compiled* HOST package is unpinned: it cannot be built offline.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))

F32, F16, BF16, S8, S32, U8, S16 = 0, 1, 2, 3, 4, 5, 6
EPI_NONE, EPI_RELU = 0, 1

_KIND_OF = {"float32": F32, "float16": F16, "bfloat16": BF16, "int8": S8, "int32": S32, "uint8": U8, "int16": S16}


def build(force: bool = False) -> None:
    """Compile hat_oracle.c into liborc_strict.so and liborc_fast.so (gcc)."""
    targets = [os.path.join(_HERE, n) for n in ("liborc_strict.so", "liborc_fast.so")]
    src = os.path.join(_HERE, "hat_oracle.c")
    if not force and all(os.path.exists(t) and os.path.getmtime(t) >= os.path.getmtime(src) for t in targets):
        return
    subprocess.run(["make", "-C", _HERE, "-B" if force else "-s"], check=True, capture_output=True)


_libs: dict = {}


def lib(fast: bool = False) -> ctypes.CDLL:
    name = "liborc_fast.so" if fast else "liborc_strict.so"
    if name not in _libs:
        path = os.path.join(_HERE, name)
        if not os.path.exists(path):
            build()
        L = ctypes.CDLL(path)
        i64, f32, vp, ci = ctypes.c_int64, ctypes.c_float, ctypes.c_void_p, ctypes.c_int
        L.orc_gemm_float.argtypes = [vp, vp, vp, ci, ci, ci, i64, i64, i64, i64, i64, i64, i64, i64, i64,
                                     f32, f32, vp, ci, i64, i64]
        L.orc_gemm_float.restype = None
        L.orc_gemm_int8.argtypes = [vp, vp, vp, ci, ci, i64, i64, i64, i64, i64, i64, i64, i64, i64, ci, ci, i64, i64]
        L.orc_gemm_int8.restype = None
        L.orc_reduce_mean_rank3.argtypes = [vp, i64, i64, i64, vp, ci]
        L.orc_reduce_mean_rank3.restype = None
        L.orc_reduce_mean_rank3_dims.argtypes = [i64, i64, i64, ci, ci, vp]
        L.orc_reduce_mean_rank3_dims.restype = ci
        L.orc_gather_rank2.argtypes = [vp, i64, i64, vp, i64, i64, vp, ci, i64]
        L.orc_gather_rank2.restype = None
        L.orc_gather_rank2_dims.argtypes = [i64, i64, i64, i64, ci, vp]
        L.orc_gather_rank2_dims.restype = None
        L.orc_range_count_f32.argtypes = [f32, f32, f32]
        L.orc_range_count_f32.restype = i64
        L.orc_range_f32.argtypes = [i64, vp, vp, f32]
        L.orc_range_f32.restype = None
        for n in ("orc_f32_to_bf16", "orc_bf16_to_f32", "orc_f32_to_f16", "orc_f16_to_f32"):
            getattr(L, n).argtypes = [vp, vp, i64]
            getattr(L, n).restype = None
        L.orc_max_threads.restype = ci
        L.orc_set_threads.argtypes = [ci]
        _libs[name] = L
    return _libs[name]


# ---------------------------------------------------------------------------
# bfloat16 helpers (numpy has no bfloat16: carried as uint16 bit patterns)
# ---------------------------------------------------------------------------

def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().orc_f32_to_bf16(x.ctypes.data, out.ctypes.data, x.size)
    return out


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    """Exact widening; keeps the memory order (C or Fortran) of the source."""
    return (np.asarray(b, dtype=np.uint16).astype(np.uint32, order="K") << 16).view(np.float32)


def _elem_strides(a: np.ndarray):
    return tuple(s // a.itemsize for s in a.strides)


def _ptr(a):
    return None if a is None else a.ctypes.data


# ---------------------------------------------------------------------------
# the three ops
# ---------------------------------------------------------------------------

def gemm(A: np.ndarray, B: np.ndarray, C: np.ndarray, *, in_kind: str = None, out_kind: str = None,
         alpha: float = 1.0, beta: float = 1.0, bias: np.ndarray = None, relu: bool = False,
         rows: tuple = None, fast: bool = False, threads: int = None) -> np.ndarray:
    """C <- epilogue(alpha * A @ B + beta * C) in place on a copy-free view; returns C.

    A is [M,K], B is [K,N], C is [M,N]; any of them may be Fortran-ordered (the
    reference's LAST_MAJOR layout) - the element strides are passed through.
    `in_kind`/`out_kind` name the element type when it cannot be read from the
    dtype ("bfloat16" arrays are uint16 bit patterns).  16-bit float inputs are
    widened exactly to fp32 before the call.  `rows=(m0, m1)` restricts the
    computation to that slice of output rows.
    """
    M, K = A.shape
    K2, N = B.shape
    assert K == K2 and C.shape == (M, N)
    in_kind = in_kind or str(A.dtype)
    out_kind = out_kind or str(C.dtype)
    L = lib(fast)
    if threads is not None:
        L.orc_set_threads(int(threads))
    m0, m1 = rows if rows is not None else (0, M)
    if in_kind in ("int8", "uint8", "int16"):
        assert out_kind == "int32" and alpha == 1.0 and beta in (0.0, 1.0) and bias is None
        sa, sb, sc = _elem_strides(A), _elem_strides(B), _elem_strides(C)
        L.orc_gemm_int8(A.ctypes.data, B.ctypes.data, C.ctypes.data, _KIND_OF[in_kind], _KIND_OF[in_kind],
                        M, N, K, sa[0], sa[1], sb[0], sb[1], sc[0], sc[1], int(beta == 0.0),
                        EPI_RELU if relu else EPI_NONE, m0, m1)
        return C
    if in_kind == "bfloat16":
        Af, Bf = _widen_bf16(A), _widen_bf16(B)
    elif in_kind == "float16":
        Af, Bf = _widen_f16(A), _widen_f16(B)
    else:
        Af, Bf = A, B
    sa, sb, sc = _elem_strides(Af), _elem_strides(Bf), _elem_strides(C)
    if bias is not None:
        bias = np.ascontiguousarray(bias, dtype=np.float32)
    L.orc_gemm_float(Af.ctypes.data, Bf.ctypes.data, C.ctypes.data, F32, F32, _KIND_OF[out_kind],
                     M, N, K, sa[0], sa[1], sb[0], sb[1], sc[0], sc[1],
                     float(alpha), float(beta), _ptr(bias), EPI_RELU if relu else EPI_NONE, m0, m1)
    return C


def _widen_bf16(x):
    return bf16_bits_to_f32(x)


def _widen_f16(x):
    return x.astype(np.float32, order="K")


def reduce_mean_rank3(data: np.ndarray, axes, keepdims: int = 1, fast: bool = False, threads: int = None) -> np.ndarray:
    """ONNX ReduceMean over a rank-3 fp32 array; sequential fp32 sum in index order."""
    data = np.ascontiguousarray(data, dtype=np.float32)
    assert data.ndim == 3
    axes = list(range(3)) if not axes else [a % 3 for a in axes]
    mask = sum(1 << a for a in set(axes))
    L = lib(fast)
    if threads is not None:
        L.orc_set_threads(int(threads))
    dims = (ctypes.c_int64 * 3)()
    n = L.orc_reduce_mean_rank3_dims(*data.shape, mask, int(keepdims), dims)
    out = np.empty(tuple(dims[i] for i in range(n)), dtype=np.float32)
    L.orc_reduce_mean_rank3(data.ctypes.data, *data.shape, out.ctypes.data, mask)
    return out


def reduce_mean_last_axis(x: np.ndarray, fast: bool = False, threads: int = None) -> np.ndarray:
    """Y[r] = mean(X[r, :]) for a rank-2 array, through the rank-3 function as dims (1, R, C), axes=[2], keepdims=0."""
    r, c = x.shape
    return reduce_mean_rank3(x.reshape(1, r, c), [2], 0, fast=fast, threads=threads).reshape(r)


def gather_rank2(data: np.ndarray, indices: np.ndarray, axis: int = 0, fast: bool = False, threads: int = None) -> np.ndarray:
    data = np.ascontiguousarray(data)
    indices = np.ascontiguousarray(indices, dtype=np.int64)
    assert data.ndim == 2 and indices.ndim == 2 and axis in (0, 1)
    L = lib(fast)
    if threads is not None:
        L.orc_set_threads(int(threads))
    dims = (ctypes.c_int64 * 3)()
    L.orc_gather_rank2_dims(*data.shape, *indices.shape, axis, dims)
    out = np.empty(tuple(dims), dtype=data.dtype)
    L.orc_gather_rank2(data.ctypes.data, *data.shape, indices.ctypes.data, *indices.shape, out.ctypes.data, axis,
                       data.itemsize)
    return out


def range_count(start, limit, delta) -> int:
    """Number of elements of Range(start, limit, delta): floor((limit - start) / delta) in fp32."""
    return int(lib().orc_range_count_f32(float(np.float32(start)), float(np.float32(limit)), float(np.float32(delta))))


def range_f32(start, delta, n: int):
    """-> (output[n], value of the running scalar after n additions): output[i] = start + delta + ... (i times),
    every addition rounded to fp32 in index order."""
    out = np.empty(int(n), dtype=np.float32)
    s = np.array([start], dtype=np.float32)
    lib().orc_range_f32(int(n), out.ctypes.data, s.ctypes.data, float(np.float32(delta)))
    return out, np.float32(s[0])


def max_threads() -> int:
    return int(lib().orc_max_threads())


# ---------------------------------------------------------------------------
# seeded inputs of the benchmark configurations (identical bytes for the oracle
# and the GPU).  Seeds are 1000 + configuration number.
# ---------------------------------------------------------------------------

def inputs_matmul_relu_f32(m=512, n=512, k=512, seed=1001):
    """Quickstart case: A, B ~ U[0,1) fp32 row-major, C zeros."""
    rng = np.random.default_rng(seed)
    A = rng.random((m, k), dtype=np.float32)
    B = rng.random((k, n), dtype=np.float32)
    C = np.zeros((m, n), dtype=np.float32)
    return A, B, C


def inputs_reduce_mean(rows=8192, cols=4096, seed=1002):
    """X ~ N(0,1) fp32 [rows, cols]."""
    rng = np.random.default_rng(seed)
    return rng.standard_normal((rows, cols), dtype=np.float32)


def inputs_gather(table_rows=32000, cols=4096, n_idx=16384, seed=1002):
    """T ~ N(0, 0.02) fp32 [table_rows, cols]; indices ~ U{0..table_rows-1} int64 [n_idx, 1]."""
    rng = np.random.default_rng(seed + 50)
    T = rng.standard_normal((table_rows, cols), dtype=np.float32)
    T *= np.float32(0.02)
    idx = rng.integers(0, table_rows, size=(n_idx, 1), dtype=np.int64)
    return T, idx


def inputs_gemm_f16(m=4096, n=4096, k=4096, seed=1003):
    """A (row-major), B (column-major) ~ U[-1,1) fp16; C zeros fp32."""
    rng = np.random.default_rng(seed)
    A = (rng.random((m, k), dtype=np.float32) * 2 - 1).astype(np.float16)
    B = np.asfortranarray((rng.random((k, n), dtype=np.float32) * 2 - 1).astype(np.float16))
    C = np.zeros((m, n), dtype=np.float32)
    return A, B, C


def inputs_gemm_s8(m=8192, n=8192, k=8192, seed=1004):
    """A (row-major), B (column-major) ~ U{-128..127} int8; C zeros int32."""
    rng = np.random.default_rng(seed)
    A = rng.integers(-128, 128, size=(m, k), dtype=np.int8)
    B = np.asfortranarray(rng.integers(-128, 128, size=(k, n), dtype=np.int8))
    C = np.zeros((m, n), dtype=np.int32)
    return A, B, C


def inputs_gemm_bf16(m=65536, n=8192, k=8192, seed=1005):
    """A ~ N(0,1) bf16 row-major, B ~ N(0, 1/sqrt(K)) bf16 column-major, as uint16 bit patterns; C zeros bf16."""
    rng = np.random.default_rng(seed)
    A = f32_to_bf16_bits(rng.standard_normal((m, k), dtype=np.float32))
    Bt = rng.standard_normal((n, k), dtype=np.float32)          # generated K-contiguous, viewed as [K, N] below
    Bt *= np.float32(1.0 / np.sqrt(k))
    B = f32_to_bf16_bits(Bt).T                                   # [K, N] column-major view
    C = np.zeros((m, n), dtype=np.uint16)
    return A, B, C
