"""Recognises the operator a traced nest / schedule / plan describes.

The reference lowers arbitrary loop nests through MLIR.  This package does not:
it accepts exactly the operator families that its hand-written kernels cover and
rejects everything else with a clear error.  Recognised forms (reference sources
of each form in parentheses):

  matmul          C[i,j] += A[i,k] * B[k,j]           (README.md:61-65; operands may be accessed
                                                       transposed, int_matmul_tests.py:55 uses B[j,k];
                                                       casts around operands or the product are allowed)
  batch matmul    C[b,i,j] += A[b,i,k] * B[b,k,j]      (mfma_tests.py:435-466; any index order inside an
                                                       access; an operand without b is shared by the batch)
  + bias          C[i,j] += bias[j]                    (new: the reference has no bias epilogue)
  + relu          C[i,j] = max(C[i,j], 0)              (README.md:67-76), fused with partial=2, or
                                                       MMAFragmentOp.ReLU as tensorize epilogue
  alpha / beta    tensorize prologue SET 0 / SCALE b, epilogue SCALE a
                                                       (docs/Tutorials/GPU/Tensor_MatMul_ElementWiseOps_GPU.md:88-99)
  reduce_mean     init / accumulate / divide nests fused (kernels/reduce_mean/naive_runtime_sized.py:66-148)
  gather          Output[i,j,k] = Data[Indices[i,j], k] | Data[i, Indices[j,k]]
                                                       (kernels/gather/naive_runtime_sized.py:26-49)
  dimension fn    Nest((1,)) whose logic only does OutDim.set(InDim)   (dsl_tests.py:1588-1594)
  range size      Nest((1,)): OutDim.set(cast(floor((limit - start) / delta), int64))   (dsl_tests.py:1450-1454)
  range           Nest([n]):  output[i] = s; s.set(s + delta)          (dsl_tests.py:1456-1462; s is an in/out Scalar)
"""
from __future__ import annotations

import dataclasses
from typing import Any, List, Optional, Tuple

from . import lang
from .lang import (Access, Array, BinOp, Call, Const, DimExpr, Dimension, Index, MMAFragmentOp, Nest, Plan, Scalar, ScalarRef,
                   Schedule)


class UnsupportedNestError(NotImplementedError):
    """The nest is not one of the operator families this package implements on the GPU."""


@dataclasses.dataclass
class GemmSpec:
    a: Array
    b: Array
    c: Array
    bias: Optional[Array]
    m: Any
    n: Any
    k: Any                     # ints or Dimensions
    a_transposed: bool         # array is indexed [k, i] instead of [i, k]
    b_transposed: bool         # array is indexed [j, k] instead of [k, j]
    relu: bool = False
    alpha: float = 1.0
    beta: float = 1.0
    compute: str = "auto"      # "auto" | "simt" | "tensor"
    kind: str = "gemm"
    # batch matmul only: number of problems, and per array the positions of its (batch, row, column)
    # indices among the array's dimensions (batch position None = the operand is shared by all problems)
    batch: Any = None
    a_pos: Optional[Tuple[Optional[int], int, int]] = None
    b_pos: Optional[Tuple[Optional[int], int, int]] = None
    c_pos: Optional[Tuple[Optional[int], int, int]] = None


@dataclasses.dataclass
class ReduceMeanSpec:
    data: Array
    reduced: Array
    axes: Tuple[int, ...]      # in terms of data's own rank
    keepdims: int
    kind: str = "reduce_mean"


@dataclasses.dataclass
class GatherSpec:
    data: Array
    indices: Array
    output: Array
    axis: int
    kind: str = "gather"


@dataclasses.dataclass
class RangeSizeSpec:
    start: Scalar
    limit: Scalar
    delta: Scalar
    size: Dimension
    kind: str = "range_size"


@dataclasses.dataclass
class RangeSpec:
    output: Array
    running: Scalar            # read as the first value, left as the value after the last addition
    delta: Scalar
    n: Any                     # int or Dimension
    kind: str = "range"


@dataclasses.dataclass
class DimsSpec:
    assignments: List[Tuple[Dimension, Any]]     # (output dimension, Dimension or int)
    kind: str = "dims"


def _strip_cast(e):
    while isinstance(e, Call) and e.fn == "cast":
        e = e.args[0]
    return e


def _is_zero(e) -> bool:
    e = _strip_cast(e)
    return isinstance(e, Const) and float(e.value) == 0.0


def _same_access(a, b) -> bool:
    return (isinstance(a, Access) and isinstance(b, Access) and a.array is b.array and len(a.indices) == len(b.indices)
            and all(x is y for x, y in zip(a.indices, b.indices)))


def _match_matmul(nest: Nest) -> Optional[GemmSpec]:
    if len(nest.shape) != 3 or len(nest.statements) != 1:
        return None
    s = nest.statements[0]
    if s.kind != "assign" or s.op != "+":
        return None
    tgt = s.target
    val = _strip_cast(s.value)
    if not (isinstance(val, BinOp) and val.op == "*") or len(tgt.indices) != 2:
        return None
    x, y = _strip_cast(val.lhs), _strip_cast(val.rhs)
    if not (isinstance(x, Access) and isinstance(y, Access)) or len(x.indices) != 2 or len(y.indices) != 2:
        return None
    i, j = tgt.indices
    idx = list(nest._indices)
    if not (isinstance(i, Index) and isinstance(j, Index)) or i is j or i not in idx or j not in idx:
        return None
    k = [q for q in idx if q is not i and q is not j][0]

    def role(acc):
        s_ = set(map(id, acc.indices))
        if s_ == {id(i), id(k)}:
            return "a"
        if s_ == {id(k), id(j)}:
            return "b"
        return None
    rx, ry = role(x), role(y)
    if {rx, ry} != {"a", "b"}:
        return None
    a_acc, b_acc = (x, y) if rx == "a" else (y, x)
    return GemmSpec(a=a_acc.array, b=b_acc.array, c=tgt.array, bias=None,
                    m=i.extent, n=j.extent, k=k.extent,
                    a_transposed=a_acc.indices[0] is k, b_transposed=b_acc.indices[0] is j)


def _match_batch_matmul(nest: Nest) -> Optional[GemmSpec]:
    if len(nest.shape) != 4 or len(nest.statements) != 1:
        return None
    s = nest.statements[0]
    if s.kind != "assign" or s.op != "+":
        return None
    tgt = s.target
    val = _strip_cast(s.value)
    if not (isinstance(val, BinOp) and val.op == "*") or len(tgt.indices) != 3:
        return None
    x, y = _strip_cast(val.lhs), _strip_cast(val.rhs)
    if not (isinstance(x, Access) and isinstance(y, Access)):
        return None
    idx = list(nest._indices)
    if not all(isinstance(q, Index) and any(q is w for w in idx) for q in tgt.indices) or len(set(map(id, tgt.indices))) != 3:
        return None
    k = [q for q in idx if not any(q is w for w in tgt.indices)][0]

    def positions(acc, batch_ix, row_ix, col_ix):
        """Positions of the three indices in the access, or None if it uses anything else / misses row or column."""
        pos = {}
        for d, q in enumerate(acc.indices):
            for name, want in (("b", batch_ix), ("r", row_ix), ("c", col_ix)):
                if q is want:
                    if name in pos:
                        return None
                    pos[name] = d
                    break
            else:
                return None
        if "r" not in pos or "c" not in pos:
            return None
        return (pos.get("b"), pos["r"], pos["c"])

    # C's indices are (b, i, j) in some order; which of them is the batch index follows from the operands:
    # b appears in C and in at least one operand together with k, i only with A's k, j only with B's k
    for b in tgt.indices:
        i_j = [q for q in tgt.indices if q is not b]
        for i, j in (i_j, i_j[::-1]):
            for a_acc, b_acc in ((x, y), (y, x)):
                pa, pb = positions(a_acc, b, i, k), positions(b_acc, b, k, j)
                pc = positions(tgt, b, i, j)
                if pa is None or pb is None or pc is None:
                    continue
                if pa[0] is None and pb[0] is None:
                    continue          # no operand carries the batch index: not a batch matmul
                return GemmSpec(a=a_acc.array, b=b_acc.array, c=tgt.array, bias=None, m=i.extent, n=j.extent,
                                k=k.extent, a_transposed=False, b_transposed=False, batch=b.extent,
                                a_pos=pa, b_pos=pb, c_pos=pc)
    return None


def _match_relu(nest: Nest, c: Array) -> bool:
    if len(nest.shape) != 2 or len(nest.statements) != 1:
        return False
    s = nest.statements[0]
    if s.kind != "assign" or s.op != "=" or s.target.array is not c:
        return False
    if tuple(s.target.indices) != tuple(nest._indices):
        return False
    v = _strip_cast(s.value)
    if not (isinstance(v, Call) and v.fn == "max" and len(v.args) == 2):
        return False
    p, q = v.args
    return (_same_access(_strip_cast(p), s.target) and _is_zero(q)) or (_same_access(_strip_cast(q), s.target) and _is_zero(p))


def _match_bias(nest: Nest, c: Array) -> Optional[Array]:
    if len(nest.shape) != 2 or len(nest.statements) != 1:
        return None
    s = nest.statements[0]
    if s.kind != "assign" or s.op != "+" or s.target.array is not c or tuple(s.target.indices) != tuple(nest._indices):
        return None
    v = _strip_cast(s.value)
    if isinstance(v, Access) and len(v.indices) == 1 and v.indices[0] is nest._indices[1]:
        return v.array
    return None


def _match_gemm(nests: List[Nest], partial: Optional[int], plan: Optional[Plan]) -> Optional[GemmSpec]:
    spec = _match_matmul(nests[0])
    if spec is None:
        spec = _match_batch_matmul(nests[0])
        if spec is not None and len(nests) > 1:
            raise UnsupportedNestError("a batch matmul takes its ReLU / scaling from tensorize(prologue_op=, epilogue_op=), "
                                       "not from fused nests")
    if spec is None:
        return None
    rest = nests[1:]
    if rest and partial != 2:
        raise UnsupportedNestError("matmul can only be fused with element-wise nests over (i, j): use partial=2")
    for n in rest:
        if tuple(n.shape) != (spec.m, spec.n):
            raise UnsupportedNestError("fused element-wise nest must cover C's (M, N) iteration space")
        if spec.relu:
            raise UnsupportedNestError("nothing may follow the ReLU nest in a fused matmul")
        bias = _match_bias(n, spec.c)
        if bias is not None and spec.bias is None:
            spec.bias = bias
        elif _match_relu(n, spec.c):
            spec.relu = True
        else:
            raise UnsupportedNestError(f"cannot fuse this nest into the GEMM epilogue: {n.statements}")
    if plan is not None and plan.tensorized:
        spec.compute = "tensor"
        if plan.prologue_op is MMAFragmentOp.SET:
            if plan.prologue_arg != 0.0:
                raise UnsupportedNestError("prologue SET is supported with 0 only (beta = 0)")
            spec.beta = 0.0
        elif plan.prologue_op is MMAFragmentOp.SCALE:
            spec.beta = plan.prologue_arg
        elif plan.prologue_op is not MMAFragmentOp.NONE:
            raise UnsupportedNestError(f"unsupported prologue op {plan.prologue_op}")
        if plan.epilogue_op is MMAFragmentOp.SCALE:
            # the epilogue scales the whole accumulator, i.e. both A@B and the beta*C it started from
            spec.alpha = plan.epilogue_arg
            spec.beta = spec.beta * plan.epilogue_arg
        elif plan.epilogue_op in (MMAFragmentOp.ReLU, MMAFragmentOp.ReLU_NoConditional):
            spec.relu = True
        elif plan.epilogue_op is MMAFragmentOp.SET:
            raise UnsupportedNestError("epilogue SET discards the product; not supported")
    elif spec.a.element_type is lang.ScalarType.float32:
        spec.compute = "simt"      # plain fp32 nests keep true fp32 arithmetic
    return spec


def _match_gather(nest: Nest) -> Optional[GatherSpec]:
    if len(nest.shape) != 3 or len(nest.statements) != 1:
        return None
    s = nest.statements[0]
    if s.kind != "assign" or s.op != "=" or tuple(s.target.indices) != tuple(nest._indices):
        return None
    v = s.value
    if not isinstance(v, Access) or len(v.indices) != 2:
        return None
    i, j, k = nest._indices
    p, q = v.indices
    if isinstance(p, Access) and q is k and tuple(p.indices) == (i, j):
        return GatherSpec(data=v.array, indices=p.array, output=s.target.array, axis=0)
    if p is i and isinstance(q, Access) and tuple(q.indices) == (j, k):
        return GatherSpec(data=v.array, indices=q.array, output=s.target.array, axis=1)
    return None


def _match_reduce_mean(nests: List[Nest], partial: Optional[int]) -> Optional[ReduceMeanSpec]:
    if len(nests) != 3:
        return None
    init, acc, div = nests
    if not (len(init.statements) == 1 and len(acc.statements) == 1 and len(div.statements) == 1):
        return None
    s0, s1, s2 = init.statements[0], acc.statements[0], div.statements[0]
    if not (s0.kind == "assign" and s0.op == "=" and _is_zero(s0.value)):
        return None
    if not (s1.kind == "assign" and s1.op == "+" and isinstance(_strip_cast(s1.value), Access)):
        return None
    if not (s2.kind == "assign" and s2.op == "/"):
        return None
    reduced = s1.target.array
    if s0.target.array is not reduced or s2.target.array is not reduced:
        return None
    src = _strip_cast(s1.value)
    data = src.array
    rank = len(data.shape)
    if len(src.indices) != rank:
        return None
    out_idx = list(s1.target.indices)
    axes = []
    kept_positions = []
    for d, ix in enumerate(src.indices):
        if any(ix is o for o in out_idx):
            kept_positions.append(d)
        else:
            axes.append(d)
    keepdims = 1 if len(out_idx) == rank and axes else 0
    if not axes:
        return None
    count = 1
    static = True
    for d in axes:
        if isinstance(data.shape[d], int):
            count *= data.shape[d]
        else:
            static = False
    dv = _strip_cast(s2.value)
    if static and isinstance(dv, Const) and float(dv.value) != float(count):
        raise UnsupportedNestError(f"reduce_mean: divisor {dv.value} is not the number of reduced elements {count}")
    return ReduceMeanSpec(data=data, reduced=reduced, axes=tuple(axes), keepdims=keepdims)


def _scalar_of(e) -> Optional[Scalar]:
    e = _strip_cast(e)
    return e.scalar if isinstance(e, ScalarRef) else None


def _match_range_size(nest: Nest) -> Optional[RangeSizeSpec]:
    if len(nest.statements) != 1 or nest.statements[0].kind != "set_dim":
        return None
    s = nest.statements[0]
    v = _strip_cast(s.value)
    if not (isinstance(v, Call) and v.fn == "floor"):
        return None
    q = _strip_cast(v.args[0])
    if not (isinstance(q, BinOp) and q.op == "/"):
        return None
    span, delta = _strip_cast(q.lhs), _scalar_of(q.rhs)
    if not (isinstance(span, BinOp) and span.op == "-") or delta is None:
        return None
    limit, start = _scalar_of(span.lhs), _scalar_of(span.rhs)
    if limit is None or start is None:
        return None
    return RangeSizeSpec(start=start, limit=limit, delta=delta, size=s.target)


def _match_range(nest: Nest) -> Optional[RangeSpec]:
    if len(nest.shape) != 1 or len(nest.statements) != 2:
        return None
    s0, s1 = nest.statements
    if not (s0.kind == "assign" and s0.op == "=" and s1.kind == "set_scalar"):
        return None
    if tuple(s0.target.indices) != tuple(nest._indices):
        return None
    running = _scalar_of(s0.value)
    if running is None or s1.target is not running:
        return None
    v = _strip_cast(s1.value)
    if not (isinstance(v, BinOp) and v.op == "+"):
        return None
    a, b = _scalar_of(v.lhs), _scalar_of(v.rhs)
    delta = b if a is running else a if b is running else None
    if delta is None or delta is running:
        return None
    return RangeSpec(output=s0.target.array, running=running, delta=delta, n=nest.shape[0])


def _match_dims(nest: Nest) -> Optional[DimsSpec]:
    if not nest.statements or any(s.kind != "set_dim" for s in nest.statements):
        return None
    out = []
    for s in nest.statements:
        v = s.value
        if isinstance(v, DimExpr):
            out.append((s.target, v.dim))
        elif isinstance(v, Const):
            out.append((s.target, int(v.value)))
        else:
            raise UnsupportedNestError("dimension functions may only copy dimensions or constants")
    return DimsSpec(out)


def recognise(source) -> Any:
    """source: Nest | Schedule | Plan -> GemmSpec | ReduceMeanSpec | GatherSpec | DimsSpec."""
    plan = source if isinstance(source, Plan) else None
    sched = plan.schedule if plan is not None else source
    if isinstance(sched, Nest):
        sched = sched.create_schedule()
    if not isinstance(sched, Schedule):
        raise TypeError("package.add takes a Nest, Schedule or Plan")
    nests = sched.nests
    if len(nests) == 1:
        rs = _match_range_size(nests[0]) or _match_range(nests[0])
        if rs is not None:
            return rs
        d = _match_dims(nests[0])
        if d is not None:
            return d
        g = _match_gather(nests[0])
        if g is not None:
            return g
    spec = _match_gemm(nests, sched.partial, plan)
    if spec is not None:
        return spec
    r = _match_reduce_mean(nests, sched.partial)
    if r is not None:
        return r
    logic = "; ".join(repr(s) for n in nests for s in n.statements)
    raise UnsupportedNestError(
        "this package implements matmul(+bias)(+ReLU), reduce_mean, gather and range on B200 kernels and does not compile "
        f"arbitrary loop nests; unrecognised logic: {logic}")
