"""The thin slice of the Accera Python DSL needed to *describe* matmul(+bias)(+ReLU),
reduce_mean and gather functions, so that existing scripts keep working:

    A = Array(role=Role.INPUT, shape=(M, K)); ...
    nest = Nest(shape=(M, N, K)); i, j, k = nest.get_indices()
    @nest.iteration_logic
    def _(): C[i, j] += A[i, k] * B[k, j]
    package.add(fuse(nest.create_schedule(), relu.create_schedule(), partial=2), args=(A, B, C), base_name=...)

Reference surface mirrored here: accera/python/accera/lang/Array.py:46-138 (Array),
lang/Nest.py:21-117 (Nest and logic capture), lang/Schedule.py:522-628 (fuse),
lang/Plan.py:208-379, 381-657, 793-825 (tensorize / cache / bind knobs),
lang/Layout.py:35-55 (strides), lang/DimensionUtilities.py:12-23 (create_dimensions),
Targets.py:833-879 (targets).

This is not a loop-nest compiler.  The iteration logic is *traced* once with
symbolic indices into a list of statements; `accera_b200.patterns` recognises
the three operator families in that trace and maps them onto the hand-written
sm_100a kernels.  Scheduling transformations (tile, split, reorder, unroll,
vectorize, cache, bind, parallelize) are accepted and recorded - they do not
change the mathematical function, and the kernels bring their own tiling - while
`Plan.tensorize` selects the tensor-core path and carries the fragment
prologue / epilogue ops (SET / SCALE / ReLU) that change the result.
"""
from __future__ import annotations

import enum
import inspect
import re
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple, Union


# ---------------------------------------------------------------------------
# enumerations
# ---------------------------------------------------------------------------

class ScalarType(enum.Enum):
    bool = "bool"
    int8 = "int8"
    int16 = "int16"
    int32 = "int32"
    int64 = "int64"
    uint8 = "uint8"
    uint16 = "uint16"
    uint32 = "uint32"
    uint64 = "uint64"
    float16 = "float16"
    bfloat16 = "bfloat16"
    float32 = "float32"
    float64 = "float64"
    index = "index"          # lowered to int64_t (TranslateToHeader.cpp:328-352)


# C spelling in the header (TranslateToHeader.cpp:308-352) and bytes per element
C_TYPE = {
    ScalarType.bool: "bool", ScalarType.int8: "int8_t", ScalarType.int16: "int16_t", ScalarType.int32: "int32_t",
    ScalarType.int64: "int64_t", ScalarType.uint8: "uint8_t", ScalarType.uint16: "uint16_t",
    ScalarType.uint32: "uint32_t", ScalarType.uint64: "uint64_t", ScalarType.float16: "float16_t",
    ScalarType.bfloat16: "bfloat16_t", ScalarType.float32: "float", ScalarType.float64: "double",
    ScalarType.index: "int64_t",
}
TYPE_BYTES = {
    ScalarType.bool: 1, ScalarType.int8: 1, ScalarType.int16: 2, ScalarType.int32: 4, ScalarType.int64: 8,
    ScalarType.uint8: 1, ScalarType.uint16: 2, ScalarType.uint32: 4, ScalarType.uint64: 8, ScalarType.float16: 2,
    ScalarType.bfloat16: 2, ScalarType.float32: 4, ScalarType.float64: 8, ScalarType.index: 8,
}


class Role(enum.Enum):
    INPUT = "input"
    INPUT_OUTPUT = "input_output"
    OUTPUT = "output"
    CONST = "const"
    TEMP = "temp"


class Layout(enum.Enum):
    FIRST_MAJOR = "first_major"     # row-major
    LAST_MAJOR = "last_major"       # column-major
    DEFERRED = "deferred"


class MMAFragmentOp(enum.Enum):
    """Accumulator-fragment ops (accera/ir/include/value/ValueMMAOp.h:64-71)."""
    NONE = 0
    ReLU = 1
    ReLU_NoConditional = 2
    SET = 3
    SCALE = 4


class MMAShape(enum.Enum):
    # accepted for source compatibility; the tcgen05 kernel picks its own instruction shape
    M64xN64xK1_B4 = 0
    M64xN64xK1_B2 = 1
    M32xN32xK2_B1 = 2
    M16xN16xK4_B1 = 3
    M64xN64xK4_B4 = 4
    M64xN64xK4_B2 = 5
    M32xN32xK8_B1 = 6
    M16xN16xK16_B1 = 7
    M32xN8xK16_B1 = 8
    M8xN32xK16_B1 = 9
    M16xN16xK8_B1 = 10


class _TensorCoreInfo:
    """Shape arithmetic the reference's GPU tests use to size their tiles before tensorizing
    (Targets.py:770-793).  The shapes are read off the MMAShape member's name."""

    @staticmethod
    def mma_shape_to_tuple(mma_shape: MMAShape) -> Tuple[int, int, int]:
        m, n, k = mma_shape.name.split("_")[0].split("x")
        return int(m[1:]), int(n[1:]), int(k[1:])

    def compute_tensor_splits(self, mma_shape: MMAShape, num_total_passes: int = 1) -> Tuple[int, int, int]:
        m, n, k = self.mma_shape_to_tuple(mma_shape)
        return m, n, k * int(num_total_passes)


class MMASchedulingPolicy(enum.Enum):
    PASS_ORDER = 0
    BLOCK_ORDER = 1


class CacheStrategy(enum.Enum):
    BLOCKED = 0
    STRIPED = 1


class _MemorySpace(enum.Enum):
    NONE = 0
    GLOBAL = 1
    SHARED = 2
    PRIVATE = 3
    MMA_FRAGMENT = 4


class _Auto:
    def __repr__(self):
        return "AUTO"


AUTO = _Auto()
inf = float("inf")


# ---------------------------------------------------------------------------
# targets
# ---------------------------------------------------------------------------

class Target:
    """HOST (the reference's default) or a GPU model.  Every function built by this package runs
    on the B200 kernels whatever target is named; the target is recorded in the .hat and takes
    part in the function-name hash, as in the reference (Package.py:310-335)."""

    class Category(enum.Enum):
        CPU = "CPU"
        GPU = "GPU"

    class Model(enum.Enum):
        HOST = "HOST"
        NVIDIA_B200 = "NVidia B200"
        NVIDIA_A100 = "NVidia A100"
        NVIDIA_V100 = "NVidia V100"
        NVIDIA_RTX_A6000 = "NVidia RTX A6000"
        AMD_MI100 = "AMD MI100"

    class Architecture(enum.Enum):
        HOST = "HOST"
        X86_64 = "x86_64"

    class GridUnit(enum.Enum):
        BLOCK_X = "block_x"
        BLOCK_Y = "block_y"
        BLOCK_Z = "block_z"
        THREAD_X = "thread_x"
        THREAD_Y = "thread_y"
        THREAD_Z = "thread_z"
        WARP_X = "warp_x"
        WARP_Y = "warp_y"

    GridUnits = GridUnit
    MemorySpace = _MemorySpace

    def __init__(self, known_name: Union[str, "Target.Model"] = Model.HOST, category: "Target.Category" = None, **kwargs):
        if isinstance(known_name, str):
            matches = [m for m in Target.Model if m.value == known_name or m.name == known_name]
            if not matches:
                raise ValueError(f"unknown target {known_name!r}")
            known_name = matches[0]
        self.model = known_name
        self.name = known_name.value
        self.category = category or (Target.Category.CPU if known_name is Target.Model.HOST else Target.Category.GPU)
        self.runtime = "CUDA" if self.category is Target.Category.GPU else "NONE"
        self.extra = dict(kwargs)
        self.tensor_core_info = _TensorCoreInfo()
        # launch limits the reference checks a bound plan against (Targets.py: "Max Block Size", "Max Threads Per
        # Block", "Warp Size"; lang/Plan.py:989-1011).  The CUDA values hold for every NVIDIA model listed here.
        gpu = self.category is Target.Category.GPU
        amd = known_name is Target.Model.AMD_MI100
        self.warp_size = kwargs.get("warp_size", (64 if amd else 32) if gpu else 0)
        self.max_threads_per_block = kwargs.get("max_threads_per_block", 1024 if gpu else 0)
        self.max_block_size = list(kwargs.get("max_block_size", [1024, 1024, 64] if gpu else []))
        self.num_sms = kwargs.get("num_sms", 148 if known_name is Target.Model.NVIDIA_B200 else 0)

    def is_compatible_with(self, other: "Target") -> bool:
        return self.category == other.category and self.runtime == other.runtime

    def __str__(self):
        return f"Target({self.name})"

    __repr__ = __str__


Target.HOST = Target(Target.Model.HOST)


# ---------------------------------------------------------------------------
# symbolic expressions
# ---------------------------------------------------------------------------

class Expr:
    def _bin(self, op, other, swap=False):
        other = as_expr(other)
        return BinOp(op, other, self) if swap else BinOp(op, self, other)

    def __add__(self, o): return self._bin("+", o)
    def __radd__(self, o): return self._bin("+", o, True)
    def __sub__(self, o): return self._bin("-", o)
    def __rsub__(self, o): return self._bin("-", o, True)
    def __mul__(self, o): return self._bin("*", o)
    def __rmul__(self, o): return self._bin("*", o, True)
    def __truediv__(self, o): return self._bin("/", o)
    def __rtruediv__(self, o): return self._bin("/", o, True)


class Const(Expr):
    def __init__(self, value, dtype: Optional[ScalarType] = None):
        self.value = value
        self.dtype = dtype

    def __repr__(self):
        return f"{self.value!r}"


class Index(Expr):
    """A loop index of a nest (or, after fuse/tile, of a schedule)."""
    _count = 0

    def __init__(self, extent, nest=None, position: int = -1, name: Optional[str] = None):
        Index._count += 1
        self.id = Index._count
        self.extent = extent
        self.nest = nest
        self.position = position
        self.name = name or f"i{self.id}"

    def __repr__(self):
        return self.name

    def __hash__(self):
        return hash(self.id)

    def __eq__(self, other):
        return self is other


class BinOp(Expr):
    def __init__(self, op: str, lhs: Expr, rhs: Expr):
        self.op, self.lhs, self.rhs = op, lhs, rhs

    def __repr__(self):
        return f"({self.lhs!r} {self.op} {self.rhs!r})"


class Call(Expr):
    """max / min / cast / abs ... applied to expressions."""
    def __init__(self, fn: str, args: Sequence[Expr], dtype: Optional[ScalarType] = None):
        self.fn, self.args, self.dtype = fn, list(args), dtype

    def __repr__(self):
        return f"{self.fn}({', '.join(map(repr, self.args))})"


class Access(Expr):
    """array[indices] used as a value; also the target of an assignment."""
    def __init__(self, array: "Array", indices: Tuple[Any, ...]):
        self.array, self.indices = array, tuple(indices)

    def __repr__(self):
        return f"{self.array.name or 'arr'}[{', '.join(map(repr, self.indices))}]"

    # `C[i, j] += expr` evaluates C.__getitem__, then __iadd__, then C.__setitem__ with the result
    def __iadd__(self, o): return _Augmented("+", self, as_expr(o))
    def __isub__(self, o): return _Augmented("-", self, as_expr(o))
    def __imul__(self, o): return _Augmented("*", self, as_expr(o))
    def __itruediv__(self, o): return _Augmented("/", self, as_expr(o))


class _Augmented:
    def __init__(self, op, target: Access, value: Expr):
        self.op, self.target, self.value = op, target, value


class DimExpr(Expr):
    """A runtime Dimension used as a value (sizes of runtime arrays, right-hand side of Dimension.set)."""
    def __init__(self, dim: "Dimension"):
        self.dim = dim

    def __repr__(self):
        return self.dim.name or "dim"


def as_expr(v) -> Expr:
    if isinstance(v, Expr):
        return v
    if isinstance(v, Dimension):
        return DimExpr(v)
    if isinstance(v, Scalar):
        return ScalarRef(v)
    if isinstance(v, (int, float, bool)):
        return Const(v)
    raise TypeError(f"cannot use {type(v).__name__} in iteration logic")


class Statement:
    """target (op)= value, where op is '=' or one of + - * /.  `set_dim` statements assign a Dimension."""
    def __init__(self, kind: str, target, value: Expr, op: str = "="):
        self.kind, self.target, self.value, self.op = kind, target, value, op

    def __repr__(self):
        return f"{self.target!r} {self.op if self.op == '=' else self.op + '='} {self.value!r}"


_trace_stack: List[List[Statement]] = []


def _record(stmt: Statement) -> None:
    if not _trace_stack:
        raise RuntimeError("arrays can only be written inside a nest's iteration logic")
    _trace_stack[-1].append(stmt)


# scalar functions usable inside iteration logic (accera/python/accera/__init__.py:19-22)
def max(a, b): return Call("max", [as_expr(a), as_expr(b)])          # noqa: A001
def min(a, b): return Call("min", [as_expr(a), as_expr(b)])          # noqa: A001
def abs(a): return Call("abs", [as_expr(a)])                         # noqa: A001
def cast(value, dtype: ScalarType): return Call("cast", [as_expr(value)], dtype)
def floor(a): return Call("floor", [as_expr(a)])
def ceil(a): return Call("ceil", [as_expr(a)])
_cast = cast


# ---------------------------------------------------------------------------
# dimensions and arrays
# ---------------------------------------------------------------------------

class Dimension:
    """A runtime dimension: an int64 function argument (lang/Array.py:249-258)."""
    def __init__(self, role: Role = Role.INPUT, value=None, name: str = ""):
        self.role = role
        self.value = value
        self.name = name
        self.type = ScalarType.index

    def set(self, value) -> None:
        _record(Statement("set_dim", self, as_expr(value)))

    def __repr__(self):
        return f"Dimension({self.name or '?'}, {self.role.name})"

    def __mul__(self, other):
        return DimExpr(self) * as_expr(other)

    __rmul__ = __mul__


class ScalarRef(Expr):
    """A Scalar used as a value inside iteration logic."""
    def __init__(self, scalar: "Scalar"):
        self.scalar = scalar

    def __repr__(self):
        return self.scalar.name or "scalar"


class Scalar:
    """A scalar function argument (the reference's `accera._lang_python._lang.Scalar`, as the range-node tests use
    it: dsl_tests.py:1438-1448): an INPUT scalar is passed by value, an INPUT_OUTPUT / OUTPUT one by pointer, a TEMP
    one lives inside the package.  Arithmetic on it builds expressions; `.set(value)` assigns it."""
    def __init__(self, type: ScalarType = ScalarType.float32, role: Role = Role.INPUT, name: str = "", value=None):
        if isinstance(type, Role):          # Scalar(role) is not a form the reference has; keep the error early
            raise TypeError("Scalar(type, role): the first argument is the element type")
        self.type = type
        self.element_type = type
        self.role = role
        self.name = name
        self.value = value

    def set(self, value) -> None:
        _record(Statement("set_scalar", self, as_expr(value)))

    def _bin(self, op, other, swap=False):
        return ScalarRef(self)._bin(op, other, swap)

    def __add__(self, o): return self._bin("+", o)
    def __radd__(self, o): return self._bin("+", o, True)
    def __sub__(self, o): return self._bin("-", o)
    def __rsub__(self, o): return self._bin("-", o, True)
    def __mul__(self, o): return self._bin("*", o)
    def __rmul__(self, o): return self._bin("*", o, True)
    def __truediv__(self, o): return self._bin("/", o)
    def __rtruediv__(self, o): return self._bin("/", o, True)

    def __repr__(self):
        return f"Scalar({self.name or '?'}, {self.type.name}, {self.role.name})"


def create_dimensions(role: Role = Role.INPUT) -> Tuple[Dimension, ...]:
    """`a, b, c = create_dimensions()` - as many dimensions as assignment targets, named after them
    (the reference reads the caller's source line the same way, lang/DimensionUtilities.py:12-23)."""
    frame = inspect.stack()[1]
    names: List[str] = []
    try:
        src = "".join(frame.code_context or [])
        m = re.match(r"\s*([\w\s,()]+?)\s*=\s*(?:\w+\.)*create_dimensions", src)
        if m:
            names = [n.strip() for n in m.group(1).strip("() ").split(",") if n.strip()]
    finally:
        del frame
    if not names:
        raise RuntimeError("create_dimensions() must be used as `a, b = create_dimensions()`")
    dims = tuple(Dimension(role=role, name=n) for n in names)
    return dims if len(dims) > 1 else dims[0]


class Array:
    """A multi-dimensional array argument (lang/Array.py:46-138)."""
    Layout = Layout

    def __init__(self, role: Role, name: str = "", data=None, element_type: Union[ScalarType, type, None] = None,
                 layout: Union[Layout, Tuple[int, ...]] = Layout.FIRST_MAJOR, offset: int = 0,
                 shape: Optional[Sequence[Union[int, Dimension]]] = None, flags=None):
        if role is Role.CONST:
            if data is None:
                raise ValueError("data is required for Role.CONST")
            shape = tuple(data.shape)
        elif shape is None:
            raise ValueError("shape is required")
        if element_type is None:
            element_type = ScalarType.float32
        elif element_type is int:
            element_type = ScalarType.int64
        elif element_type is float:
            element_type = ScalarType.float32
        elif not isinstance(element_type, ScalarType):
            raise ValueError("Unknown element type on Array instance")
        self.role = role
        self.name = name
        self.data = data
        self.element_type = element_type
        self.layout = layout
        self.offset = offset
        self._shape = tuple(shape)

    @property
    def shape(self) -> list:
        """A fresh list, as in the reference (lang/Array.py:152-154): callers concatenate and edit it."""
        return list(self._shape)

    @property
    def is_dynamic(self) -> bool:
        return any(isinstance(s, Dimension) for s in self.shape)

    def strides(self) -> Tuple[int, ...]:
        """Element strides of a statically shaped array (lang/Layout.py:35-55)."""
        if self.is_dynamic:
            raise ValueError("strides of a runtime-sized array are dense first-major from its dimension arguments")
        if isinstance(self.layout, tuple):
            return tuple(self.layout)
        n = len(self.shape)
        st = [1] * n
        if self.layout is Layout.LAST_MAJOR:
            for d in range(1, n):
                st[d] = st[d - 1] * self.shape[d - 1]
        else:
            for d in range(n - 2, -1, -1):
                st[d] = st[d + 1] * self.shape[d + 1]
        return tuple(st)

    @staticmethod
    def _norm(idx) -> Tuple[Any, ...]:
        if isinstance(idx, (list, tuple)):
            return tuple(idx)
        return (idx,)

    def __getitem__(self, idx) -> Access:
        return Access(self, self._norm(idx))

    def __setitem__(self, idx, value) -> None:
        target = Access(self, self._norm(idx))
        if isinstance(value, _Augmented):
            _record(Statement("assign", target, value.value, value.op))
        else:
            _record(Statement("assign", target, as_expr(value), "="))

    def __repr__(self):
        return f"Array({self.name or '?'}, {self.role.name}, {self.element_type.name}, {self.shape})"


# ---------------------------------------------------------------------------
# nests, schedules, plans
# ---------------------------------------------------------------------------

class Nest:
    """An iteration space plus its logic (lang/Nest.py:21-117)."""
    def __init__(self, shape: Sequence[Union[int, Dimension]]):
        self.shape = tuple(shape)
        self._indices = [Index(extent, self, pos) for pos, extent in enumerate(self.shape)]
        self.statements: List[Statement] = []
        self._logic_fns: List[Callable] = []

    def get_indices(self) -> List[Index]:
        """Always a list, also for a rank-1 nest (lang/Nest.py:62-86)."""
        return list(self._indices)

    def iteration_logic(self, fn: Callable) -> Callable:
        _trace_stack.append([])
        try:
            fn()
        finally:
            stmts = _trace_stack.pop()
        self.statements.extend(stmts)
        self._logic_fns.append(fn)
        return fn

    def create_schedule(self) -> "Schedule":
        return Schedule([self])

    def create_plan(self, target: Optional[Target] = None) -> "Plan":
        return self.create_schedule().create_plan(target)


class Schedule:
    """An ordering of one nest, or of several fused nests (lang/Schedule.py:522-628).

    `nests` are executed, for every point of the first `partial` (fused) dimensions, one after
    the other, each running all of its remaining dimensions - the "fusing index precedes the
    unfused ones" rule of docs/Reference/safety_analysis.md:28-34.
    """
    def __init__(self, nests: List[Nest], partial: Optional[int] = None, orders: Optional[List[List[Index]]] = None):
        self.nests = list(nests)
        self.partial = partial
        self.transformations: List[Tuple[str, Any]] = []
        # per nest: its own indices in the loop order they had when the schedule was built / fused
        self.orders: List[List[Index]] = [list(o) for o in orders] if orders else [list(n._indices) for n in nests]
        if len(nests) == 1:
            self._indices = list(self.orders[0])
        else:
            fused = [Index(self.orders[0][d].extent, None, d, f"f{d}") for d in range(partial)]
            fusing = Index(len(nests), None, partial, "f")
            rest: List[Index] = []
            for o in self.orders:
                rest.extend(o[partial:])
            self._indices = fused + [fusing] + rest

    def get_indices(self) -> List[Index]:
        return list(self._indices)

    def get_fusing_index(self) -> Index:
        return self._indices[self.partial] if self.partial is not None else None

    # scheduling transformations: recorded, semantically neutral
    def _new_index(self, parent: Index, size) -> Index:
        idx = Index(size, None, -1, parent.name + parent.name[-1])
        self._indices.insert(self._indices.index(parent) + 1, idx)
        # the parent now advances `size` at a time; the new index walks one block of it
        steps = self.__dict__.setdefault("_steps", {})
        steps[id(parent)] = steps.get(id(parent), 1) * int(size)
        self.__dict__.setdefault("_split_factor", {})[id(idx)] = int(size)
        return idx

    def iteration_count(self, index: Index) -> int:
        """Iterations of `index` in this schedule: its split factor if it came from a split and was not split
        again, else ceil(extent / step) (lang/Plan.py:888-893)."""
        steps = self.__dict__.get("_steps", {})
        step = steps.get(id(index), 1)
        factor = self.__dict__.get("_split_factor", {}).get(id(index))
        if step == 1 and factor is not None:
            return factor
        extent = index.extent
        if not isinstance(extent, int):
            raise ValueError("launch geometry needs static extents")
        return -(-extent // step)

    def split(self, index: Index, size) -> Index:
        self.transformations.append(("split", (index, size)))
        return self._new_index(index, size)

    def tile(self, shape: Dict[Index, int]):
        self.transformations.append(("tile", dict(shape)))
        new = tuple(self._new_index(i, s) for i, s in shape.items())
        return new if len(new) > 1 else new[0]

    def reorder(self, *order) -> None:
        if len(order) == 1 and isinstance(order[0], (list, tuple)):
            order = tuple(order[0])
        if set(map(id, order)) != set(map(id, self._indices)):
            raise ValueError("reorder must name every index of the schedule exactly once")
        self.transformations.append(("reorder", order))
        self._indices = list(order)
        if len(self.nests) == 1:
            own = set(map(id, self.nests[0]._indices))
            self.orders[0] = [ix for ix in order if id(ix) in own]

    def skew(self, index, reference_index, unroll_loops_smaller_than=None):
        self.transformations.append(("skew", (index, reference_index)))

    def pad(self, index, size):
        self.transformations.append(("pad", (index, size)))

    def create_plan(self, target: Optional[Target] = None, **_ignored) -> "Plan":
        return Plan(self, target or Target.HOST)

    def _create_tensorizable_plan(self, target, block_indices, warp_indices, tensor_indices, outer_nest_order,
                                  dynamic_shared_memory_size: int = 0, blocks_per_SM: int = 0):
        """Helper of the reference's GPU tests (lang/Schedule.py:499-519): puts the three tensor indices
        innermost, binds block and warp indices to the grid and returns (plan, tensor_indices)."""
        self.reorder(*outer_nest_order, *tensor_indices)
        plan = self.create_plan(target=target)
        (i, j), (ii, jj) = block_indices, warp_indices
        units = Target.GridUnit
        plan.bind(mapping={i: units.BLOCK_Y, j: units.BLOCK_X, ii: units.WARP_Y, jj: units.WARP_X})
        return plan, tensor_indices


def fuse(*args, partial: Optional[int] = None) -> Schedule:
    """fuse(s0, s1, ..., partial=n) or fuse((s0, s1, ...), partial=n)."""
    scheds = list(args[0]) if len(args) == 1 and isinstance(args[0], (tuple, list)) else list(args)
    nests: List[Nest] = []
    orders: List[List[Index]] = []
    for s in scheds:
        if isinstance(s, Nest):
            s = s.create_schedule()
        if not isinstance(s, Schedule):
            raise TypeError("fuse takes schedules")
        nests.extend(s.nests)
        orders.extend(s.orders)
    if partial is None:
        partial = builtins_min(len(o) for o in orders)
    first = [ix.extent for ix in orders[0][:partial]]
    for o in orders:
        if len(o) < partial:
            raise ValueError("partial exceeds a nest's rank")
        if [ix.extent for ix in o[:partial]] != first:
            raise ValueError("fused dimensions must have equal extents")
    return Schedule(nests, partial, orders)


import builtins as _builtins  # noqa: E402
builtins_min = _builtins.min


class Plan:
    """Target-specific execution plan (lang/Plan.py).  Knobs are recorded; `tensorize` also selects
    the tensor-core kernel and its prologue / epilogue fragment ops."""
    def __init__(self, schedule: Schedule, target: Target):
        self.schedule = schedule
        self.target = target
        self.options: List[Tuple[str, Any]] = []
        self.bindings: Dict[Any, Any] = {}
        self.tensorized = False
        self.prologue_op = MMAFragmentOp.NONE
        self.prologue_arg = 0.0
        self.epilogue_op = MMAFragmentOp.NONE
        self.epilogue_arg = 0.0

    def unroll(self, index): self.options.append(("unroll", index))
    def vectorize(self, index): self.options.append(("vectorize", index))
    def parallelize(self, indices, pin=None, policy="static"): self.options.append(("parallelize", indices))
    def kernelize(self, unroll_indices, vectorize_indices=None): self.options.append(("kernelize", unroll_indices))

    def bind(self, mapping=None, **kwargs):
        """Binds schedule indices (or tuples of them) to grid units (lang/Plan.py:793-825).  The hand-written
        kernels choose their own launch geometry, so the binding does not steer them; it is kept, turned into the
        block and grid it asks for, and checked against the target's limits when the plan is added to a package,
        which is where the reference rejects an impossible launch too (lang/Plan.py:989-1004)."""
        if self.target is None or self.target.category is not Target.Category.GPU:
            raise ValueError("Only supported on plans with GPU targets")
        mapping = dict(mapping or {})
        for index_or_tuple, proc in mapping.items():
            if not isinstance(proc, Target.GridUnit):
                raise TypeError("bind maps indices to Target.GridUnit values")
            self.bindings[proc] = index_or_tuple
        self.options.append(("bind", mapping))

    def launch_request(self):
        """-> (block_dims, grid_dims) the plan's bindings and splits ask for (lang/Plan.py:879-956): block units
        give the grid, thread units the block, warp units a block of (warps_x * warp_size, warps_y, 1); without
        bindings a 16 x 16 block whose sides follow the split factors of the first two nest dimensions."""
        sched = self.schedule
        units = Target.GridUnit

        def fill(unit_list, dims):
            for pos, u in enumerate(unit_list):
                bound = self.bindings.get(u)
                if bound is None:
                    continue
                if not isinstance(bound, (tuple, list)):
                    bound = (bound,)
                n = 1
                for ix in bound:
                    n *= sched.iteration_count(ix)
                dims[pos] = n

        block, grid, warps = [1, 1, 1], [1, 1, 1], [0, 0]
        if self.bindings:
            fill([units.BLOCK_X, units.BLOCK_Y, units.BLOCK_Z], grid)
            fill([units.THREAD_X, units.THREAD_Y, units.THREAD_Z], block)
            fill([units.WARP_X, units.WARP_Y], warps)
            if any(warps):
                block = [warps[0] * self.target.warp_size, warps[1], 1]
        else:
            block = [16, 16, 1]
            nest = sched.nests[0]
            factors = sched.__dict__.get("_split_factor", {})
            children = {}
            for ix in sched.get_indices():
                if id(ix) in factors:
                    children.setdefault(ix.name[:-1], factors[id(ix)])
            for pos, ix in enumerate(nest._indices[:2]):
                if ix.name in children:
                    block[pos] = children[ix.name]
                if isinstance(ix.extent, int):
                    grid[pos] = -(-ix.extent // block[pos])
        return block, grid

    def check_launch_request(self) -> None:
        """Raises ValueError for a block the target cannot run (lang/Plan.py:958-1004, same messages)."""
        if self.target is None or self.target.category is not Target.Category.GPU:
            return
        try:
            block, _ = self.launch_request()
        except ValueError:
            return                              # runtime-sized nests: nothing static to check
        limit = self.target.max_block_size
        if len(limit) == 3 and any(block[i] > limit[i] for i in range(3)):
            raise ValueError(f"Invalid block dimensions: {block}. Largest supported block dimensions: {limit}.")
        if self.target.max_threads_per_block and block[0] * block[1] * block[2] > self.target.max_threads_per_block:
            raise ValueError(f"Invalid block size {block}. Max threads per block: {self.target.max_threads_per_block}.")

    def cache(self, source, index=None, trigger_index=None, layout=None, max_elements=None, element_type=None,
              thrifty=None, location=_MemorySpace.NONE, level=None, trigger_level=None, double_buffer=False,
              double_buffer_location=AUTO, vectorize=AUTO, strategy=AUTO, **kwargs):
        self.options.append(("cache", (source, location)))
        return source

    def tensorize(self, indices, mma_shape=None, num_total_passes: int = 1, use_static_offsets: bool = False,
                  num_fused_passes: Optional[int] = None, scheduling_policy=MMASchedulingPolicy.PASS_ORDER,
                  prologue_op: MMAFragmentOp = MMAFragmentOp.NONE, prologue_arg: float = 0.0,
                  epilogue_op: MMAFragmentOp = MMAFragmentOp.NONE, epilogue_arg: float = 0.0, **kwargs):
        self.options.append(("tensorize", (indices, mma_shape)))
        self.tensorized = True
        self.prologue_op, self.prologue_arg = prologue_op, float(prologue_arg)
        self.epilogue_op, self.epilogue_arg = epilogue_op, float(epilogue_arg)
