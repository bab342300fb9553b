#!/usr/bin/env python
"""Generates the golden vectors in this directory from the reference's own Python sources.

    python tests/golden/make_golden.py /path/to/reference        (a checkout of the reference project)

The reference stores no known-answer vectors for its matmul+ReLU, reduce_mean or gather functions,
and its compiler cannot be built offline.  What it does hold, and what this script executes:

  gather       kernels/gather/naive_runtime_sized.py::generate_numpy_rank_2 - the reference's own
               numpy loop restatement of the gather nests; imported as-is (its `import accera`
               is satisfied by this repository's DSL subset) and run on seeded inputs, including
               the 5x4 / [[0,1],[1,2]] case of its verify().
  reduce_mean  kernels/reduce_mean/naive_runtime_sized.py::reduce_mean_schedule - the reference's
               nest builders (_init_buffer, _accumulate_buffer, _div_buffer, _reorder_schedule, fuse)
               are called unmodified; the schedule they return is executed point by point by the
               loop-nest interpreter below (fp32 scalars, loop order = schedule order).
  matmul+ReLU  the quickstart code block of README.md, extracted from the markdown, its sizes
               shrunk textually (512 -> 24) and package.build stripped, executed the same way.

The interpreter follows the reference's semantics for fused schedules: for every point of the
fused dimensions each nest runs, in order, over all of its remaining dimensions
(docs/Reference/safety_analysis.md:28-34).  Arithmetic is done on numpy fp32 scalars so that
every multiply and add is rounded separately, as the reference's un-vectorised HOST code does.

  range        kernels/range/naive_runtime_sized.py::generate_numpy - the reference's numpy loop, run as-is.

Outputs: gather.npz, reduce_mean.npz, matmul_relu.npz, range.npz (a few KB to a few tens of KB each).
"""
import importlib.util
import itertools
import os
import re
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import accera_b200 as acc            # noqa: E402
from accera_b200 import lang         # noqa: E402

_NP = {"float32": np.float32, "float16": np.float16, "float64": np.float64, "int8": np.int8, "int32": np.int32,
       "int64": np.int64, "index": np.int64, "uint8": np.uint8}


class Interpreter:
    """Executes a traced Schedule on numpy arrays bound to its Array objects."""

    def __init__(self, bindings):
        self.arrays = {id(a): v for a, v in bindings}

    def eval(self, e, env):
        if isinstance(e, lang.Index):
            return env[id(e)]
        if isinstance(e, lang.Const):
            return e.value
        if isinstance(e, lang.Access):
            idx = tuple(int(self.eval(i, env)) for i in e.indices)
            return self.arrays[id(e.array)][idx]
        if isinstance(e, lang.BinOp):
            a, b = self.eval(e.lhs, env), self.eval(e.rhs, env)
            return {"+": lambda: a + b, "-": lambda: a - b, "*": lambda: a * b, "/": lambda: a / b}[e.op]()
        if isinstance(e, lang.Call):
            args = [self.eval(a, env) for a in e.args]
            if e.fn == "cast":
                return _NP[e.dtype.value](args[0])
            if e.fn == "max":
                return args[0] if args[0] >= args[1] else args[1]
            if e.fn == "min":
                return args[0] if args[0] <= args[1] else args[1]
            if e.fn == "abs":
                return abs(args[0])
        raise NotImplementedError(repr(e))

    def exec_statement(self, s, env):
        arr = self.arrays[id(s.target.array)]
        idx = tuple(int(self.eval(i, env)) for i in s.target.indices)
        dt = arr.dtype.type
        v = self.eval(s.value, env)
        if s.op == "=":
            arr[idx] = dt(v)
        else:
            cur = arr[idx]
            arr[idx] = dt({"+": lambda: cur + dt(v), "-": lambda: cur - dt(v), "*": lambda: cur * dt(v),
                           "/": lambda: cur / dt(v)}[s.op]())

    def run(self, schedule):
        partial = schedule.partial or 0
        fused_extents = [ix.extent for ix in schedule.orders[0][:partial]]
        for point in itertools.product(*[range(e) for e in fused_extents]):
            for nest, order in zip(schedule.nests, schedule.orders):
                env = {id(ix): p for ix, p in zip(order[:partial], point)}
                rest = order[partial:]
                for q in itertools.product(*[range(ix.extent) for ix in rest]):
                    for ix, v in zip(rest, q):
                        env[id(ix)] = v
                    for s in nest.statements:
                        self.exec_statement(s, env)


def load_reference_module(path, name):
    """Imports a reference Python file whose only dependency is `import accera`."""
    sys.modules["accera"] = acc
    try:
        spec = importlib.util.spec_from_file_location(name, path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
    finally:
        del sys.modules["accera"]
    return mod


def make_gather(ref):
    mod = load_reference_module(os.path.join(ref, "kernels", "gather", "naive_runtime_sized.py"), "ref_gather")
    rng = np.random.default_rng(4101)
    out = {}
    cases = {"verify": (rng.standard_normal((5, 4)).astype(np.float32), np.array([[0, 1], [1, 2]], dtype=np.int64)),
             "wide": (rng.standard_normal((37, 16)).astype(np.float32), rng.integers(0, 16, size=(3, 5), dtype=np.int64)),
             "single": (rng.standard_normal((9, 130)).astype(np.float32), rng.integers(0, 9, size=(6, 1), dtype=np.int64))}
    for name, (data, idx) in cases.items():
        out[f"{name}_data"], out[f"{name}_indices"] = data, idx
        for axis in (0, 1):
            out[f"{name}_axis{axis}"] = mod.generate_numpy_rank_2(axis)(data, idx)
    np.savez(os.path.join(HERE, "gather.npz"), **out)
    return out


def make_range(ref):
    """kernels/range/naive_runtime_sized.py::generate_numpy - the reference's own numpy loop for Range
    (`output[i] = start; start += delta` on np.float32 scalars, size `int((limit - start) // delta)`), run on
    the case of its verify() (1, 5, 2), on the case of dsl_tests.py:1479-1481 (1, 5, 0.5) and on ranges that
    cross binades, run downwards, cross zero and stall (delta below half an ulp of the running value)."""
    mod = load_reference_module(os.path.join(ref, "kernels", "range", "naive_runtime_sized.py"), "ref_range")
    fn = mod.generate_numpy()
    cases = {"verify": (1.0, 5.0, 2.0), "dsl_test": (1.0, 5.0, 0.5), "tenths": (0.0, 1000.3, 0.1),
             "binades": (0.001, 300.0, 0.37), "down": (10.0, -3.0, -0.25), "cross_zero": (-7.3, 9.1, 0.013),
             "thirds": (1.0, 4097.0, 1.0 / 3.0), "stall": (16777216.0, 16779000.0, 0.75), "tie": (8388608.0, 8390000.0, 0.5),
             "tiny": (1e-40, 3e-38, 1.7e-41)}
    out = {}
    for name, (start, limit, delta) in cases.items():
        s, l, d = np.float32(start), np.float32(limit), np.float32(delta)
        with np.errstate(all="ignore"):
            y = fn(s, l, d)
        out[f"{name}_args"] = np.array([s, l, d], dtype=np.float32)
        out[f"{name}_out"] = y
    np.savez(os.path.join(HERE, "range.npz"), **out)
    return out


def make_reduce_mean(ref):
    mod = load_reference_module(os.path.join(ref, "kernels", "reduce_mean", "naive_runtime_sized.py"), "ref_reduce_mean")
    rng = np.random.default_rng(4102)
    shape = [4, 6, 5]
    data_np = rng.standard_normal(shape).astype(np.float32)
    out = {"data": data_np}
    for axes in ([0], [1], [2], [0, 1], [0, 2], [1, 2], [0, 1, 2]):
        for keepdims in (0, 1):
            oshape = [1 if d in axes else s for d, s in enumerate(shape)] if keepdims else \
                     ([s for d, s in enumerate(shape) if d not in axes] or [1])
            data = acc.Array(role=acc.Role.INPUT, element_type=acc.ScalarType.float32, shape=shape)
            reduced = acc.Array(role=acc.Role.INPUT_OUTPUT, element_type=acc.ScalarType.float32, shape=oshape)
            schedule = mod.reduce_mean_schedule(data, reduced, axes, keepdims)
            red_np = np.full(oshape, np.float32(777.0), dtype=np.float32)      # junk: the init nest must clear it
            Interpreter([(data, data_np), (reduced, red_np)]).run(schedule)
            out[f"axes{''.join(map(str, axes))}_keep{keepdims}"] = red_np
    np.savez(os.path.join(HERE, "reduce_mean.npz"), **out)
    return out


def make_matmul_relu(ref):
    text = open(os.path.join(ref, "README.md")).read()
    m = re.search(r"```python\n([ ]*import accera as acc\n.*?)```", text, re.S)
    if not m:
        raise RuntimeError("quickstart block not found in the reference README")
    code = m.group(1)
    import textwrap
    code = textwrap.dedent(code)                                   # the block sits inside a markdown list item
    code = code.replace("512", "24")
    code = re.sub(r"^print\(package\.build\(.*$", "", code, flags=re.M)
    ns = {}
    sys.modules["accera"] = acc
    try:
        exec(compile(code, "README.md:quickstart", "exec"), ns)
    finally:
        del sys.modules["accera"]
    A, B, C, schedule = ns["A"], ns["B"], ns["C"], ns["schedule"]
    out = {}
    for name, signed in (("unit", False), ("signed", True)):
        rng = np.random.default_rng(4103 + signed)
        a = rng.random((24, 24), dtype=np.float32)
        b = rng.random((24, 24), dtype=np.float32)
        c = np.zeros((24, 24), dtype=np.float32)
        if signed:
            a -= np.float32(0.5)
            b -= np.float32(0.5)
            c = rng.standard_normal((24, 24)).astype(np.float32)
        c_out = c.copy()
        Interpreter([(A, a), (B, b), (C, c_out)]).run(schedule)
        out[f"{name}_A"], out[f"{name}_B"], out[f"{name}_C_in"], out[f"{name}_C_out"] = a, b, c, c_out
    np.savez(os.path.join(HERE, "matmul_relu.npz"), **out)
    return out


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py /path/to/reference")
    ref = sys.argv[1]
    g = make_gather(ref)
    r = make_reduce_mean(ref)
    m = make_matmul_relu(ref)
    rg = make_range(ref)
    print(f"gather: {len(g)} arrays, reduce_mean: {len(r)} arrays, matmul_relu: {len(m)} arrays, range: {len(rg)} arrays")


if __name__ == "__main__":
    main()
