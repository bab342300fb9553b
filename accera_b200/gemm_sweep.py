"""GEMM shape sweep: times the library's GEMM over a CSV list of problem sizes.

Same input format and reporting as the reference's GEMM benchmarker
(tools/benchmarkers/gemm_opts.py:8-33 for the columns, tools/benchmarkers/accera_gemm.py:152-176
for what transA/transB mean there, :640-660 for the TFLOP/s formula):

    m,n,k,transA,transB,alpha,beta,lda,ldb,ldc
    2048,2048,2048,0,0,1,1,2048,2048,2048

A is M x K, B is K x N, C is M x N row-major.  transA / transB select the LAST_MAJOR
(column-major) layout for A / B, FIRST_MAJOR otherwise.  lda/ldb/ldc are read and carried along
but, as in the reference's own benchmarker, do not change the arrays (they describe the BLAS
comparators' view of the same memory).  Throughput is 2*M*N*K / t with t the smallest of the
per-batch mean times ("min_of_means", hatlib's figure).

Where the reference searches a space of schedules per shape and keeps the best one, the kernels
here bring their own tiling, so there is one timing per shape and per compute mode.

    python -m accera_b200.gemm_sweep --input shapes.csv --type h --output results.csv
"""
from __future__ import annotations

import argparse
import csv
import dataclasses
import io
import json
import sys
from typing import Iterable, List, Optional, Sequence

COLUMNS = ("m", "n", "k", "transA", "transB", "alpha", "beta", "lda", "ldb", "ldc")

# --type letters: 's' and 'h' are the reference's (single, half); the others are the extra input types of the B200 path
TYPE_NAMES = {"s": "float32", "h": "float16", "b": "bfloat16", "i": "int8", "u": "uint8"}


def output_type(type_letter: str, out_letter: Optional[str] = None) -> str:
    """Letter of C's element type: the input type unless `out_letter` asks for fp32 ('s'); 8-bit integer
    inputs always accumulate into and store int32 ('w').  These are the (input, output) pairs of the
    reference's tensor-core table (accera/python/accera/Targets.py:833-850)."""
    if type_letter in ("i", "u"):
        if out_letter not in (None, "w"):
            raise ValueError("8-bit integer GEMMs store int32")
        return "w"
    if out_letter in (None, type_letter):
        return type_letter
    if out_letter == "s":
        return "s"
    raise ValueError(f"no GEMM with input type {type_letter!r} and output type {out_letter!r}")


@dataclasses.dataclass(frozen=True)
class GemmShape:
    m: int
    n: int
    k: int
    transA: bool = False
    transB: bool = False
    alpha: float = 1.0
    beta: float = 0.0
    lda: int = 0
    ldb: int = 0
    ldc: int = 0

    def __post_init__(self):
        if self.m <= 0 or self.n <= 0 or self.k <= 0:
            raise ValueError(f"m, n and k must be positive, got {self.m}, {self.n}, {self.k}")

    @property
    def flop(self) -> float:
        return 2.0 * self.m * self.n * self.k

    def as_row(self) -> List:
        return [self.m, self.n, self.k, int(self.transA), int(self.transB), self.alpha, self.beta,
                self.lda, self.ldb, self.ldc]


def _flag(text: str) -> bool:
    t = text.strip().lower()
    if t in ("1", "true", "t", "y", "yes"):
        return True
    if t in ("0", "false", "f", "n", "no", ""):
        return False
    raise ValueError(f"not a 0/1 flag: {text!r}")


def parse_shapes(lines: Iterable[str]) -> List[GemmShape]:
    """Reads the CSV.  The header line is optional; when present it may give the columns in any order and
    leave out the trailing ones (alpha defaults to 1, beta to 0, the leading dimensions to 0).  Blank lines
    and lines starting with '#' are skipped."""
    rows = [r for r in csv.reader(l for l in lines if l.strip() and not l.lstrip().startswith("#"))]
    if not rows:
        return []
    first = [c.strip() for c in rows[0]]
    if any(c in COLUMNS for c in first):
        unknown = [c for c in first if c not in COLUMNS]
        if unknown:
            raise ValueError(f"unknown column(s) {unknown}; expected a subset of {list(COLUMNS)}")
        header, rows = first, rows[1:]
    else:
        header = list(COLUMNS)
    for need in ("m", "n", "k"):
        if need not in header:
            raise ValueError(f"column {need!r} is required")
    out = []
    for lineno, r in enumerate(rows, 1):
        if len(r) > len(header):
            raise ValueError(f"row {lineno}: {len(r)} fields for {len(header)} columns")
        f = dict(zip(header, (c.strip() for c in r)))
        try:
            out.append(GemmShape(
                m=int(f["m"]), n=int(f["n"]), k=int(f["k"]),
                transA=_flag(f.get("transA", "0")), transB=_flag(f.get("transB", "0")),
                alpha=float(f.get("alpha", "1") or 1), beta=float(f.get("beta", "0") or 0),
                lda=int(f.get("lda", "0") or 0), ldb=int(f.get("ldb", "0") or 0), ldc=int(f.get("ldc", "0") or 0)))
        except (KeyError, ValueError) as e:
            raise ValueError(f"row {lineno}: {e}") from None
    return out


def operand_strides(shape: GemmShape):
    """Element strides ((a0, a1), (b0, b1), (c0, c1)) of the three arrays for one CSV row."""
    a = (1, shape.m) if shape.transA else (shape.k, 1)
    b = (1, shape.k) if shape.transB else (shape.n, 1)
    return a, b, (shape.n, 1)


def _strided(torch, rows: int, cols: int, last_major: bool, dtype, device, gen):
    """A [rows, cols] tensor of small random values whose memory is column-major when last_major."""
    r, c = (cols, rows) if last_major else (rows, cols)
    if dtype == torch.int8:
        t = torch.randint(-4, 5, (r, c), dtype=torch.int8, device=device, generator=gen)
    elif dtype == torch.uint8:
        t = torch.randint(0, 9, (r, c), dtype=torch.uint8, device=device, generator=gen)
    else:
        t = (torch.rand(r, c, device=device, generator=gen, dtype=torch.float32) - 0.5).to(dtype)
    return t.t() if last_major else t


def make_operands(shape: GemmShape, type_letter: str, device, seed: int = 0, out_letter: Optional[str] = None):
    import torch
    letters = {"s": torch.float32, "h": torch.float16, "b": torch.bfloat16, "i": torch.int8, "u": torch.uint8,
               "w": torch.int32}
    dtype = letters[type_letter]
    out_dtype = letters[output_type(type_letter, out_letter)]
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    A = _strided(torch, shape.m, shape.k, shape.transA, dtype, device, gen)
    B = _strided(torch, shape.k, shape.n, shape.transB, dtype, device, gen)
    if out_dtype == torch.int32:
        C = torch.randint(-100, 100, (shape.m, shape.n), dtype=torch.int32, device=device, generator=gen)
    else:
        C = (torch.rand(shape.m, shape.n, device=device, generator=gen, dtype=torch.float32) - 0.5).to(out_dtype)
    return A, B, C


def _time_batches(fn, batches: int, batch_size: int) -> List[float]:
    """Mean seconds per call of each batch, timed with CUDA events on the current stream."""
    import torch
    means = []
    for _ in range(batches):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(batch_size):
            fn()
        e1.record()
        e1.synchronize()
        means.append(e0.elapsed_time(e1) * 1e-3 / batch_size)
    return means


def _reference_result(torch, A, B, C0, shape: GemmShape):
    if A.dtype in (torch.int8, torch.uint8):
        # exact: |values| <= 8, so fp64 accumulation holds every partial sum
        acc = (A.double() @ B.double()) * shape.alpha + shape.beta * C0.double()
        return acc
    return (A.float() @ B.float()) * shape.alpha + shape.beta * C0.float()


def run_shape(shape: GemmShape, type_letter: str = "h", compute: str = "tensor_preferred", device=None,
              batches: int = 5, batch_size: int = 0, warmup: int = 3, check: bool = True,
              compare_torch: bool = False, seed: int = 0, out_letter: Optional[str] = None) -> dict:
    """Times one row of the sweep on the current GPU and returns one result record."""
    import torch
    from . import runtime
    if not torch.cuda.is_available():
        raise RuntimeError("gemm_sweep needs a CUDA device: there is no CPU path")
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    A, B, C = make_operands(shape, type_letter, device, seed, out_letter)
    C0 = C.clone()
    integer = type_letter in ("i", "u")
    if type_letter == "s" and compute in ("tensor", "tensor_2sm") and (shape.transA or not shape.transB):
        raise ValueError("TF32 on the tensor cores needs K-contiguous operands (transA=0, transB=1); "
                         "use compute='tensor_preferred' or 'simt'")

    # the descriptor is built once, like the constant descriptor of a compiled HAT stub: the timed loop is C-ABI calls only
    call = runtime.gemm_call(A, B, C, alpha=shape.alpha, beta=shape.beta, compute=compute)

    rec = dict(zip(COLUMNS, shape.as_row()))
    rec.update(type=type_letter, out_type=output_type(type_letter, out_letter), compute=compute)
    if check:
        C.copy_(C0)
        call()
        torch.cuda.synchronize()
        want = _reference_result(torch, A, B, C0, shape)
        got = C.double() if integer else C.float()
        scale = float(want.abs().max().clamp_min(1e-30))
        rec["max_rel_err"] = float((got - want).abs().max()) / scale
    if batch_size <= 0:
        # enough calls per batch for ~20 ms of device time, so that launch gaps and event overhead vanish
        call()
        torch.cuda.synchronize()
        t = _time_batches(call, 1, 3)[0]
        batch_size = int(min(2000, max(5, 0.02 / max(t, 1e-7))))
    for _ in range(warmup):
        call()
    means = _time_batches(call, batches, batch_size)
    best = min(means)
    rec.update(batch_size=batch_size, min_of_means_s=best, mean_of_means_s=sum(means) / len(means),
               tflops=shape.flop / best * 1e-12)
    if compare_torch and not integer and C.dtype == A.dtype:
        alpha, beta = shape.alpha, shape.beta

        def torch_call():
            if beta == 0.0:
                torch.mm(A, B, out=C)
                if alpha != 1.0:
                    C.mul_(alpha)
            else:
                torch.addmm(C, A, B, beta=beta, alpha=alpha, out=C)

        for _ in range(warmup):
            torch_call()
        tbest = min(_time_batches(torch_call, batches, batch_size))
        rec.update(torch_min_of_means_s=tbest, torch_tflops=shape.flop / tbest * 1e-12)
    return rec


RESULT_COLUMNS = list(COLUMNS) + ["type", "out_type", "compute", "batch_size", "min_of_means_s", "mean_of_means_s", "tflops",
                                  "max_rel_err", "torch_min_of_means_s", "torch_tflops", "error"]


def write_results(records: Sequence[dict], stream) -> None:
    cols = [c for c in RESULT_COLUMNS if any(c in r for r in records)]
    w = csv.DictWriter(stream, fieldnames=cols, extrasaction="ignore")
    w.writeheader()
    for r in records:
        w.writerow({c: r.get(c, "") for c in cols})


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--input", "-i", required=True, help="CSV of shapes (columns: " + ",".join(COLUMNS) + ")")
    ap.add_argument("--type", "-t", default="h", choices=sorted(TYPE_NAMES), help="input type: s=fp32 h=fp16 b=bf16 i=int8 u=uint8 (8-bit types store int32)")
    ap.add_argument("--out-type", default=None, choices=["s", "h", "b", "w"],
                    help="C's type when it differs from the input type: s = fp32 output for h / b inputs")
    ap.add_argument("--compute", default="tensor_preferred",
                    choices=["auto", "simt", "tensor", "tensor_2sm", "tensor_preferred"])
    ap.add_argument("--output", "-o", default=None, help="CSV of results (default: stdout)")
    ap.add_argument("--batches", type=int, default=5)
    ap.add_argument("--batch-size", type=int, default=0, help="calls per timed batch (0 = sized for ~20 ms)")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-check", action="store_true", help="skip the comparison with torch's fp32 matmul")
    ap.add_argument("--torch", action="store_true", help="also time torch.mm / torch.addmm (cuBLAS) on the same operands")
    ap.add_argument("--json", action="store_true", help="one JSON object per shape instead of CSV")
    args = ap.parse_args(argv)
    with open(args.input) as f:
        shapes = parse_shapes(f)
    if not shapes:
        print("no shapes in " + args.input, file=sys.stderr)
        return 1
    from .runtime import AccbError
    records = []
    for s in shapes:
        try:
            rec = run_shape(s, args.type, args.compute, batches=args.batches, batch_size=args.batch_size,
                            warmup=args.warmup, check=not args.no_check, compare_torch=args.torch, out_letter=args.out_type)
        except (AccbError, ValueError) as e:
            # a row this type / compute mode cannot run (e.g. alpha != 1 with integer inputs) is reported, not fatal
            rec = dict(zip(COLUMNS, s.as_row()))
            rec.update(type=args.type, compute=args.compute, error=str(e))
            records.append(rec)
            print(f"{s.m}x{s.n}x{s.k} tA={int(s.transA)} tB={int(s.transB)}: skipped: {e}", file=sys.stderr)
            continue
        records.append(rec)
        print(f"{s.m}x{s.n}x{s.k} tA={int(s.transA)} tB={int(s.transB)}: {rec['tflops']:.2f} TFLOP/s"
              + (f" (torch {rec['torch_tflops']:.2f})" if "torch_tflops" in rec else "")
              + (f" err {rec['max_rel_err']:.2e}" if "max_rel_err" in rec else ""), file=sys.stderr)
    buf = io.StringIO()
    if args.json:
        for r in records:
            buf.write(json.dumps(r) + "\n")
    else:
        write_results(records, buf)
    if args.output:
        with open(args.output, "w") as f:
            f.write(buf.getvalue())
    else:
        sys.stdout.write(buf.getvalue())
    return 0


if __name__ == "__main__":
    sys.exit(main())
