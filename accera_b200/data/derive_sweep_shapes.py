"""Derives accera_b200/data/gemm_sweep_reference_shapes.csv from the shape lists of the reference's GEMM benchmarker.

    python accera_b200/data/derive_sweep_shapes.py --reference-dir <reference checkout>/tools/benchmarkers

The reference's benchmarker reads problem sizes from CSV files next to it (gemm_square.csv, gemm_bert_assorted.csv,
gemm_resnet_inception.csv; columns as in tools/benchmarkers/gemm_opts.py:8-20).  The sweep of this package runs over a
selection of them, written here once so that the sweep itself needs no reference checkout:

  * gemm_square.csv             every size with row-major operands; all four layout combinations at 1024 and 4096
  * gemm_bert_assorted.csv      every row
  * gemm_resnet_inception.csv   the distinct (m, n, k, transA, transB) sorted by size, every 16th of them

alpha and beta are the files' (1, 1: C += A @ B, the nest the HAT functions implement); the leading dimensions are
carried along unchanged.
"""
import argparse
import csv
import os

HERE = os.path.dirname(os.path.abspath(__file__))


def read(path):
    with open(path) as f:
        rows = list(csv.DictReader(f))
    return rows


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference-dir", required=True)
    ap.add_argument("--output", default=os.path.join(HERE, "gemm_sweep_reference_shapes.csv"))
    a = ap.parse_args()
    cols = ["m", "n", "k", "transA", "transB", "alpha", "beta", "lda", "ldb", "ldc"]
    out = []
    sq = read(os.path.join(a.reference_dir, "gemm_square.csv"))
    out.append(("# from gemm_square.csv: every size row-major, all four layouts at 1024 and 4096", None))
    for r in sq:
        plain = r["transA"] == "0" and r["transB"] == "0"
        if plain or r["m"] in ("1024", "4096"):
            out.append((None, r))
    out.append(("# from gemm_bert_assorted.csv: every row", None))
    for r in read(os.path.join(a.reference_dir, "gemm_bert_assorted.csv")):
        out.append((None, r))
    out.append(("# from gemm_resnet_inception.csv: every 16th distinct shape in order of size", None))
    seen = {}
    for r in read(os.path.join(a.reference_dir, "gemm_resnet_inception.csv")):
        seen.setdefault((int(r["m"]), int(r["n"]), int(r["k"]), r["transA"], r["transB"]), r)
    keys = sorted(seen, key=lambda t: (t[0] * t[1] * t[2], t))
    for key in keys[::16]:
        out.append((None, seen[key]))
    with open(a.output, "w") as f:
        f.write(",".join(cols) + "\n")
        for comment, r in out:
            if comment:
                f.write(comment + "\n")
            else:
                f.write(",".join(str(r[c]).strip() for c in cols) + "\n")
    print(f"{sum(1 for c, r in out if r)} shapes -> {a.output}")


if __name__ == "__main__":
    main()
