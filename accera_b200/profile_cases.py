"""Runs one hot-path kernel a few times on device-resident inputs - the command to put under a profiler.

    python -m accera_b200.profile_cases gemm_bf16 [--m 8192 --n 8192 --k 8192] [--compute tensor_2sm] [--iters 3] [--beta 1.0]
    python -m accera_b200.profile_cases reduce_mean [--rows 8192 --cols 4096]
    python -m accera_b200.profile_cases gather [--table-rows 32000 --cols 4096 --indices 16384]
    python -m accera_b200.profile_cases matmul_relu_f32 [--m 512 --n 512 --k 512]
    python -m accera_b200.profile_cases range [--elements 134217728]
    python -m accera_b200.profile_cases gemm_f16 | gemm_s8 | gemm_tf32 [--m --n --k]      (row-major A, column-major B)
    python -m accera_b200.profile_cases reduce_cols [--rows 4096 --cols 8192]              (mean over the first axis)
    python -m accera_b200.profile_cases gather_elem [--table-rows 4096 --cols 32000 --indices 16384]   (gather along axis 1)

Sizes default to cases whose inputs exceed the 126 MB L2 while holding well under a
few GB on the device, so that a multi-pass profiler capture stays short.
"""
from __future__ import annotations

import argparse

import torch

from . import runtime as rt


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["gemm_bf16", "gemm_f16", "gemm_s8", "gemm_tf32", "reduce_mean", "reduce_cols", "gather", "gather_elem",
                                     "matmul_relu_f32", "range"])
    ap.add_argument("--elements", type=int, default=1 << 27)
    ap.add_argument("--m", type=int, default=None)
    ap.add_argument("--n", type=int, default=None)
    ap.add_argument("--k", type=int, default=None)
    ap.add_argument("--rows", type=int, default=8192)
    ap.add_argument("--cols", type=int, default=4096)
    ap.add_argument("--table-rows", type=int, default=32000)
    ap.add_argument("--indices", type=int, default=16384)
    ap.add_argument("--compute", default="tensor_2sm")
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--beta", type=float, default=1.0, help="GEMM cases: C <- A @ B + beta * C")
    ap.add_argument("--a-col-major", action="store_true", help="gemm_bf16 / gemm_f16: A stored column-major (M contiguous)")
    ap.add_argument("--b-row-major", action="store_true", help="gemm_bf16 / gemm_f16: B stored row-major (N contiguous)")
    ap.add_argument("--option", action="append", default=[], metavar="NAME=VALUE",
                    help="a launch override for this run, e.g. gemm.group_n=16 (see accb_set_option)")
    a = ap.parse_args()
    for item in a.option:
        name, _, value = item.partition("=")
        rt.set_option(name, int(value))
    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    if a.case.startswith("gemm_"):
        m, n, k = a.m or 8192, a.n or 8192, a.k or 8192
        if a.case == "gemm_s8":
            A = torch.randint(-128, 128, (m, k), device=dev, dtype=torch.int8)
            B = torch.randint(-128, 128, (n, k), device=dev, dtype=torch.int8).t()
            C = torch.zeros(m, n, device=dev, dtype=torch.int32)
        elif a.case == "gemm_tf32":
            A = torch.randn(m, k, device=dev)
            B = (torch.randn(n, k, device=dev) / k ** 0.5).t()
            C = torch.zeros(m, n, device=dev)
        else:
            dt = torch.bfloat16 if a.case == "gemm_bf16" else torch.float16
            A = torch.randn(k, m, device=dev).to(dt).t() if a.a_col_major else torch.randn(m, k, device=dev).to(dt)
            B = (torch.randn(k, n, device=dev) / k ** 0.5).to(dt) if a.b_row_major else (torch.randn(n, k, device=dev) / k ** 0.5).to(dt).t()
            C = torch.zeros(m, n, device=dev, dtype=dt if a.case == "gemm_bf16" else torch.float32)
        for _ in range(a.iters):
            rt.gemm(A, B, C, beta=a.beta, relu=a.case != "gemm_s8", compute=a.compute)
    elif a.case == "matmul_relu_f32":
        m, n, k = a.m or 512, a.n or 512, a.k or 512
        A = torch.rand(m, k, device=dev); B = torch.rand(k, n, device=dev); C = torch.zeros(m, n, device=dev)
        for _ in range(a.iters):
            rt.gemm(A, B, C, relu=True, compute="simt")
    elif a.case == "range":
        out = torch.empty(a.elements, device=dev)
        for _ in range(a.iters):
            rt.range_f32(out, 0.0, 0.001)
    elif a.case == "reduce_cols":
        x = torch.randn(1, a.rows, a.cols, device=dev)
        y = torch.empty(a.cols, device=dev)
        for _ in range(a.iters):
            rt.reduce_mean_rank3(x, y, [1])
    elif a.case == "gather_elem":
        T = torch.randn(a.table_rows, a.cols, device=dev) * 0.02
        idx = torch.randint(0, a.cols, (a.indices, 1), device=dev)
        out = torch.empty(a.table_rows, a.indices, 1, device=dev)
        for _ in range(a.iters):
            rt.gather_rank2(T, idx, out, 1)
    elif a.case == "reduce_mean":
        x = torch.randn(1, a.rows, a.cols, device=dev)
        y = torch.empty(a.rows, device=dev)
        for _ in range(a.iters):
            rt.reduce_mean_rank3(x, y, [2])
    else:
        T = torch.randn(a.table_rows, a.cols, device=dev) * 0.02
        idx = torch.randint(0, a.table_rows, (a.indices, 1), device=dev)
        out = torch.empty(a.indices, 1, a.cols, device=dev)
        for _ in range(a.iters):
            rt.gather_rank2(T, idx, out, 0)
    rt.synchronize()
    torch.cuda.synchronize()
    print(f"{a.case}: {a.iters} launches done, {rt.launch_count()} kernels launched by the library")


if __name__ == "__main__":
    main()
