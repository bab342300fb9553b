"""What the NVLink side of the sharded GEMM achieves on this box: run under torchrun, one rank per GPU.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 -m accera_b200.sharded_probe \
        [--m 65536 --n 8192 --k 8192] [--replicas R] [--copy-ctas 0,16,24,32] [--seconds 1.0] [--json out.json]

Every rank computes its shard of C += A @ B, ReLU (bf16, the benchmark's shapes by default) and the result is
written into every GPU's copy of C, as accera_b200.sharded.ShardedGemm(gather="fused") does.  Reported, as the
maximum over ranks of CUDA-event times:

  * peer copy            device-to-device copies of the shard's output bytes to the next rank (copy engines), one
                         direction and all ranks at once: the NVLink ceiling of this box for this many bytes
  * gemm only            the shard's GEMM with no replicas
  * stores only          the same launch with K = 512: the tensor cores have almost nothing to do, so the time is what
                         the stores to the peers take
  * fused                the full launch, for each way of feeding the peers: 0 = the computing CTAs' epilogues store to
                         every replica themselves, c > 0 = c forwarding CTAs (see csrc/gemm_umma.cu, copy_tiles)

`--replicas R` (default: one per rank) lets a box with fewer GPUs reproduce the traffic of a larger one: with 2 ranks
and --replicas 8 every rank holds 8 copies of its shard-sized C, computes an 8-GPU shard (M / 8 rows) and writes it to
its own copy and to 7 copies in the one peer's memory - the bytes per GPU and direction of the 8-GPU run over one
NVLink hop through the switch.
"""
from __future__ import annotations

import argparse
import json
import os
import time


def main() -> None:
    import torch
    import torch.distributed as dist
    import torch.distributed._symmetric_memory as symm_mem
    from . import runtime as rt

    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, default=65536)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--replicas", type=int, default=0, help="copies of C fed by every rank (default: the number of ranks)")
    ap.add_argument("--copy-ctas", default="0,-1", help="comma-separated forwarding-CTA counts to try (-1 = the library's choice)")
    ap.add_argument("--seconds", type=float, default=0.0, help="also report a sustained figure over this many seconds per variant")
    ap.add_argument("--json", default="")
    a = ap.parse_args()

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    replicas = a.replicas or world
    if replicas < 1 or replicas > 8 or (replicas - 1) % max(world - 1, 1) != 0 and world > 1:
        raise SystemExit("--replicas must be 1..8 and (replicas - 1) a multiple of (ranks - 1)")
    rows = a.m // replicas                                   # the shard of one GPU of a `replicas`-GPU run
    n, k = a.n, a.k
    per_peer = (replicas - 1) // max(world - 1, 1)           # copies of C that every peer holds for me
    # symmetric memory: slot 0 = my own C shard, slots 1.. = the copies peers write into
    buf = symm_mem.empty((1 + per_peer * max(world - 1, 1), rows, n), dtype=torch.bfloat16, device=dev)
    buf.zero_()
    hdl = symm_mem.rendezvous(buf, dist.group.WORLD)
    peers = []
    for step in range(1, world):
        p = (rank + step) % world
        pb = hdl.get_buffer(p, tuple(buf.shape), buf.dtype)
        for c in range(per_peer):
            peers.append(pb[1 + (world - 1 - step) * per_peer + c] if world > 2 else pb[1 + c])
    torch.manual_seed(rank)
    A = torch.randn(rows, k, device=dev).to(torch.bfloat16)
    B = (torch.randn(n, k, device=dev) / k ** 0.5).to(torch.bfloat16).t()
    A_small, B_small = A[:, :512].contiguous(), B[:512, :].t().contiguous().t()
    out_bytes = (replicas - 1) * rows * n * 2
    results = {"ranks": world, "replicas": replicas, "shard": [rows, n, k], "bytes_out_per_gpu": out_bytes}

    def timed(fn, iters=10, warm=3, seconds=0.0):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize(dev)
        dist.barrier()
        torch.cuda.synchronize(dev)
        if seconds > 0:
            c0 = time.perf_counter()
            fn(); fn()
            torch.cuda.synchronize(dev)
            iters = int(min(5000, max(10, seconds / max((time.perf_counter() - c0) / 2, 1e-5))))
            t = torch.tensor([iters], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MIN)
            iters = int(t.item())
            dist.barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(iters):
            fn()
        e.record()
        torch.cuda.synchronize(dev)
        t = torch.tensor([s.elapsed_time(e) / iters], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def report(name, ms, bytes_moved=0, flops=0.0):
        if rank == 0:
            rec = {"ms": ms}
            txt = f"{name:58s} {ms:8.3f} ms"
            if bytes_moved:
                rec["GB/s_per_direction"] = bytes_moved / ms / 1e6
                txt += f"  {rec['GB/s_per_direction']:7.1f} GB/s out (and in) per GPU"
            if flops:
                rec["TFLOP/s_per_gpu"] = flops / ms / 1e9
                txt += f"  {rec['TFLOP/s_per_gpu']:7.0f} TFLOP/s per GPU"
            results[name] = rec
            print(txt, flush=True)

    flops = 2.0 * rows * n * k
    if world > 1:
        nxt = hdl.get_buffer((rank + 1) % world, tuple(buf.shape), buf.dtype)
        chunk = buf[0]

        def copy_out():
            for c in range(min(replicas - 1, nxt.shape[0] - 1)):
                nxt[1 + c].copy_(chunk, non_blocking=True)
        copies = min(replicas - 1, nxt.shape[0] - 1)
        ms = timed(copy_out)
        report(f"peer copy of {copies} x {rows * n * 2 >> 20} MiB to the next rank, all ranks at once", ms, copies * rows * n * 2)
    ms = timed(lambda: rt.gemm(A, B, buf[0], beta=1.0, relu=True, compute="tensor_2sm"), seconds=a.seconds)
    report("gemm only (no replicas)", ms, 0, flops)
    reps = [buf[0]] + peers
    for cc in [int(x) for x in a.copy_ctas.split(",")]:
        tag = "library's choice" if cc < 0 else ("stores from the epilogues" if cc == 0 else f"{cc} forwarding CTAs")
        with rt.options(**{"gemm.copy_ctas": cc}):
            if world > 1:
                ms = timed(lambda: rt.gemm_replicated(A_small, B_small, reps, beta=1.0, relu=True))
                report(f"stores only (K = 512), {tag}", ms, out_bytes)
            ms = timed(lambda: rt.gemm_replicated(A, B, reps, beta=1.0, relu=True))
            report(f"fused, {tag}", ms, out_bytes, flops)
            if a.seconds > 0:
                ms = timed(lambda: rt.gemm_replicated(A, B, reps, beta=1.0, relu=True), seconds=a.seconds)
                report(f"fused, {tag}, sustained {a.seconds:g} s", ms, out_bytes, flops)
    rt.synchronize()
    if rank == 0 and a.json:
        with open(a.json, "w") as f:
            json.dump(results, f, indent=1)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
