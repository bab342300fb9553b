"""GEMM(+ReLU) sharded by M-row blocks over the GPUs of one box, C reassembled with an all-gather.

The reference has no multi-GPU path at all (no collective call anywhere in its
tree); this is new work around the same HAT GEMM function.  One process per GPU:

  * B (K x N, column-major) is replicated in every GPU's own HBM.
  * C's M rows are cut into `world * chunks` blocks of `block_rows` rows and dealt
    out block-cyclically: block b belongs to rank b % world.  Rank r therefore
    owns blocks r, world + r, 2*world + r, ... and holds the matching rows of A
    concatenated in that order (`shard_rows`).
  * For chunk j every rank computes its block (j*world + r) straight into its
    slot of the full C; the `world` blocks of chunk j are adjacent in C, so one
    in-place all-gather per chunk reassembles them with no staging copy.
  * The all-gather of chunk j runs on a second stream while the GEMM of chunk
    j+1 computes.

No kernel reads or writes another GPU's memory; NCCL is the only cross-GPU mover.
The data path has no other collective.
"""
from __future__ import annotations

import dataclasses
from typing import Callable, List, Optional, Tuple


@dataclasses.dataclass(frozen=True)
class RowBlockPlan:
    """Block-cyclic partition of M rows over `world` ranks in `chunks` rounds."""
    m: int
    world: int
    chunks: int

    def __post_init__(self):
        if self.m <= 0 or self.world <= 0 or self.chunks <= 0:
            raise ValueError("m, world and chunks must be positive")
        if self.m % (self.world * self.chunks) != 0:
            raise ValueError(f"M={self.m} is not divisible by world*chunks={self.world * self.chunks}")

    @property
    def block_rows(self) -> int:
        return self.m // (self.world * self.chunks)

    @property
    def rows_per_rank(self) -> int:
        return self.block_rows * self.chunks

    def block_of(self, rank: int, chunk: int) -> int:
        return chunk * self.world + rank

    def global_row_range(self, rank: int, chunk: int) -> Tuple[int, int]:
        b = self.block_of(rank, chunk)
        return b * self.block_rows, (b + 1) * self.block_rows

    def chunk_row_range(self, chunk: int) -> Tuple[int, int]:
        """Rows of the full C covered by chunk `chunk` over all ranks (contiguous)."""
        return chunk * self.world * self.block_rows, (chunk + 1) * self.world * self.block_rows

    def local_row_range(self, chunk: int) -> Tuple[int, int]:
        return chunk * self.block_rows, (chunk + 1) * self.block_rows

    def owner_of_row(self, row: int) -> Tuple[int, int]:
        """-> (rank, local row) of a global row."""
        b, off = divmod(row, self.block_rows)
        chunk, rank = divmod(b, self.world)
        return rank, chunk * self.block_rows + off

    @staticmethod
    def choose(m: int, world: int, max_chunks: int = 4, min_block_rows: int = 1024) -> "RowBlockPlan":
        """Largest chunk count <= max_chunks that divides M and keeps blocks of at least min_block_rows rows."""
        if m % world != 0:
            raise ValueError(f"M={m} is not divisible by the number of ranks {world}")
        best = 1
        for c in range(1, max_chunks + 1):
            if m % (world * c) == 0 and m // (world * c) >= min_block_rows:
                best = c
        if world == 1:
            best = 1
        return RowBlockPlan(m, world, best)


def shard_rows(a_full, plan: RowBlockPlan, rank: int):
    """Rows of a full [M, ...] array (numpy or torch) that `rank` owns, concatenated in chunk order."""
    parts = []
    for j in range(plan.chunks):
        r0, r1 = plan.global_row_range(rank, j)
        parts.append(a_full[r0:r1])
    if type(a_full).__module__.split(".")[0] == "torch":
        import torch
        return torch.cat(parts, dim=0)
    import numpy as np
    return np.concatenate(parts, axis=0)


class ShardedGemm:
    """C_full <- epi(A @ B) with A's rows sharded over the ranks of a process group.

    `gemm_fn(a_block, b, c_block)` computes one block in place; the default is
    the library's tcgen05 GEMM through the C ABI.  `all_gather_fn(out, inp)` is
    torch.distributed.all_gather_into_tensor on `group` unless given.
    """

    def __init__(self, plan: RowBlockPlan, rank: int, group=None, gemm_fn: Optional[Callable] = None,
                 overlap: bool = True):
        self.plan = plan
        self.rank = rank
        self.group = group
        self.overlap = overlap
        self._gemm_fn = gemm_fn
        self._comm_stream = None
        self._events: List = []

    def _default_gemm(self, a, b, c):
        from . import runtime
        runtime.gemm(a, b, c, beta=0.0, relu=True, compute="tensor_2sm")

    def run(self, a_local, b, c_full) -> None:
        """a_local: this rank's rows ([rows_per_rank, K], from shard_rows); c_full: [M, N] on every rank."""
        import torch
        import torch.distributed as dist
        plan = self.plan
        gemm = self._gemm_fn or self._default_gemm
        on_gpu = bool(getattr(c_full, "is_cuda", False))
        use_streams = on_gpu and self.overlap and plan.world > 1
        if use_streams and self._comm_stream is None:
            self._comm_stream = torch.cuda.Stream(device=c_full.device)
        works = []
        for j in range(plan.chunks):
            l0, l1 = plan.local_row_range(j)
            g0, g1 = plan.global_row_range(self.rank, j)
            gemm(a_local[l0:l1], b, c_full[g0:g1])
            if plan.world == 1:
                continue
            c0, c1 = plan.chunk_row_range(j)
            out = c_full[c0:c1]
            inp = c_full[g0:g1]
            if use_streams:
                done = torch.cuda.Event()
                done.record(torch.cuda.current_stream(c_full.device))
                self._comm_stream.wait_event(done)
                with torch.cuda.stream(self._comm_stream):
                    dist.all_gather_into_tensor(out, inp, group=self.group)
            else:
                w = dist.all_gather_into_tensor(out, inp, group=self.group, async_op=not on_gpu)
                if w is not None:
                    works.append(w)
        for w in works:
            w.wait()
        if use_streams:
            torch.cuda.current_stream(c_full.device).wait_stream(self._comm_stream)
