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

Two ways to move the blocks, chosen with `gather=`:

  "nccl"         one in-place ncclAllGather per chunk (the block-cyclic layout makes the `world`
                 blocks of a chunk adjacent in C).  NCCL's kernels need SMs of their own; the
                 tensor-core GEMM holds almost all shared memory of every SM it runs on, so the
                 caller should leave a few SMs free (accb_gemm_desc.max_ctas).
  "copy_engine"  C lives in symmetric memory (torch.distributed._symmetric_memory); as soon as a
                 block is computed its owner pushes it into every peer's C with plain
                 device-to-device copies, one stream per peer.  The DMA engines do the work over
                 NVLink, no SM is taken from the GEMM, and one barrier at the end of the step
                 tells every rank that all blocks have landed.

  "fused"        C lives in symmetric memory and the GEMM kernel itself stores every output tile to
                 all replicas of C (accb_gemm_replicated): TMA stores from the epilogue's shared-memory
                 staging go to the local C and, over NVLink, to each peer's C, so the transfer overlaps
                 the math tile by tile.  One barrier at the end of the step.

                 With three or more peers the kernel sets a few CTAs aside that do nothing but forward
                 finished tiles (stores that wait for NVLink would otherwise hold up the operand fetches
                 of the SM that issued them); with one or two peers the epilogue stores to them directly.

The kernels never load from another GPU's memory and use no TMA multicast; "fused" only stores to it.

Ordering between steps.  "copy_engine" and "fused" write straight into the peers' C.  A rank must not start
writing step n+1 into a peer's C while that peer still reads step n's result, so both modes open a step
with a barrier (every rank's consumers of the previous C were enqueued before it reaches that barrier) and
close it with one (all tiles of this step have landed everywhere).  "nccl" needs neither: the collective
itself waits for every rank.

Failures are detected on the host: `rendezvous` bounds the time a rank waits for the others to join, and
`ShardedGemm.run` compares the shard geometry of all ranks before its first collective.
"""
from __future__ import annotations

import dataclasses
import datetime
from typing import Callable, List, Optional, Tuple


class ShardMismatchError(RuntimeError):
    """The ranks of a sharded GEMM do not agree on the problem (raised on every rank, before any collective)."""


class RankJoinTimeout(RuntimeError):
    """A rank did not join the process group, or a barrier, within the time allowed."""


def rendezvous(backend: str, rank: int, world: int, timeout_s: float = 600.0, init_method: Optional[str] = None,
               device_id=None):
    """torch.distributed.init_process_group with a bound on how long this rank waits for the others.

    A rank that never starts (crashed before joining, wrong world size) makes every other rank raise
    RankJoinTimeout after `timeout_s` instead of waiting forever.  MASTER_ADDR / MASTER_PORT come from the
    environment unless `init_method` is given.
    """
    import torch.distributed as dist
    kwargs = dict(backend=backend, rank=rank, world_size=world, timeout=datetime.timedelta(seconds=float(timeout_s)))
    if init_method is not None:
        kwargs["init_method"] = init_method
    if device_id is not None:
        kwargs["device_id"] = device_id
    try:
        dist.init_process_group(**kwargs)
    except Exception as exc:      # torch raises DistStoreError / DistNetworkError / RuntimeError depending on where it gave up
        raise RankJoinTimeout(f"rank {rank} of {world}: the process group did not form within {timeout_s:g} s ({exc})") from exc
    return dist.group.WORLD


def checked_barrier(group=None, timeout_s: float = 60.0) -> None:
    """A host-side barrier that names the ranks that did not arrive within `timeout_s` (gloo groups;
    other backends fall back to their own barrier and the group's timeout)."""
    import torch.distributed as dist
    try:
        if dist.get_backend(group) == "gloo":
            dist.monitored_barrier(group=group, timeout=datetime.timedelta(seconds=float(timeout_s)), wait_all_ranks=True)
        else:
            dist.barrier(group=group)
    except Exception as exc:
        raise RankJoinTimeout(f"barrier: not every rank arrived within {timeout_s:g} s ({exc})") from exc


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
                 overlap: bool = True, gather: str = "nccl", gemm_kwargs: Optional[dict] = None):
        if gather not in ("nccl", "copy_engine", "fused"):
            raise ValueError("gather must be 'nccl', 'copy_engine' or 'fused'")
        self.gemm_kwargs = dict(gemm_kwargs) if gemm_kwargs is not None else dict(beta=0.0, relu=True, compute="tensor_2sm")
        self.plan = plan
        self.rank = rank
        self.group = group
        self.overlap = overlap
        self.gather = gather
        self._gemm_fn = gemm_fn
        self._comm_stream = None
        self._events: List = []
        self._symm = None          # symmetric-memory handle of C (copy_engine)
        self._peer_c: List = []
        self._peer_streams: List = []
        self._validated = None     # signature of the operands the ranks last agreed on

    def validate(self, a_local, b, c_full) -> None:
        """Compares the shard geometry of all ranks on the host (one all_gather_object) and raises
        ShardMismatchError on EVERY rank when they differ: a rank with a shard of another size, another K, N
        or element type would otherwise make the all-gather write past its blocks, or hang it."""
        sig = (tuple(a_local.shape), tuple(b.shape), tuple(c_full.shape), str(a_local.dtype), str(c_full.dtype),
               self.plan.m, self.plan.world, self.plan.chunks)
        if sig == self._validated:
            return
        plan = self.plan
        problems = []
        if tuple(a_local.shape)[0] != plan.rows_per_rank:
            problems.append(f"A shard has {tuple(a_local.shape)[0]} rows, the plan gives every rank {plan.rows_per_rank}")
        if tuple(c_full.shape)[0] != plan.m:
            problems.append(f"C has {tuple(c_full.shape)[0]} rows, the plan says {plan.m}")
        if len(a_local.shape) != 2 or len(b.shape) != 2 or a_local.shape[1] != b.shape[0] or b.shape[1] != c_full.shape[1]:
            problems.append(f"inner dimensions disagree: A{tuple(a_local.shape)} B{tuple(b.shape)} C{tuple(c_full.shape)}")
        mine = {"rank": self.rank, "sig": sig, "problems": problems}
        if plan.world > 1:
            import torch.distributed as dist
            everyone = [None] * plan.world
            dist.all_gather_object(everyone, mine, group=self.group)
        else:
            everyone = [mine]
        bad = [e for e in everyone if e["problems"]]
        differing = [e["rank"] for e in everyone if e["sig"] != everyone[0]["sig"]]
        if bad or differing:
            lines = [f"rank {e['rank']}: {'; '.join(e['problems'])}" for e in bad]
            if differing:
                lines.append(f"ranks {differing} describe another problem than rank {everyone[0]['rank']}: "
                             + ", ".join(f"rank {e['rank']} {e['sig'][:5]}" for e in everyone))
            raise ShardMismatchError("sharded GEMM: the ranks do not agree - " + " | ".join(lines))
        self._validated = sig

    @staticmethod
    def allocate_c(m: int, n: int, dtype, device, group=None, gather: str = "nccl"):
        """Allocates the full C for this rank: ordinary device memory for "nccl", symmetric memory (mapped
        into every peer's address space) for "copy_engine"."""
        import torch
        if gather in ("copy_engine", "fused"):
            import torch.distributed as dist
            import torch.distributed._symmetric_memory as symm_mem
            c = symm_mem.empty((m, n), dtype=dtype, device=device)
            c.zero_()
            return c
        return torch.zeros(m, n, dtype=dtype, device=device)

    def _setup_copy_engine(self, c_full) -> None:
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        group = self.group if self.group is not None else dist.group.WORLD
        self._symm = symm_mem.rendezvous(c_full, group)
        if self._symm is None:
            raise RuntimeError("copy_engine gather needs C allocated with ShardedGemm.allocate_c(..., gather='copy_engine')")
        self._peer_c = [self._symm.get_buffer(r, tuple(c_full.shape), c_full.dtype) for r in range(self.plan.world)]
        self._peer_streams = [torch.cuda.Stream(device=c_full.device) for _ in range(self.plan.world)]

    def _default_gemm(self, a, b, c):
        from . import runtime
        runtime.gemm(a, b, c, **self.gemm_kwargs)

    def run(self, a_local, b, c_full) -> None:
        """a_local: this rank's rows ([rows_per_rank, K], from shard_rows); c_full: [M, N] on every rank."""
        import torch
        import torch.distributed as dist
        plan = self.plan
        self.validate(a_local, b, c_full)
        gemm = self._gemm_fn or self._default_gemm
        on_gpu = bool(getattr(c_full, "is_cuda", False))
        if self.gather == "copy_engine" and plan.world > 1:
            return self._run_copy_engine(a_local, b, c_full, gemm)
        if self.gather == "fused" and plan.world > 1:
            return self._run_fused(a_local, b, c_full)
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

    def _run_copy_engine(self, a_local, b, c_full, gemm) -> None:
        import torch
        plan = self.plan
        if self._symm is None:
            self._setup_copy_engine(c_full)
        main = torch.cuda.current_stream(c_full.device)
        # no peer may still be reading the previous step's C when my pushes start to overwrite it
        self._symm.barrier()
        for j in range(plan.chunks):
            l0, l1 = plan.local_row_range(j)
            g0, g1 = plan.global_row_range(self.rank, j)
            gemm(a_local[l0:l1], b, c_full[g0:g1])
            done = torch.cuda.Event()
            done.record(main)
            src = c_full[g0:g1]
            for step in range(1, plan.world):
                peer = (self.rank + step) % plan.world          # every rank starts with a different peer
                st = self._peer_streams[peer]
                st.wait_event(done)
                with torch.cuda.stream(st):
                    self._peer_c[peer][g0:g1].copy_(src, non_blocking=True)
        for step in range(1, plan.world):
            main.wait_stream(self._peer_streams[(self.rank + step) % plan.world])
        # all my pushes are ordered before the barrier on `main`; after it every peer's pushes have landed here
        self._symm.barrier()

    def _run_fused(self, a_local, b, c_full) -> None:
        from . import runtime
        plan = self.plan
        if self._symm is None:
            self._setup_copy_engine(c_full)
        kw = {k: v for k, v in self.gemm_kwargs.items() if k in ("alpha", "beta", "relu", "compute", "max_ctas", "bias")}
        # no peer may still be reading the previous step's C when my kernel starts to overwrite its blocks there
        self._symm.barrier()
        for j in range(plan.chunks):
            l0, l1 = plan.local_row_range(j)
            g0, g1 = plan.global_row_range(self.rank, j)
            # replica 0 is the local C (read when beta != 0); the others are the peers' C, each rank starting
            # with a different peer so that the NVLink traffic of a step is spread over all destinations
            replicas = [c_full[g0:g1]] + [self._peer_c[(self.rank + s) % plan.world][g0:g1] for s in range(1, plan.world)]
            runtime.gemm_replicated(a_local[l0:l1], b, replicas, **kw)
        # the stores of my launches are ordered before the barrier on this stream; after it all peers' tiles are here
        self._symm.barrier()

