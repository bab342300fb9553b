"""Host-side logic of the M-row sharded GEMM with 2 (and 4) gloo ranks on CPU.

The per-block GEMM is injected (the CPU oracle stands in for the CUDA kernel, which cannot run here), so what
is under test is the product's partition arithmetic, the in-place block placement and the all-gather."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from accera_b200.sharded import RowBlockPlan, ShardedGemm, shard_rows  # noqa: E402


def test_row_block_plan_partition_is_a_bijection():
    plan = RowBlockPlan(m=96, world=4, chunks=3)
    assert plan.block_rows == 8 and plan.rows_per_rank == 24
    seen = np.full(96, -1)
    for r in range(4):
        for j in range(3):
            g0, g1 = plan.global_row_range(r, j)
            assert (seen[g0:g1] == -1).all()
            seen[g0:g1] = r
            c0, c1 = plan.chunk_row_range(j)
            assert c0 <= g0 and g1 <= c1 and (g0 - c0) == r * plan.block_rows     # rank r's slot inside the chunk
    assert (seen >= 0).all()
    for row in (0, 7, 8, 40, 95):
        rank, local = plan.owner_of_row(row)
        a = np.arange(96)
        assert shard_rows(a, plan, rank)[local] == row
    with pytest.raises(ValueError):
        RowBlockPlan(m=100, world=4, chunks=3)
    assert RowBlockPlan.choose(65536, 8, max_chunks=4).chunks == 4
    assert RowBlockPlan.choose(65536, 1, max_chunks=4).chunks == 1
    assert RowBlockPlan.choose(4096, 8, max_chunks=4, min_block_rows=256).chunks == 2
    with pytest.raises(ValueError):
        RowBlockPlan.choose(1001, 8)


def _worker(rank, world, port, chunks, tmpdir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle
        m, n, k = 16 * world * chunks, 24, 40
        rng = np.random.default_rng(99)
        a_full = rng.standard_normal((m, k)).astype(np.float32)
        b = np.asfortranarray(rng.standard_normal((k, n)).astype(np.float32))
        want = oracle.gemm(a_full, b, np.zeros((m, n), np.float32), relu=True)
        plan = RowBlockPlan(m, world, chunks)

        def gemm_fn(a_blk, b_t, c_blk):                   # the oracle stands in for the kernel on CPU
            c = c_blk.numpy()
            c[...] = 0
            oracle.gemm(np.ascontiguousarray(a_blk.numpy()), b, c, relu=True)

        a_local = torch.from_numpy(shard_rows(a_full, plan, rank))
        c_full = torch.full((m, n), float("nan"))
        ShardedGemm(plan, rank, gemm_fn=gemm_fn).run(a_local, torch.from_numpy(np.ascontiguousarray(b)), c_full)
        ok = np.array_equal(c_full.numpy(), want)
        with open(os.path.join(tmpdir, f"r{rank}.txt"), "w") as f:
            f.write("ok" if ok else "bad")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,chunks", [(2, 1), (2, 3), (4, 2)])
def test_sharded_gemm_gloo(tmp_path, world, chunks):
    port = 29600 + world * 10 + chunks
    mp.spawn(_worker, args=(world, port, chunks, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert (tmp_path / f"r{r}.txt").read_text() == "ok"


def _mismatch_worker(rank, world, port, tmpdir, what):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    from accera_b200.sharded import ShardMismatchError, rendezvous
    rendezvous("gloo", rank, world, timeout_s=60)
    try:
        m, n, k = 64, 24, 40
        plan = RowBlockPlan(m, world, 2)
        rows = plan.rows_per_rank
        kk = k
        if what == "rows" and rank == 1:
            rows += 16                      # rank 1 brings a shard of another size
        if what == "k" and rank == 1:
            kk = k + 8                      # rank 1 was built for another K
        a_local = torch.zeros(rows, kk)
        b = torch.zeros(kk, n)
        c_full = torch.zeros(m, n)
        calls = []
        sg = ShardedGemm(plan, rank, gemm_fn=lambda a, bb, c: calls.append(1))
        try:
            sg.run(a_local, b, c_full)
            outcome = "no error"
        except ShardMismatchError as exc:
            outcome = f"caught calls={len(calls)} names_rank1={'rank 1' in str(exc)}"
        with open(os.path.join(tmpdir, f"r{rank}.txt"), "w") as f:
            f.write(outcome)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("what", ["rows", "k"])
def test_shard_mismatch_is_caught_on_every_rank_before_any_work(tmp_path, what):
    # one rank disagrees about the problem: every rank (also the ones whose own shard is fine) raises before a
    # GEMM is launched or a collective on C is entered
    world = 2
    mp.spawn(_mismatch_worker, args=(world, 29650 + (what == "k"), str(tmp_path), what), nprocs=world, join=True)
    for r in range(world):
        assert (tmp_path / f"r{r}.txt").read_text() == "caught calls=0 names_rank1=True"


def _late_worker(rank, world, port, tmpdir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import time
    from accera_b200.sharded import RankJoinTimeout, rendezvous
    if rank == world - 1:
        return                              # this rank dies before it joins
    t0 = time.time()
    try:
        rendezvous("gloo", rank, world, timeout_s=4)
        outcome = "joined"
    except RankJoinTimeout:
        outcome = "timeout"
    with open(os.path.join(tmpdir, f"r{rank}.txt"), "w") as f:
        f.write(f"{outcome} {time.time() - t0 < 60}")


def test_a_rank_that_never_joins_ends_the_others_with_a_timeout(tmp_path):
    world = 3
    mp.spawn(_late_worker, args=(world, 29670, str(tmp_path)), nprocs=world, join=True)
    for r in range(world - 1):
        assert (tmp_path / f"r{r}.txt").read_text() == "timeout True"


def _barrier_worker(rank, world, port, tmpdir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import time
    from accera_b200.sharded import RankJoinTimeout, checked_barrier, rendezvous
    rendezvous("gloo", rank, world, timeout_s=60)
    checked_barrier(timeout_s=30)           # everyone is here: passes
    outcome = "passed"
    if rank == 1:
        time.sleep(6)                       # rank 1 leaves between steps (nothing of it in flight) ...
    else:
        try:
            checked_barrier(timeout_s=2)    # ... and the others learn of it on the host
        except RankJoinTimeout as exc:
            outcome = "timeout"
    with open(os.path.join(tmpdir, f"r{rank}.txt"), "w") as f:
        f.write(outcome)
    os._exit(0)                             # the group is broken: leave without the collective shutdown


def test_checked_barrier_reports_a_rank_that_left(tmp_path):
    world = 2
    mp.spawn(_barrier_worker, args=(world, 29680, str(tmp_path)), nprocs=world, join=True)
    assert (tmp_path / "r0.txt").read_text() == "timeout"
    assert (tmp_path / "r1.txt").read_text() == "passed"
