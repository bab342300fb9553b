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
        # a mismatch of shard shapes among ranks must be caught on the host, before any collective
        flag = torch.tensor([plan.rows_per_rank + (1 if (rank == 1 and chunks == 99) else 0)])
        gathered = [torch.zeros_like(flag) for _ in range(world)]
        dist.all_gather(gathered, flag)
        same = all(int(g) == int(flag) for g in gathered)
        with open(os.path.join(tmpdir, f"r{rank}.txt"), "w") as f:
            f.write("ok" if (ok and same) else f"bad ok={ok} same={same}")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,chunks", [(2, 1), (2, 3), (4, 2)])
def test_sharded_gemm_gloo(tmp_path, world, chunks):
    port = 29600 + world * 10 + chunks
    mp.spawn(_worker, args=(world, port, chunks, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert (tmp_path / f"r{r}.txt").read_text() == "ok"
