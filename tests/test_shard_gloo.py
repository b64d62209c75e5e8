"""Host-side sharding logic, single-process properties and a world_size-2 gloo run on CPU."""
import os
import socket

import numpy as np
import pytest

import blaze_oracle as o
from ops_tensor_b200 import shard


def test_n_shard_covers_and_aligns():
    for N, world in ((8192, 8), (14336, 8), (7168, 8), (7168, 4), (1000, 3), (128, 8), (65536, 8)):
        edges = [shard.n_shard(N, world, r) for r in range(world)]
        assert edges[0][0] == 0 and edges[-1][1] == N
        for (a0, a1), (b0, b1) in zip(edges, edges[1:]):
            assert a1 == b0
        for n0, n1 in edges:
            assert n0 % 128 == 0 and (n1 % 128 == 0 or n1 == N)
        widths = [n1 - n0 for n0, n1 in edges]
        assert max(widths) - min(widths) < 256          # one block, plus the ragged last block
    with pytest.raises(ValueError):
        shard.n_shard(128, 2, 2)


def test_expert_plan_balances_and_covers():
    rows = o.moe_group_rows()
    for world in (1, 2, 4, 8):
        plan = shard.plan_experts(rows, world)
        covered = np.zeros(len(rows), dtype=np.int64)
        for lst in plan:
            for p in lst:
                assert 0 <= p.row_begin < p.row_end <= rows[p.expert]
                covered[p.expert] += p.rows
        assert np.array_equal(covered, rows)
        loads = shard.plan_loads(plan)
        assert sum(loads) == rows.sum()
        # the benchmark target is >= 85 % scaling efficiency: the heaviest rank stays within 1/0.85 of the mean
        assert max(loads) <= rows.sum() / world / 0.85 + 128
    # without splitting, one oversized expert would dominate a rank
    big = np.array([9000, 100, 100, 100], dtype=np.int64)
    assert max(shard.plan_loads(shard.plan_experts(big, 4, allow_split=False))) == 9000
    assert max(shard.plan_loads(shard.plan_experts(big, 4))) < 3000


def test_column_chunks_cover_whole_blocks():
    for width, chunks in ((8192, 4), (896, 4), (1000, 3), (100, 4), (128, 1), (7168, 7)):
        ranges = shard.column_chunks(width, chunks)
        assert ranges[0][0] == 0 and ranges[-1][1] == width and len(ranges) <= chunks
        for (a0, a1), (b0, b1) in zip(ranges, ranges[1:]):
            assert a1 == b0 and a0 % 128 == 0 and a1 % 128 == 0 and a1 > a0
    with pytest.raises(ValueError):
        shard.column_chunks(0, 2)


def test_overlapped_gather_single_rank_is_a_plain_chunked_gemm():
    import torch
    rng = np.random.default_rng(3)
    a = rng.standard_normal((8, 16)).astype(np.float32)
    b = rng.standard_normal((300, 16)).astype(np.float32)
    out = shard.gemm_gather_overlapped(lambda c0, c1, o_: o_.copy_(torch.from_numpy(a @ b[c0:c1].T)), 8, 300, 1,
                                       chunks=3, dtype=torch.float32)
    assert np.array_equal(out.numpy(), a @ b.T)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, fail_rank, results):
    import datetime
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    try:
        # N-sharded GEMM on de-quantised operands: every rank computes its columns, the gather restores the whole
        rng = np.random.default_rng(0)
        a = rng.standard_normal((32, 256)).astype(np.float32)
        w = (rng.standard_normal((512, 256)) * 0.02).astype(np.float32)
        qa, sa = o.quant_fp8_1x128(a)
        qb, sb = o.quant_fp8_128x128(w)
        da = o.dequant_fp8_1x128(qa, sa)
        db = o.dequant_fp8_128x128(qb, sb)
        n0, n1 = shard.n_shard(512, world, rank)
        local = torch.from_numpy(da @ db[n0:n1].T)
        whole = shard.gather_columns(local, world)
        ok_gemm = np.array_equal(whole.numpy(), da @ db.T)
        # the same product with the shard computed in column chunks, each gathered while the next one computes
        calls = []

        def run_chunk(c0, c1, out):
            calls.append((c0, c1))
            out.copy_(torch.from_numpy(da @ db[n0 + c0:n0 + c1].T))

        whole2 = shard.gemm_gather_overlapped(run_chunk, 32, n1 - n0, world, chunks=2, dtype=local.dtype)
        chunked = np.concatenate([da @ db[c:c + 128].T for c in range(0, 512, 128)], axis=1)   # same BLAS calls
        ok_gemm = ok_gemm and np.array_equal(whole2.numpy(), chunked) and calls == [(0, 128), (128, 256)]
        # grouped: every rank derives the same plan; its pieces, summed over ranks, cover every token once
        rows = o.moe_group_rows()
        plan = shard.plan_experts(rows, world)
        mine = torch.zeros(len(rows), dtype=torch.int64)
        for p in plan[rank]:
            mine[p.expert] += p.rows
        dist.all_reduce(mine)
        ok_plan = np.array_equal(mine.numpy(), rows)
        slowest = shard.max_over_ranks(1.0 + rank)
        results[rank] = (ok_gemm, ok_plan, slowest)
        # failure detection on the host: a rank that never joins makes the monitored barrier raise on rank 0
        if fail_rank is not None:
            if rank == fail_rank:
                return
            try:
                dist.monitored_barrier(timeout=datetime.timedelta(seconds=2))
                results[rank] = results[rank] + ("no-error",)
            except RuntimeError:
                results[rank] = results[rank] + ("peer-missing",)
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


@pytest.mark.parametrize("fail_rank", [None, 1])
def test_world_size_two_on_gloo(fail_rank):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    manager = ctx.Manager()
    results = manager.dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, fail_rank, results)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    for r in range(2):
        ok_gemm, ok_plan, slowest = results[r][:3]
        assert ok_gemm and ok_plan and slowest == 2.0
    if fail_rank is not None:
        assert results[0][3] == "peer-missing"
