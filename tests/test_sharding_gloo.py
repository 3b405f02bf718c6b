"""World-size-2 checks of the multi-GPU host logic on CPU (gloo): KV-head
partition, output all-gather, max-over-ranks timing and the log-sum-exp merge."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT, load_pkg


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        sh = load_pkg("sharding")
        hq, hkv, d, b = 32, 8, 16, 3
        shard = sh.kv_head_shard(hq, hkv, world, rank)
        gen = torch.Generator().manual_seed(0)
        full = torch.randn(b, hq, d, generator=gen)                 # same on every rank
        local = full[:, shard.q_lo:shard.q_hi]
        got = sh.gather_head_outputs(local)
        ok = torch.equal(got, full)
        slow = sh.max_over_ranks(1.0 + rank, "cpu")
        q.put((rank, ok, slow, (shard.kv_lo, shard.kv_hi, shard.q_lo, shard.q_hi)))
    finally:
        dist.destroy_process_group()


def test_kv_head_partition_and_output_gather_world2():
    world, port = 2, 29000 + os.getpid() % 2000
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert [r[1] for r in res] == [True, True]
    assert [r[2] for r in res] == [2.0, 2.0]                       # the slowest rank's time everywhere
    assert res[0][3] == (0, 4, 0, 16) and res[1][3] == (4, 8, 16, 32)


def test_partition_helpers_reject_uneven_splits():
    sh = load_pkg("sharding")
    with pytest.raises(ValueError):
        sh.kv_head_shard(32, 8, 3, 0)
    with pytest.raises(ValueError):
        sh.kv_head_shard(30, 8, 2, 0)
    assert sh.request_shard(7, 2, 1) == [1, 3, 5]
    covered = sorted(sum((sh.request_shard(7, 3, r) for r in range(3)), []))
    assert covered == list(range(7))


def test_lse_merge_of_disjoint_token_sets_equals_full_attention():
    sh = load_pkg("sharding")
    g = torch.Generator().manual_seed(1)
    n, d, heads = 300, 32, 4
    q = torch.randn(heads, d, generator=g, dtype=torch.float64)
    k = torch.randn(n, d, generator=g, dtype=torch.float64)
    v = torch.randn(n, d, generator=g, dtype=torch.float64)
    log2e = 1.4426950408889634
    s = (q @ k.T) * d ** -0.5 * log2e                      # exp2 domain, as the kernels keep it
    full = torch.softmax(s / log2e, dim=-1) @ v
    parts = [torch.arange(0, n, 3), torch.arange(1, n, 3), torch.arange(2, n, 3), torch.arange(0, 0)]
    outs, ms, zs = [], [], []
    for idx in parts:
        if len(idx) == 0:
            outs.append(torch.zeros(heads, d)); ms.append(torch.full((heads,), float("-inf"))); zs.append(torch.zeros(heads))
            continue
        sp = s[:, idx]
        m = sp.max(dim=-1).values
        p = torch.exp2(sp - m[:, None])
        z = p.sum(-1)
        outs.append(((p @ v[idx]) / z[:, None]).float()); ms.append(m.float()); zs.append(z.float())
    merged = sh.lse_merge(torch.stack(outs), torch.stack(ms), torch.stack(zs))
    np.testing.assert_allclose(merged.numpy(), full.float().numpy(), rtol=2e-5, atol=2e-5)


def _combine_worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        sh = load_pkg("sharding")
        gen = torch.Generator().manual_seed(5)
        full = torch.randint(1, 65536, (4, 1000), generator=gen).to(torch.int32)     # the single-GPU score rows
        pages = torch.arange(1000)
        mine = torch.where(pages % world == rank, full, torch.zeros_like(full))      # this rank scored its pages only
        as_u16 = mine.to(torch.int16)                                                # same bits as uint16 (wraps)
        got = sh.combine_disjoint_scores(as_u16)
        q.put((rank, torch.equal(got, full.to(torch.int16)), got.dtype == torch.int16, tuple(got.shape)))
    finally:
        dist.destroy_process_group()


def test_score_rows_of_disjoint_owners_combine_to_the_full_row_world2():
    """Sequence sharding: every page is scored by one rank (0 elsewhere); the all-gather + OR of
    the ranks' rows is the full row on every rank."""
    world, port = 2, 31000 + os.getpid() % 2000
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_combine_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(r[1] and r[2] and r[3] == (4, 1000) for r in res)


def _agree_worker(rank, world, port, q):
    import torch
    import torch.distributed as dist
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import bench
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        q.put((rank, bench.agree_max(torch, 140 + 3 * rank)))
    finally:
        dist.destroy_process_group()


def test_ranks_agree_on_the_replay_count_world2():
    """A CUDA graph that holds collectives must be replayed equally often on every rank; the count each
    rank derives from its own timing is replaced by the largest."""
    import multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29650 + os.getpid() % 200
    procs = [ctx.Process(target=_agree_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert got == {0: 143, 1: 143}
