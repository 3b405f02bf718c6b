"""Two-GPU test of the sequence-sharded decode step over NCCL (skipped on a single GPU):
every rank builds the same seeded request, owns the logical pages p % world == rank, and the
staged selector with all-gathers between the stages must reproduce the single-GPU token
lists and attention."""
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, result):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import torch.distributed as dist
    from helpers import make_setup, mod
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(f"cuda:{rank}"))
    try:
        sharding = mod("sharding")
        sel_mod = mod("sparse_attn.indexer.nfa_layer_batch_selector")
        nfa = mod("sparse_attn.ops.paged_region_kernels_nfa")
        setup = make_setup([30000], seed=21, device=f"cuda:{rank}")
        cache = setup.cache
        cache.plan_common(setup.req_ids)
        slots = cache.slot_mapping_for_layer(0)[:1]
        sel_mod.select_topk_for_layer_batched(cache, 0, setup.req_ids, setup.q, attention=setup.attention,
                                              decode_write=(setup.k_new, setup.v_new, slots))
        ref_out = nfa.decode_graph_ready(setup.attention, setup.q, cache).float()
        ref_gather = cache.gather_indices_for_layer(0).clone()
        ref_lens = cache.visible_lens_for_layer(0).clone()
        shard = sharding.SequenceShard(cache, setup.indexer, rank, world)
        for _ in range(2):          # twice: the second pass reuses every buffer
            merged, gather, lens = sharding.sequence_sharded_decode_step(shard, 0, setup.req_ids, setup.q,
                                                                         setup.attention)
        torch.cuda.synchronize()
        assert cache.read_status() == 0
        assert torch.equal(lens[:1], ref_lens[:1])
        n = int(ref_lens[:1].max())
        mine = gather[:1, :, :n]
        owned = mine >= 0
        assert torch.equal(mine[owned], ref_gather[:1, :, :n][owned])
        counts = owned.int()
        dist.all_reduce(counts)
        valid = torch.arange(n, device=mine.device)[None, None, :] < ref_lens[:1, :, None]
        assert bool((counts == 1)[valid].all())               # every selected token on exactly one rank
        torch.testing.assert_close(merged, ref_out, atol=2e-2, rtol=2e-2)
        result[rank] = 1
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sequence_sharded_decode_over_nccl_matches_single_gpu():
    import torch.multiprocessing as mp
    world = 2
    ctx = mp.get_context("spawn")
    result = ctx.Manager().dict()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, world, port, result)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=600)
    for p in procs:
        if p.is_alive():
            p.terminate()
            pytest.fail("a rank did not finish")
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert sorted(result.keys()) == list(range(world))
