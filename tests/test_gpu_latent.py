"""The shared-latent shape of the MLA configuration: 16 query heads on one KV head whose 576-dim row
(512 compressed dims + 64 rotary dims) is key and, in its first 512 dims, value; 64-token pages; the
scoring subspace is the 16 lowest-frequency dims of each half of the rotary part.  Selector integers
identical to the CPU oracle, attention (its own kernel: Q fragments in shared memory, output columns
split over the warps, token rows staged once by bulk copies) within the bf16 tolerance."""
import pytest
import torch

from test_gpu_parity import _check_against_oracle, _run_decode_step, _run_step

pytestmark = pytest.mark.gpu

LATENT = dict(page=64, hq=16, hkv=1, d=576, dv=512, shared_latent=True)


def test_batch_of_latent_requests_matches_oracle():
    from helpers import make_setup
    setup = make_setup([9000, 20000, 700, 3000, 131, 64, 40000, 5], seed=71, **LATENT)
    assert setup.cache.layers[0].kv_pool_v.data_ptr() == setup.cache.layers[0].kv_pool_k.data_ptr()
    out = _run_step(setup)
    assert out.shape == (8, 16, 512)
    _check_against_oracle(setup, out)


@pytest.mark.parametrize("length", [30000, 131072])
def test_single_latent_request_through_the_decode_step(length):
    from helpers import make_setup
    setup = make_setup([length], seed=73, **LATENT)
    out, launches = _run_decode_step(setup)
    assert launches in (2, 3)          # the selection may run as one launch; the latent attention is its own
    _check_against_oracle(setup, out)


def test_latent_attention_partials_merge_like_the_general_kernel():
    """(out, max, sum) of two disjoint halves of the list merge to the attention over the whole list."""
    from helpers import make_setup, mod
    ops = mod("sparse_attn.ops.paged_region_kernels")
    sharding = mod("sharding")
    setup = make_setup([12000, 900], seed=75, **LATENT)
    full = _run_step(setup)
    cache = setup.cache
    layer, gather, lens = cache.layers[0], cache.gather_indices_for_layer(0), cache.visible_lens_for_layer(0)
    col = torch.arange(gather.shape[-1], device=setup.dev)
    valid = col < lens[..., None]
    outs, ms, zs = [], [], []
    for owner in range(2):
        part = torch.where(valid & ((col % 2) == owner), gather, torch.full_like(gather, -1))
        o, lse = ops.sparse_paged_attention_gather(layer, setup.q, part, lens, cache.query_to_req_buf,
                                                   scale=setup.attention.scaling, return_lse=True)
        outs.append(o.float()); ms.append(lse[..., 0]); zs.append(lse[..., 1])
    merged = sharding.lse_merge(torch.stack(outs), torch.stack(ms), torch.stack(zs))
    torch.testing.assert_close(merged, full.float(), atol=2e-2, rtol=2e-2)
