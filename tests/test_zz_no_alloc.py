"""The allocation-free router entry point against the context-based one.

aeon_b200_router_topk_noalloc exists for callers that cannot call cudaMalloc where they
need the router (under a fixed memory budget, inside a host that forbids allocation after
start-up): it takes no context and keeps its logits scratch in an
array built into the library. Both entry points run the same kernels, so ids and weights
must be identical. Two calls in a row are made because all calls share the one scratch,
which still holds the previous call's logits when the next call starts.
"""
import numpy as np
import pytest

import aeon_b200
from aeon_b200 import synth
import gpu_support as gs

pytestmark = pytest.mark.gpu


def test_noalloc_router_matches_context_router_twice():
    import torch
    cfg = aeon_b200.preset("baseline")
    rng = np.random.default_rng(123)
    gate_bits = synth.normal_bits(rng, (cfg.experts, cfg.hidden), 0.01, cfg.act_dtype)
    gate = gs.torch_bits(gate_bits, cfg.act_dtype)
    ctx = aeon_b200.Context(cfg, max_tokens=64)
    # every buffer is made before the calls under test; the calls themselves allocate nothing
    w_new = torch.empty(64, cfg.top_k, dtype=torch.float32, device="cuda")
    ids_new = torch.empty(64, cfg.top_k, dtype=torch.int32, device="cuda")
    for call, tokens in enumerate((64, 5)):          # second call: fewer tokens, stale scratch
        x = gs.torch_bits(gs.activations(cfg, tokens, seed=40 + call), cfg.act_dtype)
        w_ref, ids_ref = ctx.router_topk(x, gate)
        w_new.fill_(-1.0)
        ids_new.fill_(-1)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        aeon_b200.router_topk_noalloc(cfg, x, gate, w_new[:tokens], ids_new[:tokens])
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert torch.equal(ids_new[:tokens], ids_ref)
        assert torch.equal(w_new[:tokens], w_ref)    # same kernels, same order: bit-identical
        assert (ids_new[tokens:] == -1).all()        # nothing written past the request
    ctx.check()


def test_noalloc_router_rejects_sizes_beyond_its_scratch():
    import torch
    cfg = aeon_b200.preset("baseline")
    gate = torch.zeros(cfg.experts, cfg.hidden, dtype=torch.bfloat16, device="cuda")
    x = torch.zeros(65, cfg.hidden, dtype=torch.bfloat16, device="cuda")
    w = torch.empty(65, cfg.top_k, dtype=torch.float32, device="cuda")
    ids = torch.empty(65, cfg.top_k, dtype=torch.int32, device="cuda")
    with pytest.raises(aeon_b200.AeonError) as e:
        aeon_b200.router_topk_noalloc(cfg, x, gate, w, ids)
    assert e.value.status == 1 and "64 tokens" in str(e.value)
