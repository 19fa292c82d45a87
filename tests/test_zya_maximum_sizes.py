"""The largest shapes the configuration rules admit (1024 experts, top-32) and the code paths
only large calls reach: the router and the permutation at 1024 experts x 32 slots, and a decode
call whose draw and work-entry lists exceed what the streaming kernels keep in shared memory
(more than 1024 draws, more than 384 entries), so they read them from global memory instead.

Collected late: first executed after the per-kernel parity tests."""
import numpy as np
import pytest

import aeon_b200
import gpu_support as gs
from aeon_b200 import synth

pytestmark = pytest.mark.gpu


def test_router_at_1024_experts_top_32(oracle):
    import torch
    cfg = aeon_b200.preset("baseline").copy(experts=1024, top_k=32)
    tokens = 5
    rng = np.random.default_rng(8)
    gate_bits = synth.normal_bits(rng, (cfg.experts, cfg.hidden), 0.01, cfg.act_dtype)
    x_bits = gs.activations(cfg, tokens, seed=3)
    ctx = aeon_b200.Context(cfg, max_tokens=tokens)
    w, ids = ctx.router_topk(gs.torch_bits(x_bits, cfg.act_dtype), gs.torch_bits(gate_bits, cfg.act_dtype))
    ctx.check()
    logits = oracle.router_logits_f32_ordered(gate_bits, cfg.act_dtype, x_bits, cfg.act_dtype)
    want_ids, want_w, _ = oracle.router_topk(logits.astype(np.float64), None, cfg.top_k, cfg.routed_scaling,
                                              cfg.score_fn)
    np.testing.assert_array_equal(ids.cpu().numpy(), want_ids)
    assert np.abs(w.cpu().numpy() - want_w).max() < 1e-5
    assert np.abs(w.cpu().numpy().sum(axis=1) - cfg.routed_scaling).max() < 1e-5


def test_permutation_at_1024_experts_32_slots():
    import torch
    cfg = aeon_b200.preset("baseline")
    tokens, slots, experts = 2048, 32, 1024
    rng = np.random.default_rng(9)
    ids = np.stack([rng.permutation(experts)[:slots] for _ in range(tokens)]).astype(np.int32)
    weights = rng.random((tokens, slots)).astype(np.float32)
    ctx = aeon_b200.Context(cfg, max_tokens=8)
    off, tok, drw, wpos = ctx.expert_permutation(torch.from_numpy(ids).cuda(), experts,
                                                 torch.from_numpy(weights).cuda())
    ctx.check()
    flat = ids.ravel()
    order = np.argsort(flat, kind="stable")
    np.testing.assert_array_equal(drw.cpu().numpy(), order)              # stable sort by expert
    np.testing.assert_array_equal(tok.cpu().numpy(), order // slots)
    np.testing.assert_array_equal(off.cpu().numpy(), np.concatenate([[0], np.cumsum(np.bincount(flat, minlength=experts))]))
    np.testing.assert_array_equal(wpos.cpu().numpy(), weights.ravel()[order])


def test_decode_with_draw_and_entry_lists_beyond_shared_memory(oracle):
    import torch
    cfg = aeon_b200.preset("baseline").copy(top_k=32)
    tokens = 128
    resident = list(range(96, 136))                     # 40 experts, every token draws 32 of them
    layer = gs.SyntheticLayer(cfg.copy(top_k=8), resident, seed=12, layer=1, with_shared=False)
    rng = np.random.default_rng(13)
    ids = np.stack([rng.permutation(resident)[:cfg.top_k] for _ in range(tokens)]).astype(np.int32)
    w = rng.random((tokens, cfg.top_k)).astype(np.float32)
    w /= w.sum(axis=1, keepdims=True)
    x_bits = gs.activations(cfg, tokens, seed=14)
    ctx = aeon_b200.Context(cfg, max_tokens=tokens)
    out = torch.zeros(tokens, cfg.hidden, dtype=torch.float32, device="cuda")
    ctx.moe_decode(layer.pool.base, layer.slot_of, gs.torch_bits(x_bits, cfg.act_dtype),
                   torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda(), out)
    ctx.check()
    distinct, entries = ctx.last_stats()
    assert distinct == len(resident) and entries > 384 and tokens * cfg.top_k > 1024
    again = torch.zeros_like(out)
    ctx.moe_decode(layer.pool.base, layer.slot_of, gs.torch_bits(x_bits, cfg.act_dtype),
                   torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda(), again)
    assert torch.equal(out, again)
    layer.cfg = cfg                                     # the oracle helper reads the slot count from the ids
    want = gs.oracle_routed(oracle, layer, x_bits, ids, w.astype(np.float64), [tokens - 1])
    gs.assert_close(oracle, want[tokens - 1], out[tokens - 1].double().cpu().numpy(), "top-32 token")
