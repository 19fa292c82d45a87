"""A whole MoE layer on the device — router, shared expert as the accumulator's initial
value, routed experts — against the oracle composition (benchmark configuration 0: one
token, 256 experts, top-8 plus the shared expert, seed 0)."""
import numpy as np
import pytest

import aeon_b200
from aeon_b200 import synth
import gpu_support as gs

pytestmark = pytest.mark.gpu


def run_layer(cfg, layer, x_bits, max_tokens=None):
    import torch
    T = x_bits.shape[0]
    ctx = aeon_b200.Context(cfg, max_tokens=max_tokens or T)
    x = gs.torch_bits(x_bits, cfg.act_dtype)
    w, ids = ctx.router_topk(x, layer.gate)
    out = torch.empty(T, cfg.hidden, dtype=torch.float32, device="cuda")
    ctx.shared_expert(layer.shared[0], layer.shared[1], layer.shared[2], x, out)
    shared_only = out.clone()
    ctx.moe_decode(layer.pool.base, layer.slot_of, x, ids, w, out)
    ctx.check()
    return (out.cpu().numpy().astype(np.float64), shared_only.cpu().numpy().astype(np.float64),
            w.cpu().numpy(), ids.cpu().numpy())


@pytest.mark.parametrize("tokens", [1, 8])
def test_layer_matches_oracle(oracle, tokens):
    cfg = aeon_b200.preset("baseline")
    layer = gs.SyntheticLayer(cfg, None, seed=0, layer=0, with_shared=True)   # all 256 experts
    x_bits = gs.activations(cfg, tokens, seed=0)
    got, shared_got, w, ids = run_layer(cfg, layer, x_bits)

    # routing: bit-exact ids against the oracle on the same-order logits
    logits = oracle.router_logits_f32_ordered(layer.gate_bits, cfg.act_dtype, x_bits, cfg.act_dtype)
    want_ids, want_w, _ = oracle.router_topk(logits.astype(np.float64), None, cfg.top_k,
                                              cfg.routed_scaling, cfg.score_fn)
    np.testing.assert_array_equal(ids, want_ids)
    assert np.abs(w - want_w).max() < 1e-5

    # shared expert alone
    x = synth.from_bits16(x_bits, cfg.act_dtype)
    w1, w3, w2 = layer.shared_bits(oracle)
    check = [0] if tokens == 1 else [0, tokens - 1]
    routed = gs.oracle_routed(oracle, layer, x_bits, want_ids, want_w, check)
    for t in check:
        shared_want = oracle.dense_ffn(w1, w3, w2, cfg.act_dtype, x[t], cfg.swiglu_limit)
        gs.assert_close(oracle, shared_want, shared_got[t], "shared expert")
        # layer output = routed sum + shared (reassociation against the fused order allowed)
        s = gs.assert_close(oracle, routed[t] + shared_want, got[t], f"layer token {t}")
        print(f"\nlayer T={tokens} token {t}: max_abs={s['max_abs']:.3e} rel_l2={s['rel_l2']:.3e}")
        # the shared contribution enters exactly once
        assert oracle.compare(routed[t] + 2 * shared_want, got[t])["rel_l2"] > 1e-3 or \
            np.abs(shared_want).max() < 1e-3
