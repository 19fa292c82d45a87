"""Router parity: logits bit-identical to the oracle's same-order fp32 sum, ids bit-exact,
weights within 1e-5 (the reference's router gate: tests/test_v4_router_oracle.cpp:73-76)."""
import numpy as np
import pytest

import aeon_b200
from aeon_b200 import synth
import gpu_support as gs

pytestmark = pytest.mark.gpu


def run_router(cfg, x_bits, gate_bits, bias=None, hash_table=None, token_ids=None):
    import torch
    ctx = aeon_b200.Context(cfg, max_tokens=max(1, x_bits.shape[0]))
    x = gs.torch_bits(x_bits, cfg.act_dtype)
    gate = gs.torch_bits(gate_bits, cfg.act_dtype)
    logits = torch.empty(x_bits.shape[0], cfg.experts, dtype=torch.float32, device="cuda")
    d_bias = None if bias is None else torch.from_numpy(bias.astype(np.float32)).cuda()
    d_table = None if hash_table is None else torch.from_numpy(hash_table).cuda()
    d_tok = None if token_ids is None else torch.from_numpy(token_ids).cuda()
    w, ids = ctx.router_topk(x, gate, d_bias, d_table, d_tok, logits_out=logits)
    ctx.check()
    return w.cpu().numpy(), ids.cpu().numpy(), logits.cpu().numpy()


@pytest.mark.parametrize("tokens", [1, 8, 16, 21, 32, 37, 128])
def test_baseline_router_matches_oracle(oracle, tokens):
    cfg = aeon_b200.preset("baseline")
    rng = np.random.default_rng(0)
    gate_bits = synth.normal_bits(rng, (cfg.experts, cfg.hidden), 0.01, cfg.act_dtype)
    x_bits = gs.activations(cfg, tokens, seed=0)
    w, ids, logits = run_router(cfg, x_bits, gate_bits)

    want_logits = oracle.router_logits_f32_ordered(gate_bits, cfg.act_dtype, x_bits, cfg.act_dtype)
    np.testing.assert_array_equal(logits, want_logits)          # bit-identical fp32 logits
    want_ids, want_w, _ = oracle.router_topk(want_logits.astype(np.float64), None, cfg.top_k,
                                              cfg.routed_scaling, cfg.score_fn)
    np.testing.assert_array_equal(ids, want_ids)                 # bit-exact ids, positional
    assert np.abs(w - want_w).max() < 1e-5
    np.testing.assert_allclose(w.sum(axis=1), 1.0, atol=1e-6)

    # Against the fp64-accumulated logits: equal wherever the oracle's selection margin is
    # above fp32 accumulation noise; the margins are reported so a flip is diagnosable.
    l64 = oracle.router_logits_f64(gate_bits, cfg.act_dtype, x_bits, cfg.act_dtype)
    assert np.abs(l64 - want_logits).max() < 2e-5
    ids64, w64, margin = oracle.router_topk(l64, None, cfg.top_k, cfg.routed_scaling, cfg.score_fn)
    safe = margin > 1e-5
    assert safe.mean() > 0.9
    np.testing.assert_array_equal(ids[safe], ids64[safe])
    assert np.abs(w[safe] - w64[safe]).max() < 1e-5


def test_ties_resolve_to_lowest_index():
    cfg = aeon_b200.preset("baseline")
    gate = np.zeros((cfg.experts, cfg.hidden))
    gate[[7, 70, 180, 255], :8] = 0.5     # four identical rows -> a four-way tie at the top
    gate_bits = synth.to_bits16(gate, cfg.act_dtype)
    x_bits = synth.to_bits16(np.ones((2, cfg.hidden)), cfg.act_dtype)
    w, ids, logits = run_router(cfg, x_bits, gate_bits)
    assert ids[0].tolist() == [7, 70, 180, 255, 0, 1, 2, 3]
    assert ids[1].tolist() == [7, 70, 180, 255, 0, 1, 2, 3]
    assert logits[0, 7] == 4.0 and logits[0, 0] == 0.0


def test_reference_preset_bias_and_hash_branch(oracle):
    cfg = aeon_b200.preset("ref_dsv4")
    rng = np.random.default_rng(3)
    gate_bits = synth.normal_bits(rng, (cfg.experts, cfg.hidden), 0.05, cfg.act_dtype)
    x_bits = gs.activations(cfg, 16, seed=3)
    bias = rng.uniform(-0.5, 0.5, cfg.experts).astype(np.float32)
    w, ids, logits = run_router(cfg, x_bits, gate_bits, bias=bias)
    want_logits = oracle.router_logits_f32_ordered(gate_bits, cfg.act_dtype, x_bits, cfg.act_dtype)
    np.testing.assert_array_equal(logits, want_logits)
    want_ids, want_w, margin = oracle.router_topk(want_logits.astype(np.float64), bias.astype(np.float64),
                                                  cfg.top_k, cfg.routed_scaling, cfg.score_fn)
    safe = margin > 1e-5     # score + bias is compared in fp32 on the device
    assert safe.mean() > 0.9
    np.testing.assert_array_equal(ids[safe], want_ids[safe])
    assert np.abs(w[safe] - want_w[safe]).max() < 1e-5
    np.testing.assert_allclose(w.sum(axis=1), 1.5, atol=1e-5)
    # the bias is load-bearing: without it the selection changes somewhere
    _, ids_nobias, _ = run_router(cfg, x_bits, gate_bits)
    assert (ids_nobias != ids).any()

    # hash branch: ids straight from the (unsorted) table row of each token id
    table = np.stack([rng.permutation(cfg.experts)[:cfg.top_k] for _ in range(50)]).astype(np.int64)
    token_ids = rng.integers(0, 50, 16).astype(np.int32)
    w, ids, _ = run_router(cfg, x_bits, gate_bits, bias=bias, hash_table=table, token_ids=token_ids)
    for t in range(16):
        hid, hw = oracle.router_hash(want_logits[t].astype(np.float64), table[token_ids[t]],
                                     cfg.routed_scaling, cfg.score_fn)
        assert ids[t].tolist() == hid.tolist()
        assert np.abs(w[t] - hw).max() < 1e-5
