"""Decode path parity: the CUDA dual product + clamped SwiGLU + W2 + slot-order accumulate
against the fp64 oracle on identical seeded inputs, through the C ABI.

Tolerance (benchmark contract): max-abs 2e-2 and relative-L2 1e-3 on the layer output
against the exact fp64 oracle. Expert ids are chosen by the tests here (routing parity is
test_gpu_router.py); the full router -> experts composition is test_gpu_layer.py."""
import numpy as np
import pytest

import aeon_b200
from aeon_b200 import synth
import gpu_support as gs

pytestmark = pytest.mark.gpu


def run_decode(cfg, layer, x_bits, ids, weights, init=None, max_tokens=None):
    import torch
    T = x_bits.shape[0]
    ctx = aeon_b200.Context(cfg, max_tokens=max_tokens or T)
    x = gs.torch_bits(x_bits, cfg.act_dtype)
    d_ids = torch.from_numpy(ids.astype(np.int32)).cuda()
    d_w = torch.from_numpy(weights.astype(np.float32)).cuda()
    out = torch.zeros(T, cfg.hidden, dtype=torch.float32, device="cuda") if init is None \
        else torch.from_numpy(init.astype(np.float32)).cuda()
    ctx.moe_decode(layer.pool.base, layer.slot_of, x, d_ids, d_w, out)
    ctx.check()
    return out.cpu().numpy().astype(np.float64), ctx


def random_routing(rng, tokens, top_k, experts):
    ids = np.stack([rng.choice(experts, top_k, replace=False) for _ in range(tokens)]).astype(np.int32)
    w = rng.random((tokens, top_k)) + 0.05
    w = (w / w.sum(axis=1, keepdims=True)).astype(np.float32)
    return ids, w


@pytest.mark.parametrize("tokens", [1, 8])
def test_baseline_decode_matches_oracle(oracle, tokens):
    cfg = aeon_b200.preset("baseline")
    resident = list(range(40, 56))
    layer = gs.SyntheticLayer(cfg, resident, seed=0, layer=0, with_shared=False)
    rng = np.random.default_rng(10 + tokens)
    ids, w = random_routing(rng, tokens, cfg.top_k, resident)
    x_bits = gs.activations(cfg, tokens, seed=1)
    got, ctx = run_decode(cfg, layer, x_bits, ids, w)
    want = gs.oracle_routed(oracle, layer, x_bits, ids, w.astype(np.float64))
    want = np.stack([want[t] for t in range(tokens)])
    s = gs.assert_close(oracle, want, got, f"decode T={tokens}")
    print(f"\nT={tokens}: max_abs={s['max_abs']:.3e} rel_l2={s['rel_l2']:.3e} peak={np.abs(want).max():.1f}")
    distinct, entries = ctx.last_stats()
    assert distinct == len(np.unique(ids)) and entries >= distinct
    # deliberately wrong control: swapping two routing weights must be visible
    if tokens == 1:
        w_bad = w.copy()
        w_bad[0, [0, 1]] = w_bad[0, [1, 0]] + np.array([0.1, -0.1], dtype=np.float32)
        bad, _ = run_decode(cfg, layer, x_bits, ids, w_bad)
        assert oracle.compare(want, bad)["rel_l2"] > 1e-2


def test_ragged_batch_with_chunked_expert_and_initial_value(oracle):
    """37 tokens over 10 experts: several experts hold more than 8 tokens (split into
    several work entries), token counts are ragged, and the accumulator starts from a
    non-zero value that must enter exactly once."""
    cfg = aeon_b200.preset("baseline")
    resident = [3, 4, 5, 6, 100, 101, 102, 200, 201, 255]
    layer = gs.SyntheticLayer(cfg, resident, seed=2, layer=1, with_shared=False)
    rng = np.random.default_rng(77)
    T = 37
    ids, w = random_routing(rng, T, cfg.top_k, resident)
    x_bits = gs.activations(cfg, T, seed=5)
    init = rng.standard_normal((T, cfg.hidden)).astype(np.float32)
    got, ctx = run_decode(cfg, layer, x_bits, ids, w, init=init, max_tokens=64)
    check = [0, 5, 17, 36]
    want = gs.oracle_routed(oracle, layer, x_bits, ids, w.astype(np.float64), check)
    for t in check:
        gs.assert_close(oracle, want[t] + init[t].astype(np.float64), got[t], f"token {t}")
    distinct, entries = ctx.last_stats()
    assert distinct == 10 and entries > 10        # 296 draws over 10 experts -> chunked
    # bit-reproducible: a second run gives identical bytes (fixed summation order, no atomics
    # in the data path)
    again, _ = run_decode(cfg, layer, x_bits, ids, w, init=init, max_tokens=64)
    np.testing.assert_array_equal(got, again)


def test_clamp_fires_and_large_activations(oracle):
    """8x activations push gate/up past the limit (reference:
    tests/test_v4_expert_oracle.cpp:444-587 runs 1x and 8x)."""
    cfg = aeon_b200.preset("baseline")
    resident = list(range(8))
    layer = gs.SyntheticLayer(cfg, resident, seed=4, layer=0, with_shared=False)
    ids = np.arange(8, dtype=np.int32)[None, :]
    w = np.full((1, 8), 0.125, dtype=np.float32)
    x_bits = gs.activations(cfg, 1, seed=9, scale=8.0)
    got, _ = run_decode(cfg, layer, x_bits, ids, w)
    la = oracle.layout_args(cfg)
    x = synth.from_bits16(x_bits, cfg.act_dtype)[0]
    payload = oracle.synth_expert_payload(la, 4, 0, 0, layer.scale_table)
    _, _, gate, up = oracle.expert_ffn(la, payload, x, cfg.swiglu_limit, 0, want_pre=True)
    assert (gate > cfg.swiglu_limit).any() and (np.abs(up) > cfg.swiglu_limit).any()
    want = gs.oracle_routed(oracle, layer, x_bits, ids, w.astype(np.float64))[0]
    s = oracle.compare(want, got[0])
    assert s["rel_l2"] <= gs.TOL_REL_L2 and s["max_abs"] <= 1e-4 * np.abs(want).max() + gs.TOL_MAX_ABS, s


def test_reference_preset_decode_matches_oracle(oracle):
    """The reference model's own shapes (hidden 4096, top-6, group 32, fp16) on payloads
    built by the oracle's fixture encoder (power-of-two scales)."""
    import torch
    cfg = aeon_b200.preset("ref_dsv4")
    la = oracle.layout_args(cfg)
    lay = oracle.layout(la)
    rng = np.random.default_rng(0xE7E)
    pool = aeon_b200.ExpertPool(cfg, 6)
    payloads = []
    for e in range(6):
        payload = np.zeros(lay["payload_bytes"], dtype=np.uint8)
        for kind in range(3):
            m = lay[("w1", "w2", "w3")[kind]]
            oracle.encode_matrix(la, kind, payload, rng.uniform(-0.06, 0.06, m["rows"] * m["cols"]))
        pool.upload(e, payload)
        payloads.append(payload)
    slot_of = np.full(cfg.experts, -1, dtype=np.int32)
    experts = [9, 200, 31, 77, 150, 3]
    slot_of[experts] = np.arange(6)
    T = 3
    ids = np.stack([rng.permutation(experts) for _ in range(T)]).astype(np.int32)
    w = rng.random((T, 6)).astype(np.float32)
    w = w / w.sum(axis=1, keepdims=True) * 1.5
    x_bits = gs.activations(cfg, T, seed=21)
    ctx = aeon_b200.Context(cfg, max_tokens=T)
    out = torch.zeros(T, cfg.hidden, dtype=torch.float32, device="cuda")
    ctx.moe_decode(pool.base, torch.from_numpy(slot_of).cuda(), gs.torch_bits(x_bits, cfg.act_dtype),
                   torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda(), out)
    ctx.check()
    x = synth.from_bits16(x_bits, cfg.act_dtype)
    got = out.cpu().numpy().astype(np.float64)
    ys = {e: oracle.expert_ffn_batch(la, payloads[experts.index(e)], x, cfg.swiglu_limit) for e in experts}
    for t in range(T):
        eo = np.stack([ys[int(e)][t] for e in ids[t]])
        want = oracle.moe_combine(eo, w[t].astype(np.float64))
        gs.assert_close(oracle, want, got[t], f"ref preset token {t}")


def test_absent_expert_is_reported_not_ignored():
    import torch
    cfg = aeon_b200.preset("baseline")
    layer = gs.SyntheticLayer(cfg, list(range(8)), seed=0, layer=0, with_shared=False)
    ids = np.array([[0, 1, 2, 3, 4, 5, 6, 99]], dtype=np.int32)      # 99 has no slot
    w = np.full((1, 8), 0.125, dtype=np.float32)
    ctx = aeon_b200.Context(cfg, max_tokens=1)
    out = torch.zeros(1, cfg.hidden, dtype=torch.float32, device="cuda")
    ctx.moe_decode(layer.pool.base, layer.slot_of, gs.torch_bits(gs.activations(cfg, 1), cfg.act_dtype),
                   torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda(), out)
    with pytest.raises(aeon_b200.AeonError) as e:
        ctx.check()
    assert e.value.status == 2
    ctx.check()    # the flag is cleared once reported; the context stays usable


def test_argument_validation():
    import torch
    cfg = aeon_b200.preset("baseline")
    layer = gs.SyntheticLayer(cfg, list(range(8)), seed=0, layer=0, with_shared=False)
    ctx = aeon_b200.Context(cfg, max_tokens=2)
    x = gs.torch_bits(gs.activations(cfg, 3), cfg.act_dtype)
    ids = torch.zeros(3, 8, dtype=torch.int32, device="cuda")
    w = torch.zeros(3, 8, dtype=torch.float32, device="cuda")
    out = torch.zeros(3, cfg.hidden, dtype=torch.float32, device="cuda")
    with pytest.raises(aeon_b200.AeonError) as e:      # more tokens than the context allows
        ctx.moe_decode(layer.pool.base, layer.slot_of, x, ids, w, out)
    assert e.value.status == 1
    with pytest.raises(aeon_b200.AeonError):           # null pool
        ctx.moe_decode(0, layer.slot_of, x[:1], ids[:1], w[:1], out[:1])


def test_group_128_at_hidden_4096_matches_oracle(oracle):
    """The group-128 kernels at the reference model's hidden width (their second instance)."""
    cfg = aeon_b200.preset("baseline").copy(hidden=4096)
    resident = [3, 4, 5, 6, 9, 10, 11, 12, 13]
    layer = gs.SyntheticLayer(cfg, resident, seed=2, layer=1, with_shared=False)
    rng = np.random.default_rng(77)
    tokens = 11                                        # one expert gets more than one work entry
    ids, w = random_routing(rng, tokens, cfg.top_k, resident)
    x_bits = gs.activations(cfg, tokens, seed=6)
    got, _ = run_decode(cfg, layer, x_bits, ids, w)
    want = gs.oracle_routed(oracle, layer, x_bits, ids, w.astype(np.float64), [0, 5, tokens - 1])
    for t in (0, 5, tokens - 1):
        gs.assert_close(oracle, want[t], got[t], f"hidden 4096 token {t}")


def test_misaligned_accumulator_is_refused_on_the_host():
    """A float4-misaligned accumulator or row stride is an argument error, never a device fault."""
    import torch
    cfg = aeon_b200.preset("baseline")
    layer = gs.SyntheticLayer(cfg, [0, 1, 2, 3, 4, 5, 6, 7], seed=0, layer=0, with_shared=False)
    ctx = aeon_b200.Context(cfg, max_tokens=2)
    x = gs.torch_bits(gs.activations(cfg, 2, seed=0), cfg.act_dtype)
    ids = torch.arange(8, dtype=torch.int32, device="cuda").repeat(2, 1).contiguous()
    w = torch.full((2, 8), 0.125, dtype=torch.float32, device="cuda")
    flat = torch.zeros(2 * (cfg.hidden + 2) + 1, dtype=torch.float32, device="cuda")
    shifted = flat[1:1 + 2 * cfg.hidden].view(2, cfg.hidden)                    # 4 bytes off a 16-byte boundary
    odd_stride = flat[:2 * (cfg.hidden + 2)].view(2, cfg.hidden + 2)[:, :cfg.hidden]   # stride not a multiple of 4
    for bad in (shifted, odd_stride):
        with pytest.raises(aeon_b200.AeonError) as e:
            ctx.moe_decode(layer.pool.base, layer.slot_of, x, ids, w, bad)
        assert e.value.status == 1
    ctx.check()
