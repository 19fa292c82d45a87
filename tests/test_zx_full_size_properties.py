"""The decode and prefill paths at the benchmark's full size (one layer, all 256 experts,
batch 128 / 4096 tokens), where the fp64 oracle is too slow to cover every token: properties
that hold at any size, plus the oracle on a sample of tokens.

  * bit-reproducibility of two runs;
  * homogeneity in the routing weights: doubling every weight doubles every output bit for
    bit (one multiply by the weight per draw, fixed-order sums, powers of two are exact);
  * the accumulator's initial value passes through: out(init) - out(0) == init up to fp32
    rounding of the sums;
  * a permutation of the tokens permutes the outputs;
  * sampled tokens of the decode path against the exact fp64 oracle, and of the grouped path
    against the fp64 oracle that applies the grouped path's operand roundings (fp16 MMA
    operands), both within the tolerance;
  * decode path and grouped path agree in relative L2 on the same batch (their max-abs
    distance is the fp16-operand rounding of the grouped path and is printed).

Collected late: it runs after the per-kernel parity tests."""
import numpy as np
import pytest

import aeon_b200
import gpu_support as gs

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def full_layer():
    cfg = aeon_b200.preset("baseline")
    return cfg, gs.SyntheticLayer(cfg, None, seed=4, layer=5, with_shared=False)


def routed(ctx, layer, x, ids, w, init=None, prefill=False):
    import torch
    out = torch.zeros(x.shape[0], layer.cfg.hidden, dtype=torch.float32, device="cuda") if init is None \
        else init.clone()
    call = ctx.moe_prefill if prefill else ctx.moe_decode
    call(layer.pool.base, layer.slot_of, x, ids, w, out)
    ctx.check()
    return out


def test_decode_batch_128_properties(oracle, full_layer):
    import torch
    cfg, layer = full_layer
    T = 128
    x_bits = gs.activations(cfg, T, seed=21)
    x = gs.torch_bits(x_bits, cfg.act_dtype)
    ctx = aeon_b200.Context(cfg, max_tokens=T)
    w, ids = ctx.router_topk(x, layer.gate)           # the benchmark's own routing (near-uniform load)
    ids_h, w_h = ids.cpu().numpy(), w.cpu().numpy()
    assert len(np.unique(ids_h)) > 200                 # the batch touches most of the 256 experts

    base = routed(ctx, layer, x, ids, w)
    again = routed(ctx, layer, x, ids, w)
    assert torch.equal(base, again)

    doubled = routed(ctx, layer, x, ids, w * 2.0)
    assert torch.equal(doubled, base * 2.0)

    init = torch.from_numpy(np.random.default_rng(2).standard_normal((T, cfg.hidden)).astype(np.float32)).cuda()
    with_init = routed(ctx, layer, x, ids, w, init=init)
    assert (with_init - base - init).abs().max().item() <= 2e-5 * max(1.0, base.abs().max().item())

    perm = torch.from_numpy(np.random.default_rng(3).permutation(T)).cuda()
    permuted = routed(ctx, layer, x[perm].contiguous(), ids[perm].contiguous(), w[perm].contiguous())
    s = oracle.compare(base[perm].double().cpu().numpy(), permuted.double().cpu().numpy())
    # not bit-identical: which tokens share a work entry decides whether the hi and lo planes of
    # the hidden vector meet before or after the K-split sum (fp32 reassociation only)
    assert s["rel_l2"] <= 5e-6 and s["max_abs"] <= 1e-3, s

    # the decode path against the exact fp64 oracle on sampled tokens, before any cross-path check
    sample = [0, 77, T - 1]
    want = gs.oracle_routed(oracle, layer, x_bits, ids_h, w_h.astype(np.float64), sample)
    for t in sample:
        s = gs.assert_close(oracle, want[t], base[t].double().cpu().numpy(), f"batch 128 token {t}")
        print(f"\nbatch 128 token {t}: decode vs exact oracle max_abs={s['max_abs']:.3e} rel_l2={s['rel_l2']:.3e}")

    # the grouped path on the same batch: against the oracle that applies its operand roundings
    # (the tolerance holds there), and against the decode path in rel-L2 only -- its max-abs
    # distance to exact arithmetic is that of fp16 MMA operands and is printed, not bounded
    grouped = routed(ctx, layer, x, ids, w, prefill=True)
    mirrored = gs.mirrored_oracle(oracle, layer, x_bits, ids_h, w_h.astype(np.float64), sample)
    for t in sample:
        s = gs.assert_close(oracle, mirrored[t], grouped[t].double().cpu().numpy(), f"grouped token {t}")
        print(f"batch 128 token {t}: grouped vs operand-mirrored oracle max_abs={s['max_abs']:.3e} "
              f"rel_l2={s['rel_l2']:.3e}")
    s = oracle.compare(base.double().cpu().numpy(), grouped.double().cpu().numpy())
    print(f"batch 128: decode vs grouped path max_abs={s['max_abs']:.3e} rel_l2={s['rel_l2']:.3e}")
    assert s["rel_l2"] <= gs.TOL_REL_L2, s


def test_prefill_4096_tokens_properties(oracle, full_layer):
    import torch
    cfg, layer = full_layer
    T = 4096
    x_bits = gs.activations(cfg, T, seed=22)
    x = gs.torch_bits(x_bits, cfg.act_dtype)
    ctx = aeon_b200.Context(cfg, max_tokens=128)
    # Zipf-like skew as in the benchmark's prefill configuration: a per-expert logit bias
    rank = np.random.default_rng(5).permutation(cfg.experts)
    bias = torch.from_numpy((0.3 * (1.0 / (1.0 + rank)) ** 1.1 * cfg.experts ** 0.5).astype(np.float32)).cuda()
    logits = torch.empty(T, cfg.experts, dtype=torch.float32, device="cuda")
    w, ids = ctx.router_topk(x, layer.gate, bias=bias, logits_out=logits)
    counts = np.bincount(ids.cpu().numpy().ravel(), minlength=cfg.experts)
    assert counts.max() > 256 and counts.min() >= 0     # ragged: some experts need several token tiles

    base = routed(ctx, layer, x, ids, w, prefill=True)
    again = routed(ctx, layer, x, ids, w, prefill=True)
    assert torch.equal(base, again)
    doubled = routed(ctx, layer, x, ids, w * 2.0, prefill=True)
    assert torch.equal(doubled, base * 2.0)

    # sampled tokens against the oracle with the grouped path's operand roundings; one of them is
    # routed to the hottest expert, whose tokens span several token tiles
    ids_h, w_h = ids.cpu().numpy(), w.cpu().numpy().astype(np.float64)
    hottest = int(counts.argmax())
    t_hot = int(np.nonzero((ids_h == hottest).any(axis=1))[0][-1])      # in the expert's last tile
    sample = sorted({0, t_hot, T - 1})
    want = gs.mirrored_oracle(oracle, layer, x_bits, ids_h, w_h, sample)
    exact = gs.oracle_routed(oracle, layer, x_bits, ids_h, w_h, [t_hot])
    for t in sample:
        s = gs.assert_close(oracle, want[t], base[t].double().cpu().numpy(), f"prefill 4096 token {t}")
        print(f"\n4096 tokens, token {t}: grouped vs operand-mirrored oracle max_abs={s['max_abs']:.3e} "
              f"rel_l2={s['rel_l2']:.3e}")
    s = oracle.compare(exact[t_hot], base[t_hot].double().cpu().numpy())
    print(f"4096 tokens, token {t_hot}: grouped vs exact oracle max_abs={s['max_abs']:.3e} rel_l2={s['rel_l2']:.3e}")
    assert s["rel_l2"] <= gs.TOL_REL_L2, s

    # the same tokens in chunks of 128 through the decode path (exact dequantisation): rel-L2
    ctx_d = aeon_b200.Context(cfg, max_tokens=128)
    for t0 in (0, 1920, T - 128):
        part = routed(ctx_d, layer, x[t0:t0 + 128], ids[t0:t0 + 128].contiguous(), w[t0:t0 + 128].contiguous())
        s = oracle.compare(part.double().cpu().numpy(), base[t0:t0 + 128].double().cpu().numpy())
        print(f"4096 tokens, rows {t0}..{t0 + 127}: decode vs grouped max_abs={s['max_abs']:.3e} rel_l2={s['rel_l2']:.3e}")
        assert s["rel_l2"] <= gs.TOL_REL_L2, (t0, s)
