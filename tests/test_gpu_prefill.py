"""Prefill path (grouped tcgen05 GEMMs) parity.

Tolerance: max-abs 2e-2 and relative-L2 1e-3 on the layer output against the fp64 oracle that
applies the same operand roundings as the tensor-core path (weights fp16(q*scale), activations
fp16, hidden vector rounded to fp16 between the GEMMs) — the reference's own method for its
grouped kernels (tests/test_v4_grouped_wmma_oracle.cpp:63-73,219-228). The distance to the
exact oracle (= the decode path, which dequantises exactly) is reported alongside."""
import numpy as np
import pytest

import aeon_b200
from aeon_b200 import synth
import gpu_support as gs

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("tokens,resident", [(40, list(range(16, 32))), (330, [1, 2, 3, 5, 8, 13, 21, 34, 55])])
def test_prefill_matches_mirrored_oracle_and_decode(oracle, tokens, resident):
    import torch
    cfg = aeon_b200.preset("baseline")
    layer = gs.SyntheticLayer(cfg, resident, seed=8, layer=2, with_shared=False)
    rng = np.random.default_rng(tokens)
    k = cfg.top_k
    ids = np.stack([rng.choice(resident, k, replace=False) for _ in range(tokens)]).astype(np.int32)
    w = rng.random((tokens, k)) + 0.05
    w = (w / w.sum(axis=1, keepdims=True)).astype(np.float32)
    x_bits = gs.activations(cfg, tokens, seed=3)
    x = gs.torch_bits(x_bits, cfg.act_dtype)
    d_ids, d_w = torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda()
    init = rng.standard_normal((tokens, cfg.hidden)).astype(np.float32)

    ctx = aeon_b200.Context(cfg, max_tokens=min(tokens, 512))
    out = torch.from_numpy(init).cuda()
    ctx.moe_prefill(layer.pool.base, layer.slot_of, x, d_ids, d_w, out)
    ctx.check()
    got = out.cpu().numpy().astype(np.float64) - init

    check = sorted({0, tokens // 3, tokens - 1})
    want = gs.mirrored_oracle(oracle, layer, x_bits, ids, w.astype(np.float64), check)
    for t in check:
        s = gs.assert_close(oracle, want[t], got[t], f"prefill token {t}")
        print(f"\nT={tokens} token {t}: vs mirrored oracle max_abs={s['max_abs']:.3e} rel_l2={s['rel_l2']:.3e}")

    # against the decode path (exact dequantisation, fp32 hidden) on identical inputs
    dec = torch.zeros(tokens, cfg.hidden, dtype=torch.float32, device="cuda")
    ctx.moe_decode(layer.pool.base, layer.slot_of, x, d_ids, d_w, dec)
    ctx.check()
    dec = dec.cpu().numpy().astype(np.float64)
    s = oracle.compare(dec, got)
    print(f"T={tokens}: prefill vs exact decode path max_abs={s['max_abs']:.3e} rel_l2={s['rel_l2']:.3e} "
          f"peak={np.abs(dec).max():.1f}")
    assert s["rel_l2"] < 1e-3                      # the operand roundings stay inside rel-L2

    # bit-reproducible: one writer per element, fixed-order sums
    again = torch.from_numpy(init).cuda()
    ctx.moe_prefill(layer.pool.base, layer.slot_of, x, d_ids, d_w, again)
    ctx.check()
    assert torch.equal(out, again)


def test_prefill_reference_preset(oracle):
    """Group 32 / hidden 4096 / fp16: the reference model's shapes through the grouped path."""
    import torch
    cfg = aeon_b200.preset("ref_dsv4")
    resident = list(range(8))
    layer = gs.SyntheticLayer(cfg, resident, seed=1, layer=0, with_shared=False)
    rng = np.random.default_rng(5)
    tokens, k = 24, cfg.top_k
    ids = np.stack([rng.choice(resident, k, replace=False) for _ in range(tokens)]).astype(np.int32)
    w = np.full((tokens, k), 1.5 / k, dtype=np.float32)
    x_bits = gs.activations(cfg, tokens, seed=4)
    x = gs.torch_bits(x_bits, cfg.act_dtype)
    ctx = aeon_b200.Context(cfg, max_tokens=tokens)
    out = torch.zeros(tokens, cfg.hidden, dtype=torch.float32, device="cuda")
    ctx.moe_prefill(layer.pool.base, layer.slot_of, x, torch.from_numpy(ids).cuda(),
                    torch.from_numpy(w).cuda(), out)
    ctx.check()
    want = gs.mirrored_oracle(oracle, layer, x_bits, ids, w.astype(np.float64), [0, tokens - 1])
    got = out.cpu().numpy().astype(np.float64)
    for t in (0, tokens - 1):
        gs.assert_close(oracle, want[t], got[t], f"ref preset prefill token {t}")
