"""Permutation against its definition (the reference's gate: tests/test_expert_permutation.cpp:
monotone offsets anchored at 0 and the draw count, every draw under its own expert, a
bijection, ascending placement, widths equal to the histogram)."""
import numpy as np
import pytest

import aeon_b200

pytestmark = pytest.mark.gpu


def check_definition(ids, experts, offsets, token_idx, draw_idx, wpos, weights):
    tokens, slots = ids.shape
    flat = ids.ravel()
    valid = (flat >= 0) & (flat < experts)
    placed = int(valid.sum())
    assert offsets[0] == 0 and offsets[experts] == placed
    assert (np.diff(offsets) >= 0).all()
    np.testing.assert_array_equal(np.diff(offsets), np.bincount(flat[valid], minlength=experts))
    seen = np.zeros(flat.size, dtype=bool)
    for e in range(experts):
        seg = draw_idx[offsets[e]:offsets[e + 1]]
        assert (flat[seg] == e).all()
        assert (np.diff(seg) > 0).all()          # ascending draw order inside an expert
        seen[seg] = True
        np.testing.assert_array_equal(token_idx[offsets[e]:offsets[e + 1]], seg // slots)
    np.testing.assert_array_equal(seen, valid)   # bijection onto the valid draws
    if weights is not None:
        np.testing.assert_array_equal(wpos[:placed], weights.ravel()[draw_idx[:placed]])
    # identical to a stable sort by expert
    order = np.argsort(np.where(valid, flat, experts), kind="stable")[:placed]
    np.testing.assert_array_equal(draw_idx[:placed], order)


@pytest.mark.parametrize("tokens,slots,experts,seed", [
    (1, 6, 256, 0x5EED0001), (7, 6, 256, 0x5EED0002), (300, 6, 256, 0x5EED0003),
    (64, 6, 8, 0x5EED0004), (128, 8, 256, 1), (4096, 8, 256, 2), (0, 8, 256, 3),
])
def test_permutation_definition(tokens, slots, experts, seed):
    import torch
    cfg = aeon_b200.preset("baseline")
    ctx = aeon_b200.Context(cfg, max_tokens=8)
    rng = np.random.default_rng(seed)
    ids = np.stack([rng.permutation(experts)[:slots] for _ in range(tokens)]).astype(np.int32) \
        if tokens else np.zeros((0, slots), dtype=np.int32)
    weights = rng.random((tokens, slots)).astype(np.float32)
    d_ids = torch.from_numpy(ids).cuda().reshape(tokens, slots)
    d_w = torch.from_numpy(weights).cuda()
    off, tok, drw, wpos = ctx.expert_permutation(d_ids, experts, d_w)
    ctx.check()
    check_definition(ids, experts, off.cpu().numpy(), tok.cpu().numpy(), drw.cpu().numpy(),
                     wpos.cpu().numpy(), weights)
    # a second run is bit-identical (placement is a pure function of the ids)
    off2, tok2, drw2, _ = ctx.expert_permutation(d_ids, experts, d_w)
    assert torch.equal(off, off2) and torch.equal(tok, tok2) and torch.equal(drw, drw2)


def test_out_of_range_ids_are_dropped():
    import torch
    cfg = aeon_b200.preset("baseline")
    ctx = aeon_b200.Context(cfg, max_tokens=8)
    ids = np.array([[3, 999, 5, -1], [5, 5, 300, 0]], dtype=np.int32)
    off, tok, drw, _ = ctx.expert_permutation(torch.from_numpy(ids).cuda(), 256)
    check_definition(ids, 256, off.cpu().numpy(), tok.cpu().numpy(), drw.cpu().numpy(), None, None)
    assert int(off[256]) == 5
