"""The peer-memory combine on one GPU (a group of one rank): push + combine must equal the
collective form of the same step (slot-order partial, then the rank-order add) bit for bit, and a combine whose flag nobody posts must run out of its wait
budget and be reported as TIMEOUT with the context still usable -- the failure is made on the
host side (the push is simply not issued); nothing faults, traps or hangs."""
import numpy as np
import pytest

import aeon_b200
import gpu_support as gs

pytestmark = pytest.mark.gpu


def _setup(tokens):
    import torch
    cfg = aeon_b200.preset("baseline")
    resident = list(range(16))
    layer = gs.SyntheticLayer(cfg, resident, seed=6, layer=0, with_shared=False)
    rng = np.random.default_rng(1)
    ids = np.stack([rng.choice(resident, cfg.top_k, replace=False) for _ in range(tokens)]).astype(np.int32)
    w = rng.random((tokens, cfg.top_k)).astype(np.float32) + 0.1
    x = gs.torch_bits(gs.activations(cfg, tokens, seed=9), cfg.act_dtype)
    return cfg, layer, x, torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda()


def test_push_and_combine_equal_the_collective_form():
    import torch
    tokens = 6
    cfg, layer, x, ids, w = _setup(tokens)
    ctx = aeon_b200.Context(cfg, max_tokens=tokens)
    group = aeon_b200.Group(aeon_b200.group_unique_id(), 0, 1, 0)
    peer = aeon_b200.PeerCombine(group, 0, tokens, cfg.hidden)
    try:
        init = torch.from_numpy(np.random.default_rng(2).standard_normal((tokens, cfg.hidden)).astype(np.float32)).cuda()
        # the collective form: the rank's partial written in slot order, then added in rank order
        partial = torch.empty(1, tokens, cfg.hidden, dtype=torch.float32, device="cuda")
        ctx.moe_decode(layer.pool.base, layer.slot_of, x, ids, w, partial[0], skip_absent=True, overwrite=True)
        want = init.clone()
        aeon_b200.ep_combine(want, partial)
        direct = init.clone()                    # and the single-GPU call, equal up to fp32 association
        ctx.moe_decode(layer.pool.base, layer.slot_of, x, ids, w, direct)
        assert (direct - want).abs().max().item() <= 1e-3
        for _ in range(3):                       # the epoch advances on the device, call after call
            got = init.clone()
            ctx.moe_decode(layer.pool.base, layer.slot_of, x, ids, w, got, defer_accumulate=True)
            peer.push(ctx, layer.slot_of, ids, tokens)
            peer.combine(ctx, got)
            ctx.check()
            assert torch.equal(got, want)
        # the same calls as a captured graph
        got = init.clone()
        static = got.clone()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            ctx.moe_decode(layer.pool.base, layer.slot_of, x, ids, w, static, defer_accumulate=True)
            peer.push(ctx, layer.slot_of, ids, tokens)
            peer.combine(ctx, static)
        for _ in range(2):
            static.copy_(init)
            graph.replay()
            ctx.check()
            assert torch.equal(static, want)
        graph.reset()
    finally:
        peer.close()
        group.close()


def test_a_flag_nobody_posts_runs_out_of_the_wait_budget():
    import time
    import torch
    tokens = 2
    cfg, layer, x, ids, w = _setup(tokens)
    ctx = aeon_b200.Context(cfg, max_tokens=tokens)
    group = aeon_b200.Group(aeon_b200.group_unique_id(), 0, 1, 0)
    peer = aeon_b200.PeerCombine(group, 0, tokens, cfg.hidden)
    try:
        peer.set_wait_budget(50.0)               # milliseconds
        out = torch.zeros(tokens, cfg.hidden, dtype=torch.float32, device="cuda")
        t0 = time.perf_counter()
        peer.combine(ctx, out)                   # no push was issued: the flag never arrives
        with pytest.raises(aeon_b200.AeonError) as e:
            ctx.check()
        waited = time.perf_counter() - t0
        assert e.value.status == 5               # TIMEOUT
        assert waited < 5.0                      # bounded: a fraction of a second, not a hang
        assert float(out.abs().max().item()) == 0.0     # nothing was added from rows that never came
        # the context is still usable
        ctx.moe_decode(layer.pool.base, layer.slot_of, x, ids, w, out)
        ctx.check()
        assert float(out.abs().max().item()) > 0.0
    finally:
        peer.close()
        group.close()


def test_peer_dispatch_of_one_rank_returns_the_rows_and_routing():
    import torch
    tokens = 6
    cfg, layer, x, ids, w = _setup(tokens)
    ctx = aeon_b200.Context(cfg, max_tokens=tokens)
    group = aeon_b200.Group(aeon_b200.group_unique_id(), 0, 1, 0)
    peer = aeon_b200.PeerCombine(group, 0, tokens, cfg.hidden)
    try:
        for _ in range(3):                       # epochs advance on the device: repeated calls stay in step
            x_all, ids_all, w_all = peer.dispatch(ctx, x, ids, w)
            ctx.check()
            assert torch.equal(x_all.view(torch.int16), x.view(torch.int16))
            assert torch.equal(ids_all, ids) and torch.equal(w_all, w)
        with pytest.raises(aeon_b200.AeonError) as e:       # an odd address cannot take 128-bit copies
            peer.dispatch(ctx, x.view(torch.int16).flatten()[1:1 + 2 * cfg.hidden].view(2, cfg.hidden).view(x.dtype),
                          ids[:2], w[:2])
        assert e.value.status == 1
    finally:
        peer.close()
        group.close()


def _absent_rank_worker(rank, world, unique_id, results):
    """Rank 1 joins the group and the peer buffers but never issues its dispatch: rank 0's wait must
    run out of its budget and report TIMEOUT. The failure is made on the host (a call not made)."""
    import time
    import torch
    torch.cuda.set_device(rank)
    cfg = aeon_b200.preset("baseline")
    tl = 4
    ctx = aeon_b200.Context(cfg, rank, max_tokens=tl * world)
    group = aeon_b200.Group(unique_id, rank, world, rank)
    peer = aeon_b200.PeerCombine(group, rank, tl, cfg.hidden)
    try:
        x = torch.zeros(tl, cfg.hidden, dtype=torch.bfloat16, device="cuda")
        ids = torch.zeros(tl, cfg.top_k, dtype=torch.int32, device="cuda")
        w = torch.zeros(tl, cfg.top_k, dtype=torch.float32, device="cuda")
        if rank == 0:
            peer.set_wait_budget(100.0)
            t0 = time.perf_counter()
            peer.dispatch(ctx, x, ids, w)
            try:
                ctx.check()
                results[rank] = ("no error", time.perf_counter() - t0)
            except aeon_b200.AeonError as e:
                results[rank] = (e.status, time.perf_counter() - t0)
        else:
            results[rank] = ("absent", 0.0)
        torch.cuda.synchronize()
        # both ranks leave between steps, nothing in flight; the peer object is out of step and is destroyed
        group.all_gather_into_tensor(torch.zeros(world, 4, dtype=torch.int32, device="cuda"),
                                     torch.zeros(1, 4, dtype=torch.int32, device="cuda"))
        torch.cuda.synchronize()
    finally:
        peer.close()
        group.close()


def test_a_rank_that_never_dispatches_is_reported_as_timeout():
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    results = mp.Manager().dict()
    mp.spawn(_absent_rank_worker, args=(2, aeon_b200.group_unique_id(), results), nprocs=2, join=True)
    status, waited = results[0]
    assert status == 5, results[0]               # TIMEOUT
    assert waited < 5.0
