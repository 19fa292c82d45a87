"""The expert-parallel protocol (dispatch all-gather -> replicated routing -> local experts ->
combine all-to-all -> rank-order sum) on CPU ranks over gloo, with a small fp64 MoE standing in
for the kernels. What is tested is the host logic of aeon_b200.stack.ep_layer_forward: token
ownership, which rank computes which expert, the layout of the combine exchange and the fixed
summation order. World sizes 2 and 4; the result must equal the single-rank layer bit for bit
in routing and to fp64 rounding in value."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from aeon_b200 import stack

E, K, H, I, T = 8, 2, 16, 12, 8


class TinyMoe:
    """fp64 MoE layer; `owned` is the set of experts resident on this rank."""

    def __init__(self, owned):
        g = torch.Generator().manual_seed(1234)
        self.gate = torch.randn(E, H, generator=g, dtype=torch.float64)
        self.w1 = torch.randn(E, I, H, generator=g, dtype=torch.float64) * 0.3
        self.w3 = torch.randn(E, I, H, generator=g, dtype=torch.float64) * 0.3
        self.w2 = torch.randn(E, H, I, generator=g, dtype=torch.float64) * 0.3
        self.sw = torch.randn(H, H, generator=g, dtype=torch.float64) * 0.1
        self.owned = set(owned)

    def router(self, x):
        scores = torch.sigmoid(x @ self.gate.T)
        w, ids = torch.topk(scores, K, dim=1)
        return w / w.sum(dim=1, keepdim=True), ids.to(torch.int32)

    def shared(self, x, out):
        out.copy_(x @ self.sw.T)

    def routed(self, x, ids, weights, out, skip_absent, overwrite=False):
        if overwrite:
            out.zero_()
        for t in range(x.shape[0]):
            for s in range(K):
                e = int(ids[t, s])
                if e not in self.owned:
                    assert skip_absent
                    continue
                h = torch.nn.functional.silu(self.w1[e] @ x[t]) * (self.w3[e] @ x[t])
                out[t] += weights[t, s] * (self.w2[e] @ h)

    def combine(self, out, recv):
        for r in range(recv.shape[0]):       # rank order
            out += recv[r]


def single_rank(x):
    moe = TinyMoe(range(E))
    w, ids = moe.router(x)
    out = torch.empty(T, H, dtype=torch.float64)
    moe.shared(x, out)
    moe.routed(x, ids, w, out, skip_absent=False)
    return out, ids


def worker(rank, world, port, results, sharded_routing=False):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        x = torch.randn(T, H, generator=torch.Generator().manual_seed(7), dtype=torch.float64)
        tl = T // world
        per = E // world
        moe = TinyMoe(range(rank * per, (rank + 1) * per))
        x_local = x[rank * tl:(rank + 1) * tl].contiguous()
        out_local = torch.empty(tl, H, dtype=torch.float64)
        x_all = torch.empty(T, H, dtype=torch.float64)
        partial = torch.empty(T, H, dtype=torch.float64)
        recv = torch.empty(world, tl, H, dtype=torch.float64)
        # sharded_routing: every rank routes its own tokens and the routing is gathered with the rows
        routing_all = (torch.empty(T, K, dtype=torch.int32), torch.empty(T, K, dtype=torch.float64)) \
            if sharded_routing else None
        w, ids = stack.ep_layer_forward(moe, dist, world, x_local, out_local, x_all, partial, recv,
                                        routing_all=routing_all)
        want, want_ids = single_rank(x)
        ok_ids = torch.equal(ids, want_ids)
        err = (out_local - want[rank * tl:(rank + 1) * tl]).abs().max().item()
        results[rank] = (ok_ids, err, torch.equal(x_all, x))
    finally:
        dist.destroy_process_group()


class TinyShardMoe(TinyMoe):
    """The same layer with only the intermediate slice [lo, hi) of every expert."""

    def __init__(self, lo, hi):
        super().__init__(range(E))
        self.lo, self.hi = lo, hi

    def routed(self, x, ids, weights, out, skip_absent, overwrite=False):
        if overwrite:
            out.zero_()
        lo, hi = self.lo, self.hi
        for t in range(x.shape[0]):
            for s in range(K):
                e = int(ids[t, s])
                h = torch.nn.functional.silu(self.w1[e, lo:hi] @ x[t]) * (self.w3[e, lo:hi] @ x[t])
                out[t] += weights[t, s] * (self.w2[e][:, lo:hi] @ h)


def tp_worker(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        x = torch.randn(T, H, generator=torch.Generator().manual_seed(7), dtype=torch.float64)
        tl = T // world
        per = I // world
        moe = TinyShardMoe(rank * per, (rank + 1) * per)
        out_local = torch.empty(tl, H, dtype=torch.float64)
        partial = torch.empty(T, H, dtype=torch.float64)
        w, ids = stack.tp_layer_forward(moe, dist, world, x, out_local, partial)
        want, want_ids = single_rank(x)
        err = (out_local - want[rank * tl:(rank + 1) * tl]).abs().max().item()
        results[rank] = (torch.equal(ids, want_ids), err)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_tp_protocol_matches_single_rank(world):
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(tp_worker, args=(world, free_port(), results), nprocs=world, join=True)
    for rank in range(world):
        ok_ids, err = results[rank]
        assert ok_ids and err < 1e-12, (rank, err)


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("sharded_routing", [False, True])
@pytest.mark.parametrize("world", [2, 4])
def test_ep_protocol_matches_single_rank(world, sharded_routing):
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(worker, args=(world, free_port(), results, sharded_routing), nprocs=world, join=True)
    assert len(results) == world
    for rank in range(world):
        ok_ids, err, gathered = results[rank]
        assert ok_ids and gathered
        assert err < 1e-12, (rank, err)


def test_combine_buffer_must_be_dense():
    class Dummy:
        def all_gather_into_tensor(self, a, b): a.copy_(b)
        def all_to_all_single(self, a, b): a.copy_(b)
    moe = TinyMoe(range(E))
    x = torch.randn(T, H, dtype=torch.float64)
    recv = torch.empty(1, 2 * T, H, dtype=torch.float64)[:, ::2]
    with pytest.raises(ValueError):
        stack.ep_layer_forward(moe, Dummy(), 1, x, torch.empty(T, H, dtype=torch.float64),
                               torch.empty(T, H, dtype=torch.float64),
                               torch.empty(T, H, dtype=torch.float64), recv)


# ---- pipeline stages x expert parallel under one topology -------------------------------------
LAYERS = 5


class TinyLayer(TinyMoe):
    """TinyMoe with per-layer weights (seeded by the layer id)."""

    def __init__(self, layer, owned):
        super().__init__(owned)
        g = torch.Generator().manual_seed(100 + layer)
        self.gate = torch.randn(E, H, generator=g, dtype=torch.float64)
        self.w1 = torch.randn(E, I, H, generator=g, dtype=torch.float64) * 0.3
        self.w3 = torch.randn(E, I, H, generator=g, dtype=torch.float64) * 0.3
        self.w2 = torch.randn(E, H, I, generator=g, dtype=torch.float64) * 0.3
        self.sw = torch.randn(H, H, generator=g, dtype=torch.float64) * 0.1


def single_rank_stack(x):
    routing = []
    for layer in range(LAYERS):
        moe = TinyLayer(layer, range(E))
        w, ids = moe.router(x)
        out = torch.empty(T, H, dtype=torch.float64)
        moe.shared(x, out)
        moe.routed(x, ids, w, out, skip_absent=False)
        x = x + 0.1 * out
        routing.append(ids)
    return x, routing


def pp_worker(rank, world, pp, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        topo = stack.StageTopology(world, pp, LAYERS)
        # every rank creates every stage's group, in the same order (a collective call)
        groups = [dist.new_group(topo.stage_ranks(s)) for s in range(pp)]
        stage, r = topo.stage_of_rank(rank), topo.rank_in_stage(rank)
        ep = topo.ranks_per_stage
        tl, per = T // ep, E // ep
        x = torch.randn(T, H, generator=torch.Generator().manual_seed(7), dtype=torch.float64)
        carry = x[r * tl:(r + 1) * tl].contiguous() if stage == 0 else torch.empty(tl, H, dtype=torch.float64)
        seen = []

        def run_layers(rows, layers):
            for layer in layers:
                moe = TinyLayer(layer, range(r * per, (r + 1) * per))
                out_local = torch.empty(tl, H, dtype=torch.float64)
                x_all = torch.empty(T, H, dtype=torch.float64)
                partial = torch.empty(T, H, dtype=torch.float64)
                recv = torch.empty(ep, tl, H, dtype=torch.float64)
                _, ids = stack.ep_layer_forward(moe, dist, ep, rows, out_local, x_all, partial, recv,
                                                group=groups[stage])
                rows = rows + 0.1 * out_local
                seen.append((layer, ids))
            return rows

        final = stack.pipeline_forward(topo, dist, rank, carry, run_layers)
        want, want_routing = single_rank_stack(x)
        ok = all(torch.equal(ids, want_routing[layer]) for layer, ids in seen)
        ok = ok and [layer for layer, _ in seen] == list(topo.stage_layers(stage))
        if stage == pp - 1:
            err = (final - want[r * tl:(r + 1) * tl]).abs().max().item()
            ok = ok and err < 1e-12
        else:
            ok = ok and final is None
        results[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,pp", [(2, 2), (4, 2), (4, 4)])
def test_pipeline_stages_compose_with_expert_parallel(world, pp):
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(pp_worker, args=(world, pp, free_port(), results), nprocs=world, join=True)
    assert dict(results) == {rank: True for rank in range(world)}


def test_stage_topology_rules():
    topo = stack.StageTopology(8, 2, 43)
    assert list(topo.stage_layers(0)) == list(range(22)) and list(topo.stage_layers(1)) == list(range(22, 43))
    assert topo.stage_ranks(1) == [4, 5, 6, 7] and topo.peer(2, 1) == 6 and topo.stage_of_rank(5) == 1
    assert topo.stage_of_layer(21) == 0 and topo.stage_of_layer(22) == 1
    for pp in (1, 2, 3, 4):
        t = stack.StageTopology(12, pp, 43)
        counts = [len(t.stage_layers(s)) for s in range(pp)]
        assert sum(counts) == 43 and counts == sorted(counts, reverse=True)
    with pytest.raises(ValueError, match="does not divide"):
        stack.StageTopology(8, 3, 43)
    with pytest.raises(ValueError, match="exceeds"):
        stack.StageTopology(64, 64, 43)
