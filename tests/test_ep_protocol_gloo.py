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

    def routed(self, x, ids, weights, out, skip_absent):
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


def worker(rank, world, port, results):
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
        w, ids = stack.ep_layer_forward(moe, dist, world, x_local, out_local, x_all, partial, recv)
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

    def routed(self, x, ids, weights, out, skip_absent):
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


@pytest.mark.parametrize("world", [2, 4])
def test_ep_protocol_matches_single_rank(world):
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(worker, args=(world, free_port(), results), nprocs=world, join=True)
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
