"""The multi-GPU group entry points of the C ABI (aeon_b200_group_* / ep_dispatch / ep_exchange /
tp_reduce / pp_send / pp_recv) on two or more GPUs, with no torch.distributed anywhere: the
parent makes the 128-byte id and hands it to the ranks as an argument, the way a C++ host would
pass it over its own channel. Every collective is checked against values computed from the
ranks' seeds; the same calls are then captured in a CUDA graph, replayed, and the group is
left in the order the library documents (graph first, then the group)."""
import numpy as np
import pytest

import aeon_b200

pytestmark = pytest.mark.gpu

TL, H = 6, 512          # rows per rank, row width


def _rows(rank, world):
    """This rank's fp32 partial rows for every token of the batch: value = rank, row, column."""
    import torch
    r = torch.arange(world * TL, dtype=torch.float32).reshape(-1, 1)
    c = torch.arange(H, dtype=torch.float32).reshape(1, -1)
    return (1000.0 * (rank + 1) + r + c / 1024.0).cuda()


def _worker(rank, world, unique_id, results):
    import torch
    torch.cuda.set_device(rank)
    g = aeon_b200.Group(unique_id, rank, world, rank)
    try:
        ok = {}
        x_local = torch.full((TL, H), float(rank + 1), dtype=torch.bfloat16, device="cuda")
        x_all = torch.zeros(world * TL, H, dtype=torch.bfloat16, device="cuda")
        partial = _rows(rank, world)
        recv = torch.zeros(world, TL, H, dtype=torch.float32, device="cuda")
        out_local = torch.zeros(TL, H, dtype=torch.float32, device="cuda")

        def step():
            g.ep_dispatch(x_local, x_all)
            g.ep_exchange(partial, recv.view(-1, H))
            g.tp_reduce(partial, out_local)

        step()
        torch.cuda.synchronize()
        want_all = torch.cat([torch.full((TL, H), float(r + 1), dtype=torch.bfloat16) for r in range(world)])
        ok["dispatch"] = torch.equal(x_all.cpu(), want_all)
        mine = slice(rank * TL, (rank + 1) * TL)
        want_recv = torch.stack([_rows(s, world)[mine] for s in range(world)])
        ok["exchange"] = torch.equal(recv, want_recv)
        want_sum = want_recv.double().sum(dim=0)
        ok["reduce"] = (out_local.double() - want_sum).abs().max().item() <= 1e-3

        # dispatch with the routing each rank made for its own tokens (one grouped call)
        ids_local = torch.full((TL, 8), rank, dtype=torch.int32, device="cuda")
        w_local = torch.full((TL, 8), rank + 0.5, dtype=torch.float32, device="cuda")
        ids_all = torch.zeros(world * TL, 8, dtype=torch.int32, device="cuda")
        w_all = torch.zeros(world * TL, 8, dtype=torch.float32, device="cuda")
        x_all.zero_()
        g.ep_dispatch_routed(x_local, x_all, ids_local, w_local, ids_all, w_all)
        torch.cuda.synchronize()
        owner = torch.arange(world).repeat_interleave(TL).reshape(-1, 1).expand(-1, 8)
        ok["dispatch_routed"] = (torch.equal(x_all.cpu(), want_all) and torch.equal(ids_all.cpu(), owner.int())
                                 and torch.equal(w_all.cpu(), owner.float() + 0.5))

        # pipeline hand-off: a ring of byte copies, rank r -> r + 1
        carry = torch.full((TL, H), float(rank), dtype=torch.bfloat16, device="cuda")
        got = torch.zeros_like(carry)
        nxt, prv = (rank + 1) % world, (rank - 1) % world
        if rank % 2 == 0:
            g.send(carry, nxt)
            g.recv(got, prv)
        else:
            g.recv(got, prv)
            g.send(carry, nxt)
        torch.cuda.synchronize()
        ok["handoff"] = bool((got == float(prv)).all().item())

        # the same collectives as a captured graph, replayed on fresh outputs
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step()
        x_all.zero_(); recv.zero_(); out_local.zero_()
        graph.replay()
        torch.cuda.synchronize()
        ok["graph"] = (torch.equal(x_all.cpu(), want_all) and torch.equal(recv, want_recv)
                       and (out_local.double() - want_sum).abs().max().item() <= 1e-3)
        graph.reset()                       # a live graph keeps NCCL's captured plan referenced
        torch.cuda.synchronize()
        results[rank] = ok
    finally:
        g.close()


@pytest.mark.parametrize("world", [2, 4])
def test_group_collectives_through_the_c_abi(world):
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    results = mp.Manager().dict()
    mp.spawn(_worker, args=(world, aeon_b200.group_unique_id(), results), nprocs=world, join=True)
    for rank in range(world):
        assert all(results[rank].values()), (rank, dict(results[rank]))


def test_group_refuses_bad_arguments():
    with pytest.raises(aeon_b200.AeonError) as e:
        aeon_b200.Group(b"short", 0, 1, 0)
    assert e.value.status == 1
    with pytest.raises(aeon_b200.AeonError) as e:
        aeon_b200.Group(aeon_b200.group_unique_id(), 3, 2, 0)        # rank outside [0, world)
    assert e.value.status == 1
