"""Expert parallelism on real GPUs (needs at least two): the stack sharded over 2 (and 4, 8
when present) ranks must route bit-identically to, and agree within the layer tolerance with,
the same stack on one GPU (benchmark configuration 3's acceptance rule)."""
import os
import socket

import numpy as np
import pytest

import aeon_b200
import gpu_support as gs

pytestmark = pytest.mark.gpu

LAYERS, TOKENS = 2, 32


def _worker(rank, world, port, results, peer_combine=False):
    import torch
    import torch.distributed as dist
    from aeon_b200 import stack, synth
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        cfg = aeon_b200.preset("baseline")
        x_bits = synth.normal_bits(np.random.default_rng(11), (LAYERS, TOKENS, cfg.hidden), 1.0, cfg.act_dtype)
        x_all = torch.from_numpy(x_bits.view(np.int16)).view(torch.bfloat16).cuda()
        tl = TOKENS // world
        x_local = x_all[:, rank * tl:(rank + 1) * tl].contiguous()

        ep = stack.MoeStack(cfg, LAYERS, TOKENS, seed=3, device=rank, rank=rank, world=world, dist=dist,
                            peer_combine=peer_combine)
        out_ep = torch.empty(LAYERS, tl, cfg.hidden, dtype=torch.float32, device="cuda")
        routing_ep = [ep.forward_layer(l, x_local[l], out_ep[l], return_routing=True) for l in range(LAYERS)]
        ep.ctx.check()
        again = torch.empty_like(out_ep)
        ep.forward(x_local, again)
        torch.cuda.synchronize()
        reproducible = torch.equal(out_ep, again)
        ep.close()
        del ep
        torch.cuda.empty_cache()

        one = stack.MoeStack(cfg, LAYERS, TOKENS, seed=3, device=rank)
        out_one = torch.empty(LAYERS, TOKENS, cfg.hidden, dtype=torch.float32, device="cuda")
        routing_one = [one.forward_layer(l, x_all[l], out_one[l], return_routing=True) for l in range(LAYERS)]
        one.ctx.check()
        torch.cuda.synchronize()

        ids_equal = all(torch.equal(a[1], b[1]) and torch.equal(a[0], b[0])
                        for a, b in zip(routing_ep, routing_one))
        want = out_one[:, rank * tl:(rank + 1) * tl].double().cpu().numpy()
        got = out_ep.double().cpu().numpy()
        diff = np.abs(want - got)
        rel_l2 = float(np.sqrt((diff ** 2).sum() / (want ** 2).sum()))
        results[rank] = (ids_equal, float(diff.max()), rel_l2, reproducible)
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("peer_combine", [False, True], ids=["nccl-combine", "peer-combine"])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_expert_parallel_matches_single_gpu(world, peer_combine):
    """peer_combine: the combine fused with the accumulate over CUDA-IPC mapped receive buffers
    (plain peer stores + one flag per rank) instead of the all-to-all collective."""
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    results = mp.Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), results, peer_combine), nprocs=world, join=True)
    for rank in range(world):
        ids_equal, max_abs, rel_l2, reproducible = results[rank]
        assert ids_equal, "routing must be bit-identical on every rank"
        assert max_abs <= gs.TOL_MAX_ABS and rel_l2 <= gs.TOL_REL_L2, (rank, max_abs, rel_l2)
        assert reproducible, "a second run at the same world size must give identical bytes"
