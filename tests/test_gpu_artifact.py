"""From the shard-aware expert container to the device: every rank of a tensor-parallel group
reads its byte range of the version-3 file (rank_slice), uploads it into its own pool and runs
the grouped path on it; the ranks' partial outputs, summed in rank order, must equal the whole
expert read from the same file at tp = 1, and the whole must agree with the fp64 oracle on
the payload the file holds. Ranks are simulated one after another on one GPU, the method of
the reference's shard gates (tests/test_expert_shard_equivalence.cpp:403-517)."""
import numpy as np
import pytest

import aeon_b200
import gpu_support as gs
from aeon_b200 import artifact, synth

pytestmark = pytest.mark.gpu


def test_tensor_parallel_ranks_from_a_v3_artifact(tmp_path, oracle):
    import torch
    k, T = 3, 40
    cfg = aeon_b200.preset("baseline").copy(hidden=1024, experts=32, top_k=k)
    used = [4, 9, 30]
    rng = np.random.default_rng(21)
    scale_table = synth.half_normal_table(0.02, 1e-4, 4096, dtype=aeon_b200.F16)
    la = oracle.layout_args(cfg)
    cache = {}

    def source_of(layer, expert):
        # every expert gets real tensors; the three routed ones are distinct
        key = expert if expert in used else -1
        if key not in cache:
            payload = oracle.synth_expert_payload(la, 33, layer, max(key, 0), scale_table)
            cache[key] = aeon_b200.unpack_expert_shards(cfg, 1, payload)
        return cache[key]

    model_dir = str(tmp_path)
    fmt = artifact.write_expert_artifact(model_dir, cfg, 1, source_of, max_tensor_parallel=8)
    art = artifact.ExpertArtifact(model_dir)
    assert (fmt.version, art.format.shard_count) == (3, 8)

    ids = np.stack([rng.permutation(used) for _ in range(T)]).astype(np.int32)
    w = (rng.random((T, k)) + 0.1).astype(np.float32)
    x_bits = gs.activations(cfg, T, seed=5)
    x = gs.torch_bits(x_bits, cfg.act_dtype)
    d_ids, d_w = torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda()
    slot_of = np.full(cfg.experts, -1, dtype=np.int32)
    slot_of[used] = np.arange(len(used))
    d_slot_of = torch.from_numpy(slot_of).cuda()

    def run(tp, rank):
        cfg_r = cfg.copy(intermediate=cfg.intermediate // tp)
        pool = aeon_b200.ExpertPool(cfg_r, len(used))
        for slot, e in enumerate(used):
            pool.upload(slot, art.rank_payload(cfg, 0, e, tp, rank))
        out = torch.zeros(T, cfg.hidden, dtype=torch.float32, device="cuda")
        ctx = aeon_b200.Context(cfg_r, max_tokens=T)
        ctx.moe_prefill(pool.base, d_slot_of, x, d_ids, d_w, out)
        ctx.check()
        return out

    whole = run(1, 0)
    # the whole expert, as stored in the file, against the fp64 oracle on three tokens
    xs = synth.from_bits16(x_bits, cfg.act_dtype)
    for t in (0, 17, T - 1):
        eo = np.stack([oracle.expert_ffn(la, aeon_b200.merge_expert_shards(cfg, 8, np.asarray(art.expert_data(0, int(e)))),
                                         xs[t], cfg.swiglu_limit) for e in ids[t]])
        want = oracle.moe_combine(eo, w[t].astype(np.float64))
        s = oracle.compare(want, whole[t].double().cpu().numpy())
        assert s["rel_l2"] <= 2e-3, s        # operand rounding of the grouped path (fp16 weights and hidden)
    for tp in (2, 8):
        total = torch.zeros_like(whole)
        for rank in range(tp):
            total += run(tp, rank)
        s = oracle.compare(whole.double().cpu().numpy(), total.double().cpu().numpy())
        print(f"\nv3 artifact, tp={tp}: sum of ranks vs whole max_abs={s['max_abs']:.3e} rel_l2={s['rel_l2']:.3e}")
        assert s["rel_l2"] <= 1e-3 and s["max_abs"] <= gs.TOL_MAX_ABS
