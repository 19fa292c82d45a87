"""W2-intermediate tensor-parallel shards on one GPU, ranks simulated one after another — the
method of the reference's own shard gates (tests/test_expert_shard_equivalence.cpp:403-517,
tests/test_w2_shard_equivalence.cpp:138-296): rank r owns intermediate [r*I/tp, (r+1)*I/tp),
i.e. rows of W1/W3 and columns of W2, extracted from the SOURCE layout and swizzled as
matrices of their own; the sum of the shards' outputs must equal the whole expert
(reference bound: 1e-3 relative)."""
import numpy as np
import pytest

import aeon_b200
import gpu_support as gs

pytestmark = pytest.mark.gpu


def shard_payload(cfg, cfg_shard, payload, rank, tp):
    """Full swizzled payload -> the payload of one intermediate-dimension shard."""
    full, part = aeon_b200.expert_layout(cfg), aeon_b200.expert_layout(cfg_shard)
    H, I, G = cfg.hidden, cfg.intermediate, cfg.group_size
    Is = I // tp
    lo, hi = rank * Is, (rank + 1) * Is
    out = np.zeros(part.payload_bytes, dtype=np.uint8)

    def region(buf, off, nbytes, dtype):
        return buf[off:off + nbytes].view(dtype)

    for name in ("w1", "w3"):
        p = region(payload, getattr(full, f"{name}_packed_offset"), full.w13_packed_bytes, np.uint32)
        s = region(payload, getattr(full, f"{name}_scale_offset"), full.w13_scale_bytes, np.uint16)
        src_p, src_s = aeon_b200.swizzle_w4a16(p, s, I, H, cfg.w13_rpw, cfg.w13_lpr, G, inverse=True)
        src_p, src_s = src_p.reshape(I, H // 8)[lo:hi], src_s.reshape(I, H // G)[lo:hi]    # N-shard: rows
        sp, ss = aeon_b200.swizzle_w4a16(src_p, src_s, Is, H, cfg.w13_rpw, cfg.w13_lpr, G)
        region(out, getattr(part, f"{name}_packed_offset"), part.w13_packed_bytes, np.uint32)[:] = sp.ravel()
        region(out, getattr(part, f"{name}_scale_offset"), part.w13_scale_bytes, np.uint16)[:] = ss.ravel()
    p = region(payload, full.w2_packed_offset, full.w2_packed_bytes, np.uint32)
    s = region(payload, full.w2_scale_offset, full.w2_scale_bytes, np.uint16)
    src_p, src_s = aeon_b200.swizzle_w4a16(p, s, H, I, cfg.w2_rpw, cfg.w2_lpr, G, inverse=True)
    src_p = np.ascontiguousarray(src_p.reshape(H, I // 8)[:, lo // 8:hi // 8])             # K-shard: columns
    src_s = np.ascontiguousarray(src_s.reshape(H, I // G)[:, lo // G:hi // G])
    sp, ss = aeon_b200.swizzle_w4a16(src_p, src_s, H, Is, cfg.w2_rpw, cfg.w2_lpr, G)
    region(out, part.w2_packed_offset, part.w2_packed_bytes, np.uint32)[:] = sp.ravel()
    region(out, part.w2_scale_offset, part.w2_scale_bytes, np.uint16)[:] = ss.ravel()
    return out


@pytest.mark.parametrize("tp", [2, 4, 8])
def test_intermediate_shards_sum_to_the_whole_expert(oracle, tp):
    import torch
    cfg = aeon_b200.preset("baseline")
    cfg_shard = cfg.copy(intermediate=cfg.intermediate // tp)
    resident = [10, 11, 12]
    layer = gs.SyntheticLayer(cfg, resident, seed=6, layer=1, with_shared=False)
    la = oracle.layout_args(cfg)
    payloads = [oracle.synth_expert_payload(la, 6, 1, e, layer.scale_table) for e in resident]

    rng = np.random.default_rng(tp)
    T, k = 48, 3
    cfg3, cfg_shard3 = cfg.copy(top_k=k), cfg_shard.copy(top_k=k)
    ids = np.stack([rng.permutation(resident) for _ in range(T)]).astype(np.int32)
    w = rng.random((T, k)).astype(np.float32) + 0.1
    x = gs.torch_bits(gs.activations(cfg, T, seed=12), cfg.act_dtype)
    d_ids, d_w = torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda()

    whole = torch.zeros(T, cfg.hidden, dtype=torch.float32, device="cuda")
    ctx = aeon_b200.Context(cfg3, max_tokens=T)
    ctx.moe_prefill(layer.pool.base, layer.slot_of, x, d_ids, d_w, whole)
    ctx.check()

    total = torch.zeros_like(whole)
    ctx_s = aeon_b200.Context(cfg_shard3, max_tokens=T)
    for rank in range(tp):
        pool = aeon_b200.ExpertPool(cfg_shard, len(resident))
        for slot, payload in enumerate(payloads):
            pool.upload(slot, shard_payload(cfg, cfg_shard, payload, rank, tp))
        partial = torch.zeros_like(whole)
        ctx_s.moe_prefill(pool.base, layer.slot_of, x, d_ids, d_w, partial)
        ctx_s.check()
        total += partial                      # rank order
    want = whole.double().cpu().numpy()
    got = total.double().cpu().numpy()
    s = oracle.compare(want, got)
    print(f"\ntp={tp}: sum of shards vs whole max_abs={s['max_abs']:.3e} rel_l2={s['rel_l2']:.3e}")
    assert s["rel_l2"] <= 1e-3 and s["max_abs"] <= gs.TOL_MAX_ABS
    # the shard of rank 0 alone is far from the whole (the sum is not vacuous)
    assert oracle.compare(want, partial.double().cpu().numpy())["rel_l2"] > 0.1
