"""The steps either side of the MoE FFN on the device (hyper-connection pre-mix + FFN RMSNorm,
post expansion) against the fp64 oracle that is pinned bit-exactly to the reference's
(oracle/ref_check.cpp), and the whole FFN half of a layer composed on the device.

Collected late: the composition builds on the router, the shared expert and the routed path, so
it runs after their own checks."""
import numpy as np
import pytest

import aeon_b200
import gpu_support as gs
from aeon_b200 import stack, synth

pytestmark = pytest.mark.gpu


def hc_inputs(cfg, tokens, seed):
    rng = np.random.default_rng([seed, 0x4C])
    H = cfg.hidden
    res_mid = synth.normal_bits(rng, (tokens, 4, H), 1.0, cfg.act_dtype)
    fn = (rng.standard_normal((24, 4 * H)) * 0.02).astype(np.float32)
    base = (rng.standard_normal(24) * 0.5).astype(np.float32)
    scale = (0.5 + rng.random(3)).astype(np.float32)
    norm = synth.to_bits16(1.0 + 0.1 * rng.standard_normal(H), cfg.act_dtype)
    return res_mid, fn, base, scale, norm


def ulp16(values, dtype):
    """Spacing of the 16-bit type at |values| (bf16: 8 bits of significand, fp16: 11)."""
    bits = 8 if dtype == aeon_b200.BF16 else 11
    return np.maximum(np.abs(values), 1e-30) * 2.0 ** (1 - bits)


@pytest.mark.parametrize("preset,tokens", [("baseline", 5), ("ref_dsv4", 3)])
def test_front_and_post_match_the_oracle(oracle, preset, tokens):
    import torch
    cfg = aeon_b200.preset(preset)
    H = cfg.hidden
    res_bits, fn, base, scale, norm_bits = hc_inputs(cfg, tokens, seed=7)
    ctx = aeon_b200.Context(cfg, max_tokens=tokens)
    d_res = gs.torch_bits(res_bits.reshape(tokens, 4 * H), cfg.act_dtype).reshape(tokens, 4, H)
    d_fn, d_base, d_scale = (torch.from_numpy(a).cuda() for a in (fn, base, scale))
    d_norm = gs.torch_bits(norm_bits, cfg.act_dtype)
    ffn_norm, pre, post, comb = ctx.hc_ffn_front(d_res, d_fn, d_base, d_scale, d_norm)
    moe_out = torch.from_numpy(np.random.default_rng(3).standard_normal((tokens, H)).astype(np.float32) * 5).cuda()
    res_out = ctx.hc_post(moe_out, d_res, post, comb)
    ctx.check()

    res = synth.from_bits16(res_bits, cfg.act_dtype)
    norm_w = synth.from_bits16(norm_bits, cfg.act_dtype)
    got_norm = synth.from_bits16(ffn_norm.view(torch.int16).cpu().numpy().view(np.uint16), cfg.act_dtype)
    got_out = synth.from_bits16(res_out.view(torch.int16).cpu().numpy().view(np.uint16), cfg.act_dtype)
    for t in range(tokens):
        want = oracle.ffn_front(res[t], fn, base, scale, norm_w, 1e-6)
        np.testing.assert_allclose(pre[t].cpu().numpy(), want["pre"], rtol=2e-5, atol=1e-7)
        np.testing.assert_allclose(post[t].cpu().numpy(), want["post"], rtol=2e-5, atol=1e-7)
        np.testing.assert_allclose(comb[t].cpu().numpy().reshape(4, 4), want["comb"], rtol=1e-4, atol=1e-7)
        # 16-bit outputs: within one spacing of the type of the fp64 value
        assert np.all(np.abs(got_norm[t] - want["ffn_norm"]) <= ulp16(want["ffn_norm"], cfg.act_dtype) + 1e-6)
        want_out = oracle.hc_post(moe_out[t].double().cpu().numpy(), res[t], want["post"], want["comb"])
        assert np.all(np.abs(got_out[t] - want_out) <= ulp16(want_out, cfg.act_dtype) + 1e-5)
    # the comb is applied as comb[i][j]: stream i into stream j (the transposed reading is far)
    first = oracle.ffn_front(res[0], fn, base, scale, norm_w, 1e-6)
    wrong = oracle.hc_post(moe_out[0].double().cpu().numpy(), res[0], first["post"], first["comb"],
                           transpose_comb=True)
    assert np.abs(wrong - got_out[0]).max() > 1e-2


def test_ffn_half_of_a_layer_on_the_device(oracle):
    """res_mid -> front -> router -> shared + routed experts -> post, against the oracle fed the
    device's own activation bits and selection (the method of the reference's layer gates,
    src/architecture/deepseek_v4/reference/dsv4_oracle.hpp:2497-2511)."""
    import torch
    cfg = aeon_b200.preset("baseline")
    H, tokens = cfg.hidden, 4
    layer = gs.SyntheticLayer(cfg, None, seed=9, layer=2, with_shared=True)
    res_bits, fn, base, scale, norm_bits = hc_inputs(cfg, tokens, seed=11)
    hc = dict(fn=torch.from_numpy(fn).cuda(), base=torch.from_numpy(base).cuda(),
              scale=torch.from_numpy(scale).cuda(), norm=gs.torch_bits(norm_bits, cfg.act_dtype))
    ctx = aeon_b200.Context(cfg, max_tokens=tokens)
    d_res = gs.torch_bits(res_bits.reshape(tokens, 4 * H), cfg.act_dtype).reshape(tokens, 4, H)
    res_out, ffn_norm, weights, ids, moe_out = stack.layer_body_moe(ctx, layer, hc, d_res)
    ctx.check()

    x_bits = ffn_norm.view(torch.int16).cpu().numpy().view(np.uint16)
    ids_h, w_h = ids.cpu().numpy(), weights.cpu().numpy().astype(np.float64)
    # routing: the device's ids are the oracle's on the device's activation bits
    logits = oracle.router_logits_f32_ordered(layer.gate_bits, cfg.act_dtype, x_bits, cfg.act_dtype)
    want_ids, _, _ = oracle.router_topk(logits.astype(np.float64), None, cfg.top_k, cfg.routed_scaling,
                                        cfg.score_fn)
    np.testing.assert_array_equal(ids_h, want_ids)
    routed = gs.oracle_routed(oracle, layer, x_bits, ids_h, w_h, token_subset=[0, tokens - 1])
    w1, w3, w2 = layer.shared_bits(oracle)
    x = synth.from_bits16(x_bits, cfg.act_dtype)
    res = synth.from_bits16(res_bits, cfg.act_dtype)
    norm_w = synth.from_bits16(norm_bits, cfg.act_dtype)
    got_out = synth.from_bits16(res_out.view(torch.int16).cpu().numpy().view(np.uint16), cfg.act_dtype)
    for t in (0, tokens - 1):
        want_moe = routed[t] + oracle.dense_ffn(w1, w3, w2, cfg.act_dtype, x[t], cfg.swiglu_limit)
        gs.assert_close(oracle, want_moe, moe_out[t].double().cpu().numpy(), f"moe_out token {t}")
        front = oracle.ffn_front(res[t], fn, base, scale, norm_w, 1e-6)
        want_out = oracle.hc_post(want_moe, res[t], front["post"], front["comb"])
        # one spacing of the 16-bit type plus the path's own tolerance scaled by the post gate
        bound = ulp16(want_out, cfg.act_dtype) + gs.TOL_MAX_ABS * np.abs(front["post"]).max()
        assert np.all(np.abs(got_out[t] - want_out) <= bound.reshape(4, H))


def test_checkpoint_to_device_to_residual_out(tmp_path, oracle):
    """The whole chain a deployment runs: a safetensors checkpoint with the reference's tensor
    names -> the two containers (aeon_b200.artifact.convert_checkpoint) -> device weights
    (stack.LoadedLayer) -> residual streams through the FFN half of the layer, against the
    oracle evaluated on the checkpoint's own tensors. Small shapes through the grouped path."""
    import json
    import torch
    from aeon_b200 import artifact
    from test_artifact import source_tensors, write_safetensors
    cfg = aeon_b200.preset("baseline").copy(hidden=1024, intermediate=512, experts=32, top_k=4)
    H, I, tokens = cfg.hidden, cfg.intermediate, 6
    rng = np.random.default_rng(31)
    tensors = {}
    names6 = (("w1", "weight_packed"), ("w1", "weight_scale"), ("w2", "weight_packed"), ("w2", "weight_scale"),
              ("w3", "weight_packed"), ("w3", "weight_scale"))
    for e in range(cfg.experts):
        for (w, t), arr in zip(names6, source_tensors(cfg, 0, e)):
            tensors[f"layers.0.ffn.experts.{e}.{w}.{t}"] = ("I32" if t == "weight_packed" else "F16", arr)
    gate_bits = synth.normal_bits(rng, (cfg.experts, H), 0.05, cfg.act_dtype)
    shared_bits = [synth.normal_bits(rng, shape, 0.02, cfg.act_dtype) for shape in ((I, H), (I, H), (H, I))]
    fn = (rng.standard_normal((24, 4 * H)) * 0.02).astype(np.float32)
    base = (rng.standard_normal(24) * 0.5).astype(np.float32)
    scale = (0.5 + rng.random(3)).astype(np.float32)
    norm_bits = synth.to_bits16(1.0 + 0.1 * rng.standard_normal(H), cfg.act_dtype)
    tensors.update({
        "layers.0.ffn.gate.weight": ("BF16", gate_bits),
        "layers.0.ffn.shared_experts.w1.weight": ("BF16", shared_bits[0]),
        "layers.0.ffn.shared_experts.w3.weight": ("BF16", shared_bits[1]),
        "layers.0.ffn.shared_experts.w2.weight": ("BF16", shared_bits[2]),
        "layers.0.hc_ffn_fn": ("F32", fn), "layers.0.hc_ffn_base": ("F32", base),
        "layers.0.hc_ffn_scale": ("F32", scale), "layers.0.ffn_norm.weight": ("BF16", norm_bits),
    })
    src_dir, out_dir = tmp_path / "hf", tmp_path / "aeon"
    src_dir.mkdir()
    write_safetensors(src_dir / "model.safetensors", tensors)
    artifact.convert_checkpoint(str(src_dir), str(out_dir), cfg)

    layer = stack.LoadedLayer(cfg, str(out_dir), 0)
    ctx = aeon_b200.Context(cfg, max_tokens=tokens)
    res_bits = synth.normal_bits(rng, (tokens, 4, H), 1.0, cfg.act_dtype)
    d_res = gs.torch_bits(res_bits.reshape(tokens, 4 * H), cfg.act_dtype).reshape(tokens, 4, H)
    res_out, ffn_norm, weights, ids, moe_out = stack.layer_body_moe(ctx, layer, layer.hc, d_res, prefill=True)
    ctx.check()

    x_bits = ffn_norm.view(torch.int16).cpu().numpy().view(np.uint16)
    ids_h, w_h = ids.cpu().numpy(), weights.cpu().numpy().astype(np.float64)
    logits = oracle.router_logits_f32_ordered(gate_bits, cfg.act_dtype, x_bits, cfg.act_dtype)
    want_ids, _, _ = oracle.router_topk(logits.astype(np.float64), None, cfg.top_k, cfg.routed_scaling, cfg.score_fn)
    np.testing.assert_array_equal(ids_h, want_ids)
    la = oracle.layout_args(cfg)
    x = synth.from_bits16(x_bits, cfg.act_dtype)
    res = synth.from_bits16(res_bits, cfg.act_dtype)
    norm_w = synth.from_bits16(norm_bits, cfg.act_dtype)
    got_out = synth.from_bits16(res_out.view(torch.int16).cpu().numpy().view(np.uint16), cfg.act_dtype)
    for t in (0, tokens - 1):
        front = oracle.ffn_front(res[t], fn, base, scale, norm_w, 1e-6)
        assert np.all(np.abs(x[t] - front["ffn_norm"]) <= ulp16(front["ffn_norm"], cfg.act_dtype) + 1e-6)
        eo = np.stack([oracle.expert_ffn(la, np.asarray(layer.artifact.expert_data(0, int(e))), x[t], cfg.swiglu_limit)
                       for e in ids_h[t]])
        want_moe = oracle.moe_combine(eo, w_h[t]) + oracle.dense_ffn(shared_bits[0], shared_bits[1], shared_bits[2],
                                                                     cfg.act_dtype, x[t], cfg.swiglu_limit)
        s = oracle.compare(want_moe, moe_out[t].double().cpu().numpy())
        assert s["rel_l2"] <= 2e-3, s                   # grouped path: fp16 operand and hidden roundings
        want_out = oracle.hc_post(moe_out[t].double().cpu().numpy(), res[t], front["post"], front["comb"])
        assert np.all(np.abs(got_out[t] - want_out) <= ulp16(want_out, cfg.act_dtype) + 1e-4)
