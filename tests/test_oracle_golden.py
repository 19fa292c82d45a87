"""The CPU oracle against the golden fixture the reference's own functions produced.

tests/golden/ref_dsv4_golden.json is written by oracle/ref_check.cpp (`make -C oracle golden`),
which links the unmodified reference headers; here the restated oracle has to reproduce those
values bit for bit from the seeds alone, on any machine.
"""
import json
import os

import numpy as np
import pytest

import aeon_b200

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "ref_dsv4_golden.json")


@pytest.fixture(scope="module")
def golden():
    with open(GOLDEN) as f:
        return json.load(f)


@pytest.fixture(scope="module")
def ref_cfg():
    return aeon_b200.preset("ref_dsv4")


def hexfloats(values):
    return np.array([float.fromhex(v) for v in values], dtype=np.float64)


def test_expert_fixture_bit_exact(oracle, golden, ref_cfg):
    la = oracle.layout_args(ref_cfg)
    lay = oracle.layout(la)
    assert lay["payload_bytes"] == 14155776
    n13, n2 = 2048 * 4096, 4096 * 2048
    # One SplitMix64 stream, drawn W1 then W3 then W2 (the reference test's order).
    src = oracle.rng_fill(0x0E7E1217, 0.06, 2 * n13 + n2)
    payload = np.zeros(lay["payload_bytes"], dtype=np.uint8)
    oracle.encode_matrix(la, 0, payload, src[:n13])
    oracle.encode_matrix(la, 2, payload, src[n13:2 * n13])
    oracle.encode_matrix(la, 1, payload, src[2 * n13:])
    assert f"{oracle.fnv1a(payload):016x}" == golden["payload_fnv1a"]

    w2 = oracle.decode_matrix(la, 1, payload)
    assert f"{oracle.fnv1a(w2):016x}" == golden["decoded_w2_fnv1a"]

    x = oracle.rng_fill(0xAC7100, 1.0, 4096)
    y = oracle.expert_ffn(la, payload, x)
    assert f"{oracle.fnv1a(y):016x}" == golden["expert_ffn_fnv1a"]
    np.testing.assert_array_equal(y[:64], hexfloats(golden["expert_ffn_first64"]))


def test_router_fixture_bit_exact(oracle, golden):
    draws = oracle.rng_fill(0x1207E8C0, 1.0, 512)
    logits = (draws[:256] * 4.0).astype(np.float32).astype(np.float64)
    bias = (draws[256:] * 0.5).astype(np.float32).astype(np.float64)
    ids, w, _ = oracle.router_topk(logits[None, :], bias, 6, 1.5, 0)
    assert ids[0].tolist() == golden["router_ids"]
    np.testing.assert_array_equal(w[0], hexfloats(golden["router_weights"]))

    tied = np.zeros((1, 256))
    tied[0, [7, 70, 180, 255]] = 3.0
    ids, _, margin = oracle.router_topk(tied, None, 6, 1.5, 0)
    assert ids[0].tolist() == golden["tie_ids"] == [7, 70, 180, 255, 0, 1]
    assert margin[0] == 0.0

    hids, hw = oracle.router_hash(logits, [200, 3, 77, 150, 9, 31], 1.5, 0)
    assert hids.tolist() == golden["hash_ids"]
    np.testing.assert_array_equal(hw, hexfloats(golden["hash_weights"]))


def test_swiglu_and_dense_fixture_bit_exact(oracle, golden):
    probes = [-40, -12, -5, 0, 5, 12, 40, 3]
    got = [oracle.clamped_swiglu(g, u, 10.0, 0) for g in probes for u in probes]
    np.testing.assert_array_equal(np.array(got), hexfloats(golden["swiglu_probe_grid"]))
    # the asymmetric clamp really is asymmetric: a very negative gate is NOT clamped
    assert oracle.clamped_swiglu(-40, 5, 10.0, 0) != oracle.clamped_swiglu(-40, 5, 10.0, 1)

    I, H = 96, 160
    s = oracle.rng_fill(0x5A4ED00, 1.0, H + 3 * I * H)
    x = s[:H]
    w1 = (s[H:H + I * H] * 0.3).reshape(I, H)
    w3 = (s[H + I * H:H + 2 * I * H] * 0.3).reshape(I, H)
    w2 = (s[H + 2 * I * H:] * 0.3).reshape(H, I)
    y = oracle.dense_ffn_f64(w1, w3, w2, x)
    np.testing.assert_array_equal(y, hexfloats(golden["dense_ffn"]))


def test_hyper_connection_front_and_post_bit_exact(oracle, golden):
    """The steps either side of the MoE FFN (hyper-connection pre-mix with Sinkhorn comb, FFN
    RMSNorm, post expansion) reproduce the reference's own outputs bit for bit; the inputs are
    rebuilt from the reference's generator stream."""
    hidden, hc = 192, 4
    n_mix = hc * (hc + 2)
    total = hc * hidden + n_mix * hc * hidden + n_mix + 3 + hidden + hidden
    u01 = (oracle.rng_u64(0x4C0FFEE, total) >> np.uint64(11)).astype(np.float64) * (1.0 / 9007199254740992.0)
    sym = u01 * 2.0 - 1.0
    at = 0
    def take(n):
        nonlocal at
        at += n
        return slice(at - n, at)
    res_mid = (sym[take(hc * hidden)] * 1.5).reshape(hc, hidden)
    fn = (sym[take(n_mix * hc * hidden)] * 0.05).astype(np.float32).reshape(n_mix, hc * hidden)
    base = (sym[take(n_mix)] * 0.5).astype(np.float32)
    scale = (0.5 + u01[take(3)]).astype(np.float32)
    norm_w = sym[take(hidden)] * 1.0
    layer_out = sym[take(hidden)] * 2.0
    front = oracle.ffn_front(res_mid, fn, base, scale, norm_w, 1e-6)
    got = np.concatenate([front["pre"], front["post"], front["comb"].ravel(), front["ffn_norm"][:16]])
    np.testing.assert_array_equal(got, hexfloats(golden["hc_pre_post_comb_norm16"]))
    post = oracle.hc_post(layer_out, res_mid, front["post"], front["comb"]).ravel()
    np.testing.assert_array_equal(np.concatenate([post[:16], post[-16:]]),
                                  hexfloats(golden["hc_post_first16_last16"]))
    # definitions, independently in numpy
    np.testing.assert_allclose(front["ffn_pre"], front["pre"] @ res_mid, rtol=1e-13)
    np.testing.assert_allclose(post.reshape(hc, hidden),
                               np.outer(front["post"], layer_out) + front["comb"].T @ res_mid, rtol=1e-12)
    assert np.abs(front["comb"].sum(axis=0) - 1).max() < 1e-4 and np.abs(front["comb"].sum(axis=1) - 1).max() < 1e-4
    wrong = oracle.hc_post(layer_out, res_mid, front["post"], front["comb"], transpose_comb=True).ravel()
    assert np.abs(wrong - post).max() > 1e-2


def test_wrong_format_readings_are_far(oracle, ref_cfg):
    """The two plausible-but-wrong decodings differ materially (reference:
    tests/test_v4_expert_oracle.cpp section A: forks > 1e-1 apart)."""
    la = oracle.layout_args(ref_cfg)
    table = np.full(64, 0x2C00, dtype=np.uint16)   # scale 1/16
    payload = oracle.synth_expert_payload(la, 7, 0, 3, table)
    good = oracle.decode_matrix(la, 0, payload, 0)
    unsigned = oracle.decode_matrix(la, 0, payload, 1)
    unpermuted = oracle.decode_matrix(la, 0, payload, 2)
    assert np.abs(good - unsigned).max() > 1e-1
    assert np.abs(good - unpermuted).max() > 1e-1
    assert good.min() == -8 / 16 and good.max() == 7 / 16
