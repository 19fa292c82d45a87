"""CPU checks of the C ABI: the library loads, exports every declared symbol, the geometry
and the host swizzle agree with the oracle. No compute call is made (there is no GPU here)."""
import ctypes
import os
import re

import numpy as np
import pytest

import aeon_b200

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "aeon_b200.h")).read()
    declared = set(re.findall(r"\b(aeon_b200_[a-z0-9_]+)\s*\(", header))
    assert declared == set(aeon_b200.EXPORTED_SYMBOLS)
    L = aeon_b200.lib()
    for name in declared:
        assert getattr(L, name) is not None
    assert b"sm_100a" in L.aeon_b200_version()


def test_presets_and_geometry_match_oracle(oracle):
    ref = aeon_b200.preset("ref_dsv4")
    assert (ref.hidden, ref.intermediate, ref.experts, ref.top_k, ref.group_size) == (4096, 2048, 256, 6, 32)
    base = aeon_b200.preset("baseline")
    assert (base.hidden, base.top_k, base.group_size, base.act_dtype) == (7168, 8, 128, aeon_b200.BF16)
    for cfg, want in ((ref, 14155776), (base, 22708224)):
        lay = aeon_b200.expert_layout(cfg)
        ol = oracle.layout(oracle.layout_args(cfg))
        assert lay.payload_bytes == ol["payload_bytes"] == want
        assert lay.w1_packed_offset == ol["w1"]["packed_offset"]
        assert lay.w1_scale_offset == ol["w1"]["scale_offset"]
        assert lay.w2_packed_offset == ol["w2"]["packed_offset"]
        assert lay.w2_scale_offset == ol["w2"]["scale_offset"]
        assert lay.w3_packed_offset == ol["w3"]["packed_offset"]
        assert lay.w3_scale_offset == ol["w3"]["scale_offset"]
    with pytest.raises(aeon_b200.AeonError) as e:
        aeon_b200.preset("nope")
    assert e.value.status == 1


def test_config_validation_refuses_bad_shapes():
    L = aeon_b200.lib()
    good = aeon_b200.preset("baseline")
    assert L.aeon_b200_config_validate(ctypes.byref(good)) == 0
    for change in (dict(hidden=7000), dict(group_size=64), dict(top_k=0), dict(experts=250),
                   dict(w13_rpw=8), dict(act_dtype=5), dict(swiglu_limit=0.0)):
        bad = good.copy(**change)
        assert L.aeon_b200_config_validate(ctypes.byref(bad)) == 1, change
        assert len(L.aeon_b200_last_error()) > 0


def make_source(N, K, group, seed):
    """Checkpoint-order words and scales from the reference tests' formulas
    (tests/test_w2_shard_equivalence.cpp:80-87,155-157)."""
    i = np.arange(N * K // 8, dtype=np.uint64)
    words = np.zeros(i.size, dtype=np.uint64)
    for n in range(8):
        words |= ((i * 3 + n * 5 + seed) % 16) << np.uint64(4 * n)
    j = np.arange(N * K // group)
    scales = (2.0 ** -8 * (1 + (j + seed) % 29)).astype(np.float16).view(np.uint16)
    return words.astype(np.uint32).reshape(N, K // 8), scales.reshape(N, K // group)


@pytest.mark.parametrize("N,K,rpw,lpr,group", [
    (2048, 4096, 4, 8, 32), (4096, 2048, 8, 4, 32),      # the reference's W1/W3 and W2
    (256, 7168, 4, 8, 128), (512, 2048, 8, 4, 128),      # benchmark shapes (rows trimmed)
    (1024, 1024, 4, 8, 64), (1024, 1024, 8, 4, 64),
])
def test_swizzle_round_trip_and_address_identity(oracle, N, K, rpw, lpr, group):
    src_p, src_s = make_source(N, K, group, seed=11)
    swz_p, swz_s = aeon_b200.swizzle_w4a16(src_p, src_s, N, K, rpw, lpr, group)
    back_p, back_s = aeon_b200.swizzle_w4a16(swz_p, swz_s, N, K, rpw, lpr, group, inverse=True)
    np.testing.assert_array_equal(back_p, src_p)
    np.testing.assert_array_equal(back_s, src_s)
    assert not np.array_equal(swz_p, src_p)

    # Nibble-by-nibble identity against the oracle's independent address arithmetic.
    if (rpw, lpr) == (4, 8):
        la = oracle_args(oracle, K, N, group)
        kind = 0
    else:
        la = oracle_args(oracle, N, K, group)
        kind = 1
    rng = np.random.default_rng(5)
    flat_p = swz_p.ravel()
    flat_s = swz_s.ravel()
    for row, col in zip(rng.integers(0, N, 400), rng.integers(0, K, 400)):
        slot, word, nib = oracle.swizzled_address(la, kind, int(row), int(col))
        got = (int(flat_p[word]) >> (4 * nib)) & 0xF
        want = (int(src_p[row, col // 8]) >> (4 * (col % 8))) & 0xF
        assert got == want
        assert flat_s[slot] == src_s[row, col // group]


def oracle_args(oracle, hidden, intermediate, group):
    return oracle.LayoutArgs(hidden, intermediate, group, 4, 8, 8, 4)


def test_swizzle_matches_oracle_whole_matrix(oracle):
    cfg = aeon_b200.preset("baseline")
    la = oracle.LayoutArgs(1024, 1024, 128, 4, 8, 8, 4)
    lay = oracle.layout(la)
    for kind, (rpw, lpr) in ((0, (4, 8)), (1, (8, 4))):
        src_p, src_s = make_source(1024, 1024, 128, seed=3 + kind)
        payload = np.zeros(lay["payload_bytes"], dtype=np.uint8)
        oracle.swizzle_from_source(la, kind, src_p, src_s, payload)
        swz_p, swz_s = aeon_b200.swizzle_w4a16(src_p, src_s, 1024, 1024, rpw, lpr, 128)
        name = ("w1", "w2")[kind]
        po, so = lay[name]["packed_offset"], lay[name]["scale_offset"]
        np.testing.assert_array_equal(payload[po:po + swz_p.nbytes].view(np.uint32), swz_p.ravel())
        np.testing.assert_array_equal(payload[so:so + swz_s.nbytes].view(np.uint16), swz_s.ravel())
    assert cfg.group_size == 128


def test_swizzle_refuses_bad_arguments():
    src_p, src_s = make_source(64, 1024, 32, seed=1)
    with pytest.raises(aeon_b200.AeonError):
        aeon_b200.swizzle_w4a16(src_p, src_s, 64, 1024, 4, 4, 32)      # rpw*lpr != 32
    with pytest.raises(aeon_b200.AeonError):
        aeon_b200.swizzle_w4a16(src_p, src_s, 62, 1024, 4, 8, 32)      # N % rpw
    with pytest.raises(aeon_b200.AeonError):
        aeon_b200.swizzle_w4a16(src_p, src_s, 64, 1024, 16, 2, 128)    # lanes < atoms per group


def test_no_device_is_an_error_not_a_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    with pytest.raises(aeon_b200.AeonError) as e:
        aeon_b200.Context(aeon_b200.preset("baseline"))
    assert e.value.status == 3
