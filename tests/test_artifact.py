"""CPU checks of the artifact files either side of the path: the expert container in the
reference's version 2 and in the shard-aware version 3 it plans
(plans-and-docs/execution/active/MULTI_GPU_EXECUTION_PLAN.md:151-181 — "rank slices are
contiguous, 4 KiB-aligned and disjoint, and together cover the payload exactly; v2 still loads
as D = 1; per-shard unswizzle round-trip is bit-exact and reassembling the shards reproduces the
source tensor exactly"), and the dense container that carries the gate and the shared expert."""
import json
import os
import struct

import numpy as np
import pytest

import aeon_b200
from aeon_b200 import artifact


def small_cfg(**changes):
    # the smallest shapes the configuration rules admit with 8 intermediate shards
    return aeon_b200.preset("baseline").copy(hidden=256, intermediate=2048, experts=32, top_k=4, **changes)


def source_tensors(cfg, layer, expert):
    """Seeded checkpoint-order tensors (words of eight nibbles, fp16 scale bits)."""
    rng = np.random.default_rng([layer, expert, cfg.group_size])
    out = []
    for shape, dtype in zip(aeon_b200.source_shapes(cfg), (np.uint32, np.uint16) * 3):
        if dtype == np.uint32:
            out.append(rng.integers(0, 2 ** 32, size=shape, dtype=np.uint64).astype(np.uint32))
        else:
            out.append(np.abs(rng.standard_normal(shape) * 0.02 + 1e-4).astype(np.float16).view(np.uint16))
    return out


def slice_source(cfg, src, first, count):
    G = cfg.group_size
    rows = slice(first, first + count)
    return [src[0][rows], src[1][rows], src[2][:, first // 8:(first + count) // 8],
            src[3][:, first // G:(first + count) // G], src[4][rows], src[5][rows]]


@pytest.mark.parametrize("group", [32, 128])
def test_one_shard_is_the_v2_payload_and_shards_round_trip(group, oracle):
    cfg = small_cfg(group_size=group)
    src = source_tensors(cfg, 0, 0)
    lay = aeon_b200.expert_layout(cfg)
    whole = aeon_b200.pack_expert_shards(cfg, 1, src)
    assert whole.size == lay.payload_bytes
    # region by region the same bytes as the per-matrix swizzle, and as the oracle's own
    # restatement of the reference swizzle
    la = oracle.layout_args(cfg)
    want = np.zeros(lay.payload_bytes, dtype=np.uint8)
    for kind, (p, s) in enumerate(((src[0], src[1]), (src[2], src[3]), (src[4], src[5]))):
        oracle.swizzle_from_source(la, kind, p, s, want)
    assert np.array_equal(whole, want)
    for shards in (2, 4, 8):
        sharded = aeon_b200.pack_expert_shards(cfg, shards, src)
        assert sharded.size == shards * aeon_b200.expert_shard_bytes(cfg, shards)
        back = aeon_b200.unpack_expert_shards(cfg, shards, sharded)
        assert all(np.array_equal(a, b) for a, b in zip(src, back))
        # W1/W3 shards are row-block ranges of the whole matrix: their packed regions,
        # concatenated, are the whole matrix's packed region
        unit = aeon_b200.expert_layout(cfg.copy(intermediate=cfg.intermediate // shards))
        sb = aeon_b200.expert_shard_bytes(cfg, shards)
        for name in ("w1", "w3"):
            off = getattr(unit, f"{name}_packed_offset")
            cat = np.concatenate([sharded[s * sb + off:s * sb + off + unit.w13_packed_bytes] for s in range(shards)])
            woff = getattr(lay, f"{name}_packed_offset")
            assert np.array_equal(cat, whole[woff:woff + lay.w13_packed_bytes])


def test_shard_is_decoded_by_the_oracle_as_the_slice_of_the_whole(oracle):
    """The oracle's independent swizzled reader, pointed at one shard, sees exactly the rows
    (W1, W3) and columns (W2) of the whole expert; the shards' FFN partials sum to the whole
    expert's output (the shard gates of tests/test_expert_shard_equivalence.cpp:403-517)."""
    cfg = small_cfg()
    shards = 4
    src = source_tensors(cfg, 1, 5)
    whole = aeon_b200.pack_expert_shards(cfg, 1, src)
    sharded = aeon_b200.pack_expert_shards(cfg, shards, src)
    cfg_s = cfg.copy(intermediate=cfg.intermediate // shards)
    la, la_s = oracle.layout_args(cfg), oracle.layout_args(cfg_s)
    sb = aeon_b200.expert_shard_bytes(cfg, shards)
    Is = cfg_s.intermediate
    w = [oracle.decode_matrix(la, kind, whole) for kind in range(3)]      # W1, W2, W3
    x = np.random.default_rng(3).standard_normal(cfg.hidden)
    total = np.zeros(cfg.hidden)
    for s in range(shards):
        piece = np.ascontiguousarray(sharded[s * sb:(s + 1) * sb])
        assert np.array_equal(oracle.decode_matrix(la_s, 0, piece), w[0][s * Is:(s + 1) * Is])
        assert np.array_equal(oracle.decode_matrix(la_s, 2, piece), w[2][s * Is:(s + 1) * Is])
        assert np.array_equal(oracle.decode_matrix(la_s, 1, piece), w[1][:, s * Is:(s + 1) * Is])
        total += oracle.expert_ffn(la_s, piece, x)
    want = oracle.expert_ffn(la, whole, x)
    stats = oracle.compare(want, total)
    assert stats["rel_l2"] < 1e-12


def test_rank_slices_are_contiguous_aligned_disjoint_and_cover_the_payload():
    cfg = small_cfg()
    for shards in (1, 2, 4, 8):
        sb = aeon_b200.expert_shard_bytes(cfg, shards)
        assert sb % 4096 == 0
        for tp in (1, 2, 4, 8):
            if shards % tp:
                with pytest.raises(aeon_b200.AeonError) as e:
                    aeon_b200.expert_rank_slice(cfg, shards, tp, 0)
                assert e.value.status == 1 and "does not divide" in str(e.value)
                continue
            cursor = 0
            for rank in range(tp):
                off, length = aeon_b200.expert_rank_slice(cfg, shards, tp, rank)
                assert off == cursor and off % 4096 == 0 and length == shards * sb // tp
                cursor += length
            assert cursor == shards * sb
            with pytest.raises(aeon_b200.AeonError) as e:
                aeon_b200.expert_rank_slice(cfg, shards, tp, tp)
            assert e.value.status == 4
    with pytest.raises(aeon_b200.AeonError):
        aeon_b200.expert_shard_bytes(cfg, 3)            # 2048 / 3 is not whole
    with pytest.raises(aeon_b200.AeonError):
        aeon_b200.expert_shard_bytes(cfg, 16)           # shards of 128 columns are too narrow


def test_sharding_adds_no_padding_at_the_model_shapes():
    """Each region of a shard stays a multiple of 4 KiB at the reference's and the benchmark's
    shapes, so a version-3 payload is exactly as large as the version-2 one."""
    for name, want in (("ref_dsv4", 14155776), ("baseline", 22708224)):
        cfg = aeon_b200.preset(name)
        for shards in (1, 2, 4, 8):
            assert shards * aeon_b200.expert_shard_bytes(cfg, shards) == want


def test_rank_slice_merges_into_the_payload_of_the_rank():
    cfg = small_cfg()
    src = source_tensors(cfg, 0, 9)
    sharded = aeon_b200.pack_expert_shards(cfg, 8, src)
    for tp in (1, 2, 4, 8):
        cfg_r = cfg.copy(intermediate=cfg.intermediate // tp)
        for rank in range(tp):
            off, length = aeon_b200.expert_rank_slice(cfg, 8, tp, rank)
            merged = aeon_b200.merge_expert_shards(cfg_r, 8 // tp, sharded[off:off + length])
            direct = aeon_b200.pack_expert_shards(
                cfg_r, 1, slice_source(cfg, src, rank * cfg_r.intermediate, cfg_r.intermediate))
            assert np.array_equal(merged, direct), (tp, rank)


@pytest.mark.parametrize("max_tp", [1, 8])
def test_expert_container_files(tmp_path, max_tp):
    cfg = small_cfg()
    layers = 2
    source_of = lambda layer, expert: source_tensors(cfg, layer, expert)
    fmt = artifact.write_expert_artifact(str(tmp_path), cfg, layers, source_of, max_tensor_parallel=max_tp)
    assert fmt.version == (3 if max_tp > 1 else 2)
    # header bytes as the reference packs them ("<12sIIIQ", scripts/convert_safetensors_to_aeon.py:310)
    raw = open(tmp_path / artifact.INDEX_FILENAME, "rb").read()
    magic, version, n_layers, n_experts, payload = struct.unpack_from("<12sIIIQ", raw, 0)
    assert (magic, version, n_layers, n_experts, payload) == (
        b"AEON_EXPERTS", fmt.version, layers, cfg.experts, max_tp * aeon_b200.expert_shard_bytes(cfg, max_tp))
    assert len(raw) == (32 if max_tp == 1 else 48) + 16 * layers * cfg.experts
    manifest = json.load(open(tmp_path / artifact.MANIFEST_FILENAME))
    assert manifest["max_tensor_parallel"] == max_tp and manifest["artifact"]["expert_shard_count"] == max_tp

    art = artifact.ExpertArtifact(str(tmp_path), expected_payload_bytes=payload)
    assert (art.format.shard_count, art.format.shard_bytes) == (max_tp, payload // max_tp)
    off, length = art.expert_location(1, 7)
    assert off == (cfg.experts + 7) * payload and length == payload
    want = aeon_b200.pack_expert_shards(cfg, max_tp, source_of(1, 7))
    assert np.array_equal(np.asarray(art.expert_data(1, 7)), want)
    assert artifact.verify_conversion(str(tmp_path), cfg, source_of, sample=[(0, 0), (1, 31)]) == 2
    with pytest.raises(IndexError):
        art.expert_location(2, 0)
    with pytest.raises(ValueError):
        artifact.ExpertArtifact(str(tmp_path), expected_payload_bytes=payload + 4096)

    # rank slices of one expert tile the expert's byte range; what a rank uploads equals the
    # payload built directly from its slice of the source
    for tp in (1, 2, 4, 8):
        if max_tp % tp:
            with pytest.raises(ValueError):
                art.rank_slice(0, 3, tp, 0)
            continue
        base, _ = art.expert_location(0, 3)
        cursor = base
        for rank in range(tp):
            o, n = art.rank_slice(0, 3, tp, rank)
            assert o == cursor and o % 4096 == 0
            cursor += n
        assert cursor == base + payload
        cfg_r = cfg.copy(intermediate=cfg.intermediate // tp)
        got = art.rank_payload(cfg, 0, 3, tp, tp - 1)
        direct = aeon_b200.pack_expert_shards(
            cfg_r, 1, slice_source(cfg, source_of(0, 3), (tp - 1) * cfg_r.intermediate, cfg_r.intermediate))
        assert np.array_equal(got, direct)


def test_reshard_v2_artifact_into_v3(tmp_path):
    cfg = small_cfg()
    source_of = lambda layer, expert: source_tensors(cfg, layer, expert)
    v2, v3 = str(tmp_path / "v2"), str(tmp_path / "v3")
    artifact.write_expert_artifact(v2, cfg, 1, source_of, max_tensor_parallel=1)
    fmt = artifact.reshard_expert_artifact(v2, v3, cfg, 4)
    assert (fmt.version, fmt.shard_count) == (3, 4)
    assert artifact.verify_conversion(v3, cfg, source_of, sample=[(0, 0), (0, 17)]) == 2
    with pytest.raises(ValueError, match="shapes do not match"):
        artifact.reshard_expert_artifact(v2, str(tmp_path / "bad"), cfg.copy(hidden=512), 4)


def test_reshard_command_line_round_trip(tmp_path, monkeypatch):
    cfg = small_cfg()
    source_of = lambda layer, expert: source_tensors(cfg, layer, expert)
    v2, v3, again = str(tmp_path / "v2"), str(tmp_path / "v3"), str(tmp_path / "again")
    artifact.write_expert_artifact(v2, cfg, 1, source_of, max_tensor_parallel=1)
    monkeypatch.setattr(aeon_b200, "preset", lambda name: cfg)
    assert artifact._main([v2, v3, "--max-tensor-parallel", "8"]) == 0
    assert artifact._main([v3, again, "--max-tensor-parallel", "1"]) == 0
    for name in (artifact.INDEX_FILENAME, artifact.EXPERTS_FILENAME):
        assert open(os.path.join(v2, name), "rb").read() == open(os.path.join(again, name), "rb").read()


def test_corrupt_or_truncated_expert_container_is_refused(tmp_path):
    cfg = small_cfg()
    source_of = lambda layer, expert: source_tensors(cfg, layer, expert)
    artifact.write_expert_artifact(str(tmp_path), cfg, 1, source_of, max_tensor_parallel=2)
    index = tmp_path / artifact.INDEX_FILENAME
    good = index.read_bytes()
    # flipped payload byte: the round-trip verification notices
    data = tmp_path / artifact.EXPERTS_FILENAME
    blob = bytearray(data.read_bytes())
    blob[12345] ^= 0x10
    data.write_bytes(bytes(blob))
    with pytest.raises(ValueError, match="does not round-trip"):
        artifact.verify_conversion(str(tmp_path), cfg, source_of, sample=[(0, 0)])
    for bad, message in (
        (b"AEON_EXPERTZ" + good[12:], "magic"),
        (good[:40], "too small"),
        (good[:-8], "incomplete"),
        (good[:12] + struct.pack("<I", 4) + good[16:], "unsupported version"),
        (good[:32] + struct.pack("<IIQ", 3, 0, struct.unpack_from("<Q", good, 40)[0]) + good[48:], "shard_count"),
        (good[:48] + struct.pack("<QQ", 100, struct.unpack_from("<Q", good, 56)[0]) + good[64:], "invalid payload entry"),
    ):
        index.write_bytes(bad)
        with pytest.raises(ValueError, match=message):
            artifact.ExpertArtifact(str(tmp_path))
    index.write_bytes(good)
    data.write_bytes(bytes(blob[:-4096]))
    with pytest.raises(ValueError, match="outside the experts file"):
        artifact.ExpertArtifact(str(tmp_path))


def test_dense_container_round_trip_and_refusals(tmp_path):
    cfg = small_cfg()
    rng = np.random.default_rng(0)
    names = artifact.moe_layer_tensor_names(3)
    tensors = [
        (names["gate"], "BF16", rng.integers(0, 2 ** 16, size=(cfg.experts, cfg.hidden), dtype=np.uint16)),
        (names["gate_bias"], "F32", rng.standard_normal(cfg.experts).astype(np.float32)),
        (names["shared_w1"], "BF16", rng.integers(0, 2 ** 16, size=(cfg.intermediate, cfg.hidden), dtype=np.uint16)),
        (names["shared_w2"], "BF16", rng.integers(0, 2 ** 16, size=(cfg.hidden, cfg.intermediate), dtype=np.uint16)),
        (names["shared_w3"], "BF16", rng.integers(0, 2 ** 16, size=(cfg.intermediate, cfg.hidden), dtype=np.uint16)),
        (artifact.moe_layer_tensor_names(0, hash_layer=True)["tid2eid"], "I64",
         rng.integers(0, cfg.experts, size=(64, cfg.top_k), dtype=np.int64)),
    ]
    path = str(tmp_path / artifact.DENSE_FILENAME)
    artifact.write_dense_container(path, tensors)
    raw = open(path, "rb").read()
    magic, version, count, dir_len = struct.unpack_from("<12sIIQ", raw, 0)
    assert (magic, version, count) == (b"AEON_DENSE\x00\x00", 1, len(tensors))
    data_start = (28 + dir_len + 4095) // 4096 * 4096
    assert raw[data_start:data_start + 8] == tensors[0][2].tobytes()[:8]
    dense = artifact.DenseContainer(path)
    assert set(dense.names()) == {t[0] for t in tensors}
    for name, dtype, array in tensors:
        assert dense.has_tensor(name) and dense.dtype_of(name) == dtype
        assert np.array_equal(dense.get_tensor(name), array)
    assert not dense.has_tensor("layers.3.ffn.gate.missing")
    with pytest.raises(KeyError):
        dense.get_tensor("layers.3.ffn.gate.missing")
    for bad, message in (
        (b"AEON_DENSF\x00\x00" + raw[12:], "magic"),
        (raw[:12] + struct.pack("<I", 7) + raw[16:], "version"),
        (raw[:16] + struct.pack("<I", count + 1) + raw[20:], "count"),
        (raw[:20] + struct.pack("<Q", len(raw)) + raw[28:], "Directory length"),
        (raw[:data_start + 100], "exceeds payload"),
    ):
        open(path, "wb").write(bad)
        with pytest.raises(ValueError, match=message):
            artifact.DenseContainer(path)


def test_shard_packing_properties_over_random_shapes():
    """Random legal shapes: packing into D shards then unpacking is the identity, every rank's
    merged slice equals the payload packed from its slice of the source, and the payload bytes of
    different ranks never overlap."""
    from hypothesis import given, settings, strategies as st

    @settings(max_examples=25, deadline=None)
    @given(hidden=st.sampled_from([256, 512, 768]), inter_blocks=st.sampled_from([1, 2, 4, 8]),
           group=st.sampled_from([32, 128]), shards=st.sampled_from([1, 2, 4, 8]),
           tp=st.sampled_from([1, 2, 4, 8]), seed=st.integers(0, 2 ** 16))
    def run(hidden, inter_blocks, group, shards, tp, seed):
        cfg = aeon_b200.preset("baseline").copy(hidden=hidden, intermediate=256 * inter_blocks, experts=32,
                                                top_k=4, group_size=group)
        if inter_blocks % shards:
            with pytest.raises(aeon_b200.AeonError):
                aeon_b200.expert_shard_bytes(cfg, shards)
            return
        rng = np.random.default_rng(seed)
        src = [rng.integers(0, 2 ** 32, size=shape, dtype=np.uint64).astype(np.uint32) if i % 2 == 0
               else rng.integers(0, 2 ** 16, size=shape, dtype=np.uint32).astype(np.uint16)
               for i, shape in enumerate(aeon_b200.source_shapes(cfg))]
        payload = aeon_b200.pack_expert_shards(cfg, shards, src)
        back = aeon_b200.unpack_expert_shards(cfg, shards, payload)
        assert all(np.array_equal(a, b) for a, b in zip(src, back))
        if shards % tp:
            with pytest.raises(aeon_b200.AeonError):
                aeon_b200.expert_rank_slice(cfg, shards, tp, 0)
            return
        cfg_r = cfg.copy(intermediate=cfg.intermediate // tp)
        covered = np.zeros(payload.size, dtype=np.uint8)
        for rank in range(tp):
            off, length = aeon_b200.expert_rank_slice(cfg, shards, tp, rank)
            covered[off:off + length] += 1
            merged = aeon_b200.merge_expert_shards(cfg_r, shards // tp, payload[off:off + length])
            direct = aeon_b200.pack_expert_shards(
                cfg_r, 1, slice_source(cfg, src, rank * cfg_r.intermediate, cfg_r.intermediate))
            assert np.array_equal(merged, direct)
        assert np.all(covered == 1)

    run()


def write_safetensors(path, tensors):
    """Minimal writer of the safetensors layout: u64 header length, JSON header, raw bytes."""
    header, blobs, offset = {}, [], 0
    for name, (dtype, array) in tensors.items():
        raw = np.ascontiguousarray(array).tobytes()
        header[name] = {"dtype": dtype, "shape": list(array.shape), "data_offsets": [offset, offset + len(raw)]}
        blobs.append(raw)
        offset += len(raw)
    head = json.dumps(header).encode("utf-8")
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(head)))
        f.write(head)
        for raw in blobs:
            f.write(raw)


def test_safetensors_checkpoint_to_containers(tmp_path):
    """A two-shard checkpoint with the reference's tensor names becomes the dense container, the
    expert container (here shard-aware, D = 2) and a manifest; everything reads back bit-exactly
    (the conversion the reference's scripts/convert_safetensors_to_aeon.py performs for version 2)."""
    cfg = aeon_b200.preset("baseline").copy(hidden=256, intermediate=512, experts=32, top_k=4)
    layers = 2
    src_dir, out_dir = tmp_path / "hf", tmp_path / "aeon"
    src_dir.mkdir()
    rng = np.random.default_rng(17)
    shards = [{}, {}]
    weight_map = {}
    sources = {}
    names6 = (("w1", "weight_packed"), ("w1", "weight_scale"), ("w2", "weight_packed"), ("w2", "weight_scale"),
              ("w3", "weight_packed"), ("w3", "weight_scale"))
    for layer in range(layers):
        for expert in range(cfg.experts):
            src = source_tensors(cfg, layer, expert)
            sources[(layer, expert)] = src
            for (w, t), arr in zip(names6, src):
                name = f"layers.{layer}.ffn.experts.{expert}.{w}.{t}"
                shards[layer][name] = ("I32" if t == "weight_packed" else "F16", arr)
                weight_map[name] = f"model-{layer}.safetensors"
        dense = {
            f"layers.{layer}.ffn.gate.weight": ("BF16", rng.integers(0, 2 ** 16, (cfg.experts, cfg.hidden), dtype=np.uint16)),
            f"layers.{layer}.ffn.gate.bias": ("F32", rng.standard_normal(cfg.experts).astype(np.float32)),
            f"layers.{layer}.ffn.shared_experts.w1.weight": ("BF16", rng.integers(0, 2 ** 16, (cfg.intermediate, cfg.hidden), dtype=np.uint16)),
            f"layers.{layer}.ffn_norm.weight": ("BF16", rng.integers(0, 2 ** 16, (cfg.hidden,), dtype=np.uint16)),
        }
        for name, value in dense.items():
            shards[layer][name] = value
            weight_map[name] = f"model-{layer}.safetensors"
    shards[0]["embed.weight"] = ("BF16", rng.integers(0, 2 ** 16, (64, cfg.hidden), dtype=np.uint16))
    weight_map["embed.weight"] = "model-0.safetensors"
    for i, tensors in enumerate(shards):
        write_safetensors(src_dir / f"model-{i}.safetensors", tensors)
    (src_dir / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    (src_dir / "config.json").write_text(json.dumps({"model_type": "deepseek_v4"}))

    fmt = artifact.convert_checkpoint(str(src_dir), str(out_dir), cfg, max_tensor_parallel=2)
    assert (fmt.version, fmt.num_layers, fmt.shard_count) == (3, layers, 2)
    art = artifact.ExpertArtifact(str(out_dir))
    for key in ((0, 0), (1, 31)):
        back = aeon_b200.unpack_expert_shards(cfg, 2, np.asarray(art.expert_data(*key)))
        assert all(np.array_equal(a, b) for a, b in zip(back, sources[key]))
    dense = artifact.DenseContainer(str(out_dir / artifact.DENSE_FILENAME))
    want_dense = {n for n in weight_map if ".ffn.experts." not in n}
    assert set(dense.names()) == want_dense and "layers.1.ffn.shared_experts.w1.weight" in want_dense
    for name in want_dense:
        dtype, array = shards[0].get(name) or shards[1][name]
        assert dense.dtype_of(name) == dtype and dense.raw(name).tobytes() == array.tobytes()
    assert json.load(open(out_dir / "config.json"))["model_type"] == "deepseek_v4"
    assert json.load(open(out_dir / artifact.MANIFEST_FILENAME))["max_tensor_parallel"] == 2

    # the command-line form, first layer only
    one = tmp_path / "one"
    import unittest.mock as mock
    with mock.patch.object(aeon_b200, "preset", lambda name: cfg):
        assert artifact._main([str(src_dir), str(one), "--from-safetensors", "--max-tensor-parallel", "1",
                               "--max-layers", "1"]) == 0
    first = artifact.ExpertArtifact(str(one))
    assert (first.format.version, first.format.num_layers) == (2, 1)
    assert set(artifact.DenseContainer(str(one / artifact.DENSE_FILENAME)).names()) == \
        {n for n in want_dense if not n.startswith("layers.1.")}

    # refusals: a missing expert tensor, a wrong shape
    del weight_map["layers.1.ffn.experts.7.w2.weight_scale"]
    (src_dir / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    with pytest.raises(KeyError, match="Missing tensor"):
        artifact.convert_checkpoint(str(src_dir), str(tmp_path / "bad"), cfg)
    with pytest.raises(ValueError, match="expected"):
        artifact.convert_checkpoint(str(src_dir), str(tmp_path / "bad2"), cfg.copy(hidden=512), max_layers=1)
