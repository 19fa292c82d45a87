"""Artifact files either side of the routed-expert path.

Expert container (reference: writer scripts/convert_safetensors_to_aeon.py:440-520, loader
src/infrastructure/artifact/aeon_loader.hpp:318-441):

    model_experts_swizzled.index   "AEON_EXPERTS", u32 version, u32 layers, u32 experts per
                                   layer, u64 payload bytes            (v2: 32-byte header)
                                   + u32 shard count, u32 zero, u64 shard bytes   (v3: 48 bytes)
                                   then (u64 offset, u64 length) per expert, layer-major
    model_experts_swizzled.aeon    the payloads, each on a 4 KiB boundary

Version 3 is the shard-aware layout the reference plans for tensor parallelism
(plans-and-docs/execution/active/MULTI_GPU_EXECUTION_PLAN.md:151-181): a payload is
`shard_count` self-contained shards of the intermediate dimension written shard-major, so
rank r of a tensor-parallel group of degree tp reads exactly one contiguous range,
offset + r * (shard_count / tp) * shard_bytes, payload_bytes / tp long (`rank_slice`), with no
read amplification. Version 2 is the same file with shard_count = 1.

Dense container (reference: writer :348-436, loader aeon_loader.hpp:243-316,441-479):
"AEON_DENSE\\0\\0", u32 version, u32 tensor count, u64 directory length, a JSON directory of
{name, offset, size, dtype, shape}, then the tensor bytes from the next 4 KiB boundary. The
router gate (layers.N.ffn.gate.weight / .bias / .tid2eid) and the shared expert
(layers.N.ffn.shared_experts.w{1,2,3}.weight) live there
(src/architecture/deepseek_v4/spec/v4_dense_weight_binding.hpp:123-137).
"""
from __future__ import annotations

import json
import os
import struct
from dataclasses import dataclass

import numpy as np

import aeon_b200

SECTOR_SIZE = 4096
EXPERT_MAGIC = b"AEON_EXPERTS"
DENSE_MAGIC = b"AEON_DENSE\x00\x00"
EXPERTS_FILENAME = "model_experts_swizzled.aeon"
INDEX_FILENAME = "model_experts_swizzled.index"
DENSE_FILENAME = "model_dense.aeon"
MANIFEST_FILENAME = "model_manifest.json"
DENSE_FORMAT_VERSION = 1

_DTYPES = {"BF16": np.uint16, "F16": np.uint16, "F32": np.float32, "I64": np.int64,
           "I32": np.int32, "U8": np.uint8}


@dataclass(frozen=True)
class ExpertFormat:
    """ExpertFormatDescriptor (src/infrastructure/expert/storage/expert_format.hpp:10-60) plus the
    planned shard fields; version 2 means shard_count 1 and shard_bytes = payload_bytes."""
    version: int
    num_layers: int
    experts_per_layer: int
    payload_bytes: int
    shard_count: int = 1
    shard_bytes: int = 0
    sector_size: int = SECTOR_SIZE

    def validate(self) -> None:
        if self.version not in (2, 3):
            raise ValueError(f"expert index: unsupported version {self.version}")
        if self.num_layers <= 0 or self.experts_per_layer <= 0:
            raise ValueError("expert index: empty expert catalog")
        if self.payload_bytes <= 0 or self.payload_bytes % self.sector_size:
            raise ValueError("expert index: payload must be a positive multiple of the sector size")
        if self.shard_count <= 0 or self.shard_count * self.shard_bytes != self.payload_bytes:
            raise ValueError("expert index: shard_count * shard_bytes must equal payload_bytes")
        if self.shard_bytes % self.sector_size:
            raise ValueError("expert index: shard_bytes must be a multiple of the sector size")


def _header(fmt: ExpertFormat) -> bytes:
    head = struct.pack("<12sIIIQ", EXPERT_MAGIC, fmt.version, fmt.num_layers, fmt.experts_per_layer,
                       fmt.payload_bytes)
    if fmt.version >= 3:
        head += struct.pack("<IIQ", fmt.shard_count, 0, fmt.shard_bytes)
    return head


def write_expert_artifact(model_dir: str, cfg, layers: int, source_of, max_tensor_parallel: int = 1,
                          write_manifest: bool = True) -> ExpertFormat:
    """Writes the expert container of `layers` x cfg.experts experts.

    source_of(layer, expert) returns the six checkpoint-order tensors of the expert
    (aeon_b200.source_shapes). max_tensor_parallel = D in {1, 2, 4, 8} writes D shards per
    expert (index version 3); D = 1 writes the reference's version 2, byte for byte."""
    D = int(max_tensor_parallel)
    if D not in (1, 2, 4, 8):
        raise ValueError("max_tensor_parallel must be 1, 2, 4 or 8")
    if (cfg.intermediate // 256) % D:
        raise ValueError("max_tensor_parallel must divide intermediate / 256")
    shard_bytes = aeon_b200.expert_shard_bytes(cfg, D)
    fmt = ExpertFormat(3 if D > 1 else 2, layers, cfg.experts, D * shard_bytes, D, shard_bytes)
    fmt.validate()
    os.makedirs(model_dir, exist_ok=True)
    entries = []
    offset = 0
    with open(os.path.join(model_dir, EXPERTS_FILENAME), "wb") as out:
        for layer in range(layers):
            for expert in range(cfg.experts):
                payload = aeon_b200.pack_expert_shards(cfg, D, source_of(layer, expert))
                assert payload.size == fmt.payload_bytes and offset % SECTOR_SIZE == 0
                out.write(payload.tobytes())
                entries.append((offset, fmt.payload_bytes))
                offset += fmt.payload_bytes
    with open(os.path.join(model_dir, INDEX_FILENAME), "wb") as idx:
        idx.write(_header(fmt))
        for off, length in entries:
            idx.write(struct.pack("<QQ", off, length))
    if write_manifest:
        write_model_manifest(model_dir, fmt)
    return fmt


def write_model_manifest(model_dir: str, fmt: ExpertFormat, model_family: str = "deepseek",
                         architecture: str = "deepseek_v4") -> dict:
    """model_manifest.json as the reference's loader reads it
    (src/infrastructure/artifact/model_manifest.hpp:102-209: identity, weight backend, file names,
    versions, sizes) plus the shard fields of the shard-aware container. dense_file_bytes is taken
    from the dense file if it is already there; write_dense_container fills it in otherwise."""
    dense_path = os.path.join(model_dir, DENSE_FILENAME)
    manifest = {
        "manifest_version": 2 if fmt.shard_count > 1 else 1,
        "model_family": model_family,
        "architecture": architecture,
        "weight_backend": "swizzled_w4a16",
        "dense_file_bytes": os.path.getsize(dense_path) if os.path.exists(dense_path) else 0,
        "num_layers": fmt.num_layers,
        "experts_per_layer": fmt.experts_per_layer,
        "max_tensor_parallel": fmt.shard_count,
        "artifact": {
            "experts_filename": EXPERTS_FILENAME,
            "index_filename": INDEX_FILENAME,
            "dense_filename": DENSE_FILENAME,
            "dense_format_version": DENSE_FORMAT_VERSION,
            "expert_format": "swizzled_w4a16",
            "expert_format_version": fmt.version,
            "expert_sector_size": fmt.sector_size,
            "expert_payload_bytes": fmt.payload_bytes,
            "expert_shard_count": fmt.shard_count,
            "expert_shard_bytes": fmt.shard_bytes or fmt.payload_bytes,
        },
    }
    with open(os.path.join(model_dir, MANIFEST_FILENAME), "w", encoding="utf-8") as f:
        json.dump(manifest, f, indent=2)
        f.write("\n")
    return manifest


def read_model_manifest(model_dir: str) -> dict | None:
    path = os.path.join(model_dir, MANIFEST_FILENAME)
    if not os.path.exists(path):
        return None
    with open(path, encoding="utf-8") as f:
        return json.load(f)


class ExpertArtifact:
    """Reader of the expert container: the expert half of AeonModelLoader
    (src/infrastructure/artifact/aeon_loader.hpp:145-166) plus the planned rank_slice."""

    def __init__(self, model_dir: str, expected_payload_bytes: int | None = None):
        index_path = os.path.join(model_dir, INDEX_FILENAME)
        with open(index_path, "rb") as f:
            buf = f.read()
        if len(buf) < 32:
            raise ValueError("AeonModelLoader: Expert index too small for header!")
        magic, version, layers, experts, payload = struct.unpack_from("<12sIIIQ", buf, 0)
        if magic != EXPERT_MAGIC:
            raise ValueError("AeonModelLoader: Invalid expert index magic!")
        head = 32
        shard_count, shard_bytes = 1, payload
        if version == 3:
            if len(buf) < 48:
                raise ValueError("AeonModelLoader: Expert index too small for header!")
            shard_count, zero, shard_bytes = struct.unpack_from("<IIQ", buf, 32)
            head = 48
        self.format = ExpertFormat(version, layers, experts, payload, shard_count, shard_bytes)
        self.format.validate()
        if expected_payload_bytes is not None and payload != expected_payload_bytes:
            raise ValueError("AeonModelLoader: Expert payload size does not match the artifact specification")
        total = layers * experts
        if len(buf) < head + 16 * total:
            raise ValueError("AeonModelLoader: Expert index has incomplete entries!")
        table = np.frombuffer(buf, dtype="<u8", count=2 * total, offset=head).reshape(total, 2)
        if np.any(table[:, 1] != payload) or np.any(table[:, 0] % SECTOR_SIZE):
            raise ValueError("AeonModelLoader: Expert index contains an invalid payload entry")
        self._offsets = table[:, 0].astype(np.int64)
        self._data = np.memmap(os.path.join(model_dir, EXPERTS_FILENAME), dtype=np.uint8, mode="r")
        if total and int(self._offsets.max()) + payload > self._data.size:
            raise ValueError("AeonModelLoader: Expert payload lies outside the experts file")

    def _index(self, layer: int, expert: int) -> int:
        if not (0 <= layer < self.format.num_layers and 0 <= expert < self.format.experts_per_layer):
            raise IndexError("AeonModelLoader: expert id out of range")
        return layer * self.format.experts_per_layer + expert

    def expert_location(self, layer: int, expert: int):
        return int(self._offsets[self._index(layer, expert)]), self.format.payload_bytes

    def expert_data(self, layer: int, expert: int) -> np.ndarray:
        off, length = self.expert_location(layer, expert)
        return self._data[off:off + length]

    def rank_slice(self, layer: int, expert: int, tp: int, rank: int):
        """(file offset, length) of what rank `rank` of a tensor-parallel group of `tp` reads."""
        D = self.format.shard_count
        if tp <= 0 or D % tp:
            raise ValueError(f"tensor_parallel={tp} does not divide the artifact's max tensor-parallel "
                             f"degree {D}")
        if not 0 <= rank < tp:
            raise IndexError("rank out of range")
        off, _ = self.expert_location(layer, expert)
        per_rank = (D // tp) * self.format.shard_bytes
        return off + rank * per_rank, per_rank

    def rank_payload(self, cfg, layer: int, expert: int, tp: int, rank: int) -> np.ndarray:
        """The payload rank `rank` uploads into its pool (config: cfg with intermediate / tp):
        its slice, with the slice's shards merged into one swizzled payload."""
        off, length = self.rank_slice(layer, expert, tp, rank)
        cfg_rank = cfg.copy(intermediate=cfg.intermediate // tp)
        return aeon_b200.merge_expert_shards(cfg_rank, self.format.shard_count // tp,
                                             np.asarray(self._data[off:off + length]))


def verify_conversion(model_dir: str, cfg, source_of, sample=None) -> int:
    """Every (sampled) expert of the artifact unswizzles, shard by shard, to exactly the source
    tensors it was written from. Returns the number of experts checked."""
    art = ExpertArtifact(model_dir)
    pairs = sample if sample is not None else [
        (l, e) for l in range(art.format.num_layers) for e in range(art.format.experts_per_layer)]
    for layer, expert in pairs:
        back = aeon_b200.unpack_expert_shards(cfg, art.format.shard_count, np.asarray(art.expert_data(layer, expert)))
        for got, want in zip(back, source_of(layer, expert)):
            if not np.array_equal(got, np.asarray(want)):
                raise ValueError(f"verify_conversion: layer {layer} expert {expert} does not round-trip")
    return len(pairs)


def reshard_expert_artifact(src_dir: str, dst_dir: str, cfg, max_tensor_parallel: int,
                            verify: bool = True) -> ExpertFormat:
    """Rewrites an expert container (version 2 or 3) with `max_tensor_parallel` shards per expert.
    The conversion of an existing single-device artifact into the shard-aware one: every
    payload is unswizzled to the checkpoint order and re-cut, so no original checkpoint is needed."""
    src = ExpertArtifact(src_dir)
    if src.format.experts_per_layer != cfg.experts:
        raise ValueError("reshard: the configuration's expert count does not match the artifact")
    if src.format.payload_bytes != src.format.shard_count * aeon_b200.expert_shard_bytes(cfg, src.format.shard_count):
        raise ValueError("reshard: the configuration's shapes do not match the artifact's payload size")

    def source_of(layer, expert):
        return aeon_b200.unpack_expert_shards(cfg, src.format.shard_count, np.asarray(src.expert_data(layer, expert)))

    fmt = write_expert_artifact(dst_dir, cfg, src.format.num_layers, source_of, max_tensor_parallel)
    if verify:
        verify_conversion(dst_dir, cfg, source_of)
    return fmt


# ---------------------------------------------------------------------------------------------
# Dense container
# ---------------------------------------------------------------------------------------------
def write_dense_container(path: str, tensors) -> None:
    """tensors: iterable of (name, dtype string, numpy array); 16-bit floats are passed as uint16
    bit patterns with dtype "BF16" or "F16"."""
    directory, blobs, offset = [], [], 0
    for name, dtype, array in tensors:
        if dtype not in _DTYPES:
            raise ValueError(f"dense container: unsupported dtype {dtype}")
        a = np.ascontiguousarray(array, dtype=_DTYPES[dtype])
        directory.append({"name": name, "offset": offset, "size": a.nbytes, "dtype": dtype,
                          "shape": list(a.shape)})
        blobs.append(a)
        offset += a.nbytes
    dir_json = json.dumps(directory, indent=2).encode("utf-8")
    head = struct.pack("<12sIIQ", DENSE_MAGIC, DENSE_FORMAT_VERSION, len(directory), len(dir_json))
    pad = (-(len(head) + len(dir_json))) % SECTOR_SIZE
    with open(path, "wb") as f:
        f.write(head)
        f.write(dir_json)
        f.write(b"\x00" * pad)
        for a in blobs:
            f.write(a.tobytes())
    _record_dense_size(path)


def _record_dense_size(dense_path: str) -> None:
    """A manifest beside a freshly written dense file learns the file's size."""
    model_dir = os.path.dirname(os.path.abspath(dense_path))
    manifest = read_model_manifest(model_dir)
    if manifest is not None and os.path.basename(dense_path) == manifest["artifact"]["dense_filename"]:
        manifest["dense_file_bytes"] = os.path.getsize(dense_path)
        with open(os.path.join(model_dir, MANIFEST_FILENAME), "w", encoding="utf-8") as f:
            json.dump(manifest, f, indent=2)
            f.write("\n")


class DenseContainer:
    def __init__(self, path: str, expected_version: int = DENSE_FORMAT_VERSION):
        self._data = np.memmap(path, dtype=np.uint8, mode="r")
        if self._data.size < 28:
            raise ValueError("AeonModelLoader: Dense file too small for header: " + path)
        magic, version, count, dir_len = struct.unpack_from("<12sIIQ", self._data[:28].tobytes(), 0)
        if magic != DENSE_MAGIC:
            raise ValueError("AeonModelLoader: Invalid dense magic in " + path)
        if version != expected_version:
            raise ValueError(f"AeonModelLoader: Unexpected dense format version {version}, "
                             f"expected {expected_version}")
        if dir_len > self._data.size - 28:
            raise ValueError("AeonModelLoader: Directory length exceeds file size!")
        entries = json.loads(self._data[28:28 + dir_len].tobytes().decode("utf-8"))
        start = 28 + dir_len
        start += (-start) % SECTOR_SIZE
        if start > self._data.size:
            raise ValueError("AeonModelLoader: Dense payload starts beyond file size")
        room = self._data.size - start
        self._tensors = {}
        for e in entries:
            off, size = int(e["offset"]), int(e["size"])
            if off < 0 or size < 0:
                raise ValueError("AeonModelLoader: Dense directory contains a negative range")
            if off > room or size > room - off:
                raise ValueError("AeonModelLoader: Dense tensor range exceeds payload")
            if e["name"] in self._tensors:
                raise ValueError("AeonModelLoader: Duplicate dense tensor: " + e["name"])
            self._tensors[e["name"]] = (start + off, size, e["dtype"], tuple(int(d) for d in e["shape"]))
        if len(entries) != count:
            raise ValueError("AeonModelLoader: Dense directory count does not match its header")

    def has_tensor(self, name: str) -> bool:
        return name in self._tensors

    def names(self):
        return list(self._tensors)

    def get_tensor(self, name: str) -> np.ndarray:
        if name not in self._tensors:
            raise KeyError("AeonModelLoader: Missing dense tensor: " + name)
        off, size, dtype, shape = self._tensors[name]
        return self._data[off:off + size].view(_DTYPES[dtype]).reshape(shape)

    def dtype_of(self, name: str) -> str:
        return self._tensors[name][2]

    def raw(self, name: str) -> np.ndarray:
        """The tensor's bytes, whatever its element type."""
        if name not in self._tensors:
            raise KeyError("AeonModelLoader: Missing dense tensor: " + name)
        off, size, _, _ = self._tensors[name]
        return self._data[off:off + size]


def moe_layer_tensor_names(layer: int, hash_layer: bool = False) -> dict:
    """Names of the dense tensors the path reads for one layer."""
    p = f"layers.{layer}.ffn."
    names = {"gate": p + "gate.weight", "shared_w1": p + "shared_experts.w1.weight",
             "shared_w2": p + "shared_experts.w2.weight", "shared_w3": p + "shared_experts.w3.weight"}
    names["tid2eid" if hash_layer else "gate_bias"] = p + ("gate.tid2eid" if hash_layer else "gate.bias")
    return names


# ---------------------------------------------------------------------------------------------
# Checkpoint front end: safetensors shards -> the two containers
# ---------------------------------------------------------------------------------------------
_ST_SIZES = {"BF16": 2, "F16": 2, "F32": 4, "F64": 8, "I64": 8, "I32": 4, "U32": 4, "I16": 2, "U16": 2,
             "I8": 1, "U8": 1, "BOOL": 1, "F8_E4M3": 1, "F8_E5M2": 1}


class SafetensorsFile:
    """One safetensors shard, read without interpreting the element types (bf16 has no numpy
    type): u64 header length, JSON header {name: {dtype, shape, data_offsets}}, then the bytes."""

    def __init__(self, path: str):
        self.path = path
        self._data = np.memmap(path, dtype=np.uint8, mode="r")
        if self._data.size < 8:
            raise ValueError("safetensors: file too small: " + path)
        (n,) = struct.unpack("<Q", self._data[:8].tobytes())
        if n > self._data.size - 8:
            raise ValueError("safetensors: header length exceeds the file: " + path)
        header = json.loads(self._data[8:8 + n].tobytes().decode("utf-8"))
        self._base = 8 + n
        self.tensors = {}
        for name, meta in header.items():
            if name == "__metadata__":
                continue
            start, end = meta["data_offsets"]
            shape = tuple(int(d) for d in meta["shape"])
            count = int(np.prod(shape)) if shape else 1
            if meta["dtype"] not in _ST_SIZES or end - start != count * _ST_SIZES[meta["dtype"]]:
                raise ValueError(f"safetensors: tensor {name} has an inconsistent size in {path}")
            if end > self._data.size - self._base or start > end:
                raise ValueError(f"safetensors: tensor {name} lies outside {path}")
            self.tensors[name] = (meta["dtype"], shape, start, end)

    def raw(self, name: str) -> np.ndarray:
        _, _, start, end = self.tensors[name]
        return self._data[self._base + start:self._base + end]


class SafetensorsCheckpoint:
    """A checkpoint directory: `model.safetensors.index.json` (weight_map: tensor -> shard) or a
    single `model.safetensors` (the source side of scripts/convert_safetensors_to_aeon.py:196-260)."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        index_path = os.path.join(model_dir, "model.safetensors.index.json")
        self._files = {}
        if os.path.exists(index_path):
            with open(index_path, "r", encoding="utf-8") as f:
                weight_map = json.load(f).get("weight_map", {})
            self._where = dict(weight_map)
        else:
            single = os.path.join(model_dir, "model.safetensors")
            if not os.path.exists(single):
                raise FileNotFoundError("Missing Safetensors index: " + index_path)
            self._where = {name: "model.safetensors" for name in self._file("model.safetensors").tensors}
        for name, shard in self._where.items():
            if name not in self._file(shard).tensors:
                raise KeyError(f"Missing tensor in Safetensors: {name} (expected in {shard})")

    def _file(self, shard: str) -> SafetensorsFile:
        if shard not in self._files:
            self._files[shard] = SafetensorsFile(os.path.join(self.model_dir, shard))
        return self._files[shard]

    def names(self):
        return sorted(self._where)

    def meta(self, name: str):
        if name not in self._where:
            raise KeyError("Missing tensor in Safetensors: " + name)
        dtype, shape, _, _ = self._file(self._where[name]).tensors[name]
        return dtype, shape

    def raw(self, name: str) -> np.ndarray:
        if name not in self._where:
            raise KeyError("Missing tensor in Safetensors: " + name)
        return self._file(self._where[name]).raw(name)


def convert_checkpoint(source_dir: str, output_dir: str, cfg, max_tensor_parallel: int = 1,
                       max_layers: int | None = None, verify: bool = True) -> ExpertFormat:
    """safetensors checkpoint -> model_dense.aeon + model_experts_swizzled.{aeon,index} + manifest.

    Routed experts are the tensors `layers.L.ffn.experts.E.{w1,w2,w3}.{weight_packed,weight_scale}`
    (packed words [N, K/8], fp16 scales [N, K/group]; scripts/convert_safetensors_to_aeon.py:489-511);
    every other tensor goes to the dense container byte for byte (:361-364). With
    max_tensor_parallel > 1 the experts are written shard-aware (index version 3)."""
    ckpt = SafetensorsCheckpoint(source_dir)
    names = ckpt.names()
    routed = [n for n in names if ".ffn.experts." in n and "shared_experts" not in n]
    layer_ids = sorted({int(n.split(".")[1]) for n in routed})
    if not layer_ids or layer_ids != list(range(len(layer_ids))):
        raise ValueError("checkpoint: routed-expert layers must be numbered 0..L-1")
    layers = len(layer_ids) if max_layers is None else min(max_layers, len(layer_ids))
    shapes = aeon_b200.source_shapes(cfg)

    def source_of(layer, expert):
        out = []
        for i, (w, t) in enumerate((("w1", "weight_packed"), ("w1", "weight_scale"), ("w2", "weight_packed"),
                                    ("w2", "weight_scale"), ("w3", "weight_packed"), ("w3", "weight_scale"))):
            key = f"layers.{layer}.ffn.experts.{expert}.{w}.{t}"
            dtype, shape = ckpt.meta(key)
            want = ("I32", "U32") if i % 2 == 0 else ("F16",)
            if dtype not in want or tuple(shape) != shapes[i]:
                raise ValueError(f"checkpoint: {key} is {dtype}{list(shape)}, expected {want[0]}{list(shapes[i])}")
            out.append(np.asarray(ckpt.raw(key)).view(np.uint32 if i % 2 == 0 else np.uint16).reshape(shapes[i]))
        return out

    fmt = write_expert_artifact(output_dir, cfg, layers, source_of, max_tensor_parallel)

    def keep(name):
        if name in routed:
            return False
        if max_layers is not None and name.startswith("layers."):
            return int(name.split(".")[1]) < max_layers
        return True

    dense = []
    for name in names:
        if keep(name):
            dtype, shape = ckpt.meta(name)
            dense.append((name, dtype, shape, ckpt.raw(name)))
    _write_dense_raw(os.path.join(output_dir, DENSE_FILENAME), dense)
    for aux in ("config.json", "generation_config.json", "tokenizer.json", "tokenizer_config.json"):
        src = os.path.join(source_dir, aux)
        if os.path.isfile(src):
            with open(src, "rb") as fi, open(os.path.join(output_dir, aux), "wb") as fo:
                fo.write(fi.read())
    if verify:
        verify_conversion(output_dir, cfg, source_of)
        back = DenseContainer(os.path.join(output_dir, DENSE_FILENAME))
        for name, dtype, shape, raw in dense:
            if back.dtype_of(name) != dtype or back.raw(name).tobytes() != np.asarray(raw).tobytes():
                raise ValueError("verify_conversion: dense tensor does not round-trip: " + name)
    return fmt


def _write_dense_raw(path: str, tensors) -> None:
    """tensors: (name, dtype string, shape, raw uint8 bytes); any safetensors dtype passes through."""
    directory, offset = [], 0
    for name, dtype, shape, raw in tensors:
        directory.append({"name": name, "offset": offset, "size": int(raw.size), "dtype": dtype,
                          "shape": [int(d) for d in shape]})
        offset += int(raw.size)
    dir_json = json.dumps(directory, indent=2).encode("utf-8")
    head = struct.pack("<12sIIQ", DENSE_MAGIC, DENSE_FORMAT_VERSION, len(directory), len(dir_json))
    pad = (-(len(head) + len(dir_json))) % SECTOR_SIZE
    with open(path, "wb") as f:
        f.write(head)
        f.write(dir_json)
        f.write(b"\x00" * pad)
        for _, _, _, raw in tensors:
            f.write(np.asarray(raw).tobytes())
    _record_dense_size(path)


def _main(argv=None) -> int:
    import argparse
    ap = argparse.ArgumentParser(
        prog="python -m aeon_b200.artifact",
        description="Rewrite an expert container with shard-aware (version 3) payloads, or, with "
                    "--from-safetensors, convert a safetensors checkpoint into the two containers.")
    ap.add_argument("source_dir")
    ap.add_argument("output_dir")
    ap.add_argument("--from-safetensors", action="store_true")
    ap.add_argument("--max-layers", type=int, default=None)
    ap.add_argument("--preset", default="ref_dsv4", help="shape preset of the experts (ref_dsv4, baseline)")
    ap.add_argument("--max-tensor-parallel", type=int, default=8, choices=(1, 2, 4, 8))
    ap.add_argument("--no-verify", action="store_true")
    args = ap.parse_args(argv)
    cfg = aeon_b200.preset(args.preset)
    if args.from_safetensors:
        fmt = convert_checkpoint(args.source_dir, args.output_dir, cfg, args.max_tensor_parallel,
                                 max_layers=args.max_layers, verify=not args.no_verify)
    else:
        fmt = reshard_expert_artifact(args.source_dir, args.output_dir, cfg, args.max_tensor_parallel,
                                      verify=not args.no_verify)
    print(f"wrote {fmt.num_layers} x {fmt.experts_per_layer} experts, version {fmt.version}, "
          f"{fmt.shard_count} shards of {fmt.shard_bytes} bytes")
    return 0


if __name__ == "__main__":
    raise SystemExit(_main())
