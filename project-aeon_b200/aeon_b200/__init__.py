"""ctypes binding of libaeon_b200.so (the C ABI declared in include/aeon_b200.h).

PyTorch is used only as the owner of device memory and streams: every call takes
``tensor.data_ptr()`` values and the current CUDA stream handle. There is no CPU
fallback: importing works anywhere (so the symbols can be checked), but any
compute call needs an sm_100 device and raises ``AeonError`` otherwise.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import (POINTER, c_char_p, c_float, c_int, c_int32, c_int64, c_uint16, c_uint32,
                    c_uint64, c_void_p)

_HERE = os.path.dirname(os.path.abspath(__file__))
# AEON_B200_LIBRARY selects another build of the same library (the bounds-checked one, say)
LIB_PATH = os.environ.get("AEON_B200_LIBRARY") or os.path.join(os.path.dirname(_HERE), "lib", "libaeon_b200.so")

F16, BF16 = 0, 1
SCORE_SQRT_SOFTPLUS, SCORE_SIGMOID = 0, 1
DECODE_SKIP_ABSENT = 1
DECODE_DEFER_ACCUMULATE = 2
DECODE_OVERWRITE = 4

STATUS_NAMES = {0: "OK", 1: "INVALID_ARGUMENT", 2: "LOGIC", 3: "CUDA", 4: "OUT_OF_RANGE",
                5: "TIMEOUT", 6: "UNSUPPORTED"}

# Every symbol include/aeon_b200.h declares (checked by the CPU test-suite).
EXPORTED_SYMBOLS = [
    "aeon_b200_last_error", "aeon_b200_version", "aeon_b200_config_preset",
    "aeon_b200_config_validate", "aeon_b200_expert_layout_of", "aeon_b200_swizzle_w4a16",
    "aeon_b200_unswizzle_w4a16", "aeon_b200_ctx_create", "aeon_b200_ctx_destroy",
    "aeon_b200_ctx_scratch_bytes", "aeon_b200_ctx_check", "aeon_b200_ctx_launches",
    "aeon_b200_pool_create", "aeon_b200_pool_destroy", "aeon_b200_pool_upload",
    "aeon_b200_router_topk", "aeon_b200_expert_permutation", "aeon_b200_shared_expert",
    "aeon_b200_moe_decode", "aeon_b200_ctx_last_stats", "aeon_b200_synth_fill_experts",
    "aeon_b200_synth_fill_dense16", "aeon_b200_ctx_set_timing", "aeon_b200_ctx_kernel_times",
    "aeon_b200_ep_combine", "aeon_b200_router_topk_noalloc", "aeon_b200_moe_prefill", "aeon_b200_moe_accumulate",
    "aeon_b200_expert_shard_bytes", "aeon_b200_pack_expert_shards", "aeon_b200_unpack_expert_shards",
    "aeon_b200_expert_rank_slice", "aeon_b200_merge_expert_shards",
    "aeon_b200_hc_params_default", "aeon_b200_hc_ffn_front", "aeon_b200_hc_post",
    "aeon_b200_group_unique_id", "aeon_b200_group_create", "aeon_b200_group_destroy",
    "aeon_b200_group_rank", "aeon_b200_group_world", "aeon_b200_ep_dispatch", "aeon_b200_ep_dispatch_routed", "aeon_b200_ep_exchange",
    "aeon_b200_ep_peer_dispatch",
    "aeon_b200_tp_reduce", "aeon_b200_pp_send", "aeon_b200_pp_recv",
    "aeon_b200_device_count", "aeon_b200_device_current", "aeon_b200_device_select",
    "aeon_b200_device_describe", "aeon_b200_device_enable_peer_access", "aeon_b200_device_alloc",
    "aeon_b200_device_free", "aeon_b200_stream_create", "aeon_b200_stream_destroy",
    "aeon_b200_stream_synchronize", "aeon_b200_stream_wait_event", "aeon_b200_event_create",
    "aeon_b200_event_destroy", "aeon_b200_event_record", "aeon_b200_event_synchronize",
    "aeon_b200_host_alloc_pinned", "aeon_b200_host_free_pinned", "aeon_b200_copy_to_device_async",
    "aeon_b200_copy_to_host_async", "aeon_b200_ctx_set_pool_slots", "aeon_b200_bounds_checked",
    "aeon_b200_ep_peer_create", "aeon_b200_ep_peer_destroy", "aeon_b200_ep_peer_set_wait_budget",
    "aeon_b200_moe_accumulate_push", "aeon_b200_ep_peer_combine",
]


class AeonError(RuntimeError):
    """Mirrors the reference's exception kinds through the status code."""

    def __init__(self, status: int, message: str):
        super().__init__(f"[{STATUS_NAMES.get(status, status)}] {message}")
        self.status = status


class MoeConfig(ctypes.Structure):
    _fields_ = [("hidden", c_int32), ("intermediate", c_int32), ("experts", c_int32),
                ("top_k", c_int32), ("group_size", c_int32), ("act_dtype", c_int32),
                ("score_fn", c_int32), ("renormalize", c_int32), ("routed_scaling", c_float),
                ("swiglu_limit", c_float), ("w13_rpw", c_int32), ("w13_lpr", c_int32),
                ("w2_rpw", c_int32), ("w2_lpr", c_int32)]

    def copy(self, **changes) -> "MoeConfig":
        out = MoeConfig.from_buffer_copy(bytes(self))
        for key, value in changes.items():
            setattr(out, key, value)
        return out


class HcParams(ctypes.Structure):
    _fields_ = [("rms_eps", c_float), ("pre_eps", c_float), ("sinkhorn_eps", c_float),
                ("post_mult", c_float), ("norm_eps", c_float), ("sinkhorn_iters", c_int32)]


class ExpertLayout(ctypes.Structure):
    _fields_ = [(name, c_uint64) for name in (
        "payload_bytes", "w1_packed_offset", "w1_scale_offset", "w2_packed_offset",
        "w2_scale_offset", "w3_packed_offset", "w3_scale_offset", "w13_packed_bytes",
        "w13_scale_bytes", "w2_packed_bytes", "w2_scale_bytes")]


_lib = None


def lib() -> ctypes.CDLL:
    """Loads the shared library; a missing build is an error, never a fallback."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise AeonError(3, f"{LIB_PATH} is missing: run `python -c 'import __graft_entry__ as g; "
                           "g.build()'` (or make -C project-aeon_b200/csrc) first")
    L = ctypes.CDLL(LIB_PATH)
    L.aeon_b200_last_error.restype = c_char_p
    L.aeon_b200_version.restype = c_char_p
    L.aeon_b200_ctx_scratch_bytes.restype = c_uint64
    L.aeon_b200_ctx_scratch_bytes.argtypes = [c_void_p]
    L.aeon_b200_ctx_launches.restype = c_uint64
    L.aeon_b200_ctx_launches.argtypes = [c_void_p]
    L.aeon_b200_config_preset.argtypes = [c_char_p, POINTER(MoeConfig)]
    L.aeon_b200_config_validate.argtypes = [POINTER(MoeConfig)]
    L.aeon_b200_expert_layout_of.argtypes = [POINTER(MoeConfig), POINTER(ExpertLayout)]
    swz = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int]
    L.aeon_b200_swizzle_w4a16.argtypes = swz
    L.aeon_b200_unswizzle_w4a16.argtypes = swz
    L.aeon_b200_expert_shard_bytes.argtypes = [POINTER(MoeConfig), c_int, POINTER(c_uint64)]
    six = [c_void_p] * 6
    L.aeon_b200_pack_expert_shards.argtypes = [POINTER(MoeConfig), c_int] + six + [c_void_p]
    L.aeon_b200_unpack_expert_shards.argtypes = [POINTER(MoeConfig), c_int, c_void_p] + six
    L.aeon_b200_expert_rank_slice.argtypes = [POINTER(MoeConfig), c_int, c_int, c_int,
                                              POINTER(c_uint64), POINTER(c_uint64)]
    L.aeon_b200_merge_expert_shards.argtypes = [POINTER(MoeConfig), c_int, c_void_p, c_void_p]
    L.aeon_b200_ctx_create.argtypes = [POINTER(MoeConfig), c_int, c_int, POINTER(c_void_p)]
    L.aeon_b200_ctx_destroy.argtypes = [c_void_p]
    L.aeon_b200_ctx_check.argtypes = [c_void_p, c_void_p]
    L.aeon_b200_ctx_last_stats.argtypes = [c_void_p, c_void_p, POINTER(c_int32), POINTER(c_int32)]
    L.aeon_b200_ctx_set_timing.argtypes = [c_void_p, c_int]
    L.aeon_b200_ctx_kernel_times.argtypes = [c_void_p, c_void_p, POINTER(ctypes.c_double),
                                             POINTER(c_int64)]
    L.aeon_b200_pool_create.argtypes = [c_uint64, c_uint32, c_int, POINTER(c_void_p)]
    L.aeon_b200_pool_destroy.argtypes = [c_void_p, c_int]
    L.aeon_b200_pool_upload.argtypes = [c_void_p, c_uint64, c_uint32, c_void_p, c_void_p]
    L.aeon_b200_router_topk.argtypes = [c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p,
                                        c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p]
    L.aeon_b200_router_topk_noalloc.argtypes = [POINTER(MoeConfig), c_void_p, c_int64, c_void_p,
                                                c_void_p, c_int, c_void_p, c_void_p, c_void_p]
    L.aeon_b200_expert_permutation.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p,
                                               c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]
    L.aeon_b200_shared_expert.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                                          c_int, c_void_p, c_int64, c_void_p]
    L.aeon_b200_moe_decode.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p,
                                       c_void_p, c_int, c_void_p, c_int64, c_uint32, c_void_p]
    L.aeon_b200_moe_prefill.argtypes = L.aeon_b200_moe_decode.argtypes
    L.aeon_b200_moe_accumulate.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int64,
                                           c_uint32, c_void_p]
    L.aeon_b200_ep_combine.argtypes = [c_void_p, c_int64, c_void_p, c_int, c_int, c_int, c_void_p]
    L.aeon_b200_hc_params_default.argtypes = [POINTER(HcParams)]
    L.aeon_b200_hc_ffn_front.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                         POINTER(HcParams), c_void_p, c_int64, c_void_p, c_void_p,
                                         c_void_p, c_void_p]
    L.aeon_b200_hc_post.argtypes = [c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int,
                                    c_void_p, c_void_p]
    L.aeon_b200_synth_fill_experts.argtypes = [POINTER(MoeConfig), c_void_p, c_uint32, c_uint32,
                                               c_uint64, c_uint32, c_uint32, c_void_p, c_uint32,
                                               c_void_p]
    L.aeon_b200_synth_fill_dense16.argtypes = [c_void_p, c_uint64, c_uint64, c_uint32, c_uint32,
                                               c_void_p, c_uint32, c_void_p]
    L.aeon_b200_ctx_set_pool_slots.argtypes = [c_void_p, c_int]
    L.aeon_b200_ep_peer_create.argtypes = [c_void_p, c_int, c_int, c_int, POINTER(c_void_p)]
    L.aeon_b200_ep_peer_destroy.argtypes = [c_void_p]
    L.aeon_b200_ep_peer_set_wait_budget.argtypes = [c_void_p, ctypes.c_double]
    L.aeon_b200_moe_accumulate_push.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p]
    L.aeon_b200_ep_peer_combine.argtypes = [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p]
    L.aeon_b200_ep_peer_dispatch.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                             POINTER(c_void_p), POINTER(c_void_p), POINTER(c_void_p), c_void_p]
    L.aeon_b200_group_unique_id.argtypes = [c_void_p]
    L.aeon_b200_group_create.argtypes = [c_void_p, c_int, c_int, c_int, POINTER(c_void_p)]
    L.aeon_b200_group_destroy.argtypes = [c_void_p]
    L.aeon_b200_group_rank.argtypes = [c_void_p]
    L.aeon_b200_group_world.argtypes = [c_void_p]
    L.aeon_b200_ep_dispatch.argtypes = [c_void_p, c_void_p, c_int, c_int64, c_void_p, c_void_p]
    L.aeon_b200_ep_dispatch_routed.argtypes = [c_void_p, c_void_p, c_int, c_int64, c_void_p, c_void_p, c_void_p,
                                               c_int, c_void_p, c_void_p, c_void_p]
    L.aeon_b200_ep_exchange.argtypes = [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p]
    L.aeon_b200_tp_reduce.argtypes = [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p]
    L.aeon_b200_pp_send.argtypes = [c_void_p, c_void_p, c_uint64, c_int, c_void_p]
    L.aeon_b200_pp_recv.argtypes = [c_void_p, c_void_p, c_uint64, c_int, c_void_p]
    _lib = L
    return L


def check(status: int) -> None:
    if status != 0:
        raise AeonError(status, lib().aeon_b200_last_error().decode())


def bounds_checked() -> bool:
    """True when the library is the bounds-checked build (-DAEON_B200_BOUNDS=1)."""
    return bool(lib().aeon_b200_bounds_checked())


def preset(name: str) -> MoeConfig:
    cfg = MoeConfig()
    check(lib().aeon_b200_config_preset(name.encode(), ctypes.byref(cfg)))
    return cfg


def expert_layout(cfg: MoeConfig) -> ExpertLayout:
    out = ExpertLayout()
    check(lib().aeon_b200_expert_layout_of(ctypes.byref(cfg), ctypes.byref(out)))
    return out


def swizzle_w4a16(src_packed, src_scale, N, K, rpw, lpr, group, inverse=False):
    """Host re-layout of one matrix; numpy uint32 [N, K/8] and uint16 [N, K/group] in and out."""
    import numpy as np
    src_packed = np.ascontiguousarray(src_packed, dtype=np.uint32)
    src_scale = np.ascontiguousarray(src_scale, dtype=np.uint16)
    dst_packed = np.empty_like(src_packed)
    dst_scale = np.empty_like(src_scale)
    fn = lib().aeon_b200_unswizzle_w4a16 if inverse else lib().aeon_b200_swizzle_w4a16
    check(fn(src_packed.ctypes.data, src_scale.ctypes.data, dst_packed.ctypes.data,
             dst_scale.ctypes.data, N, K, rpw, lpr, group))
    return dst_packed, dst_scale


def expert_shard_bytes(cfg: MoeConfig, shards: int) -> int:
    """Bytes of one shard of an expert payload cut into `shards` intermediate-dimension shards."""
    out = c_uint64()
    check(lib().aeon_b200_expert_shard_bytes(ctypes.byref(cfg), shards, ctypes.byref(out)))
    return out.value


def source_shapes(cfg: MoeConfig):
    """Checkpoint-order shapes: (w1_packed, w1_scale, w2_packed, w2_scale, w3_packed, w3_scale)."""
    H, I, G = cfg.hidden, cfg.intermediate, cfg.group_size
    return ((I, H // 8), (I, H // G), (H, I // 8), (H, I // G), (I, H // 8), (I, H // G))


def pack_expert_shards(cfg: MoeConfig, shards: int, source):
    """Six checkpoint-order arrays (see source_shapes) -> payload of `shards` shards (numpy uint8)."""
    import numpy as np
    arrays = []
    for arr, shape, dtype in zip(source, source_shapes(cfg), (np.uint32, np.uint16) * 3):
        a = np.ascontiguousarray(arr, dtype=dtype)
        if a.shape != shape:
            raise AeonError(1, f"pack_expert_shards: source tensor has shape {a.shape}, expected {shape}")
        arrays.append(a)
    payload = np.empty(shards * expert_shard_bytes(cfg, shards), dtype=np.uint8)
    check(lib().aeon_b200_pack_expert_shards(ctypes.byref(cfg), shards, *[a.ctypes.data for a in arrays],
                                             payload.ctypes.data))
    return payload


def unpack_expert_shards(cfg: MoeConfig, shards: int, payload):
    """Inverse of pack_expert_shards: the six checkpoint-order arrays of the whole expert."""
    import numpy as np
    payload = np.ascontiguousarray(payload, dtype=np.uint8)
    if payload.size != shards * expert_shard_bytes(cfg, shards):
        raise AeonError(1, "unpack_expert_shards: payload size does not match shards * shard bytes")
    out = [np.empty(shape, dtype=dtype)
           for shape, dtype in zip(source_shapes(cfg), (np.uint32, np.uint16) * 3)]
    check(lib().aeon_b200_unpack_expert_shards(ctypes.byref(cfg), shards, payload.ctypes.data,
                                               *[a.ctypes.data for a in out]))
    return out


def expert_rank_slice(cfg: MoeConfig, shards: int, tp: int, rank: int):
    """(offset, length) in bytes, inside one payload, of the shards rank `rank` of `tp` reads."""
    off, length = c_uint64(), c_uint64()
    check(lib().aeon_b200_expert_rank_slice(ctypes.byref(cfg), shards, tp, rank, ctypes.byref(off),
                                            ctypes.byref(length)))
    return off.value, length.value


def merge_expert_shards(cfg_slice: MoeConfig, shards: int, slice_bytes):
    """A rank's slice of `shards` shards -> one payload of width cfg_slice.intermediate."""
    import numpy as np
    slice_bytes = np.ascontiguousarray(slice_bytes, dtype=np.uint8)
    if slice_bytes.size != shards * expert_shard_bytes(cfg_slice, shards):
        raise AeonError(1, "merge_expert_shards: slice size does not match shards * shard bytes")
    out = np.empty(expert_layout(cfg_slice).payload_bytes, dtype=np.uint8)
    check(lib().aeon_b200_merge_expert_shards(ctypes.byref(cfg_slice), shards, slice_bytes.ctypes.data,
                                              out.ctypes.data))
    return out


def _ptr(t):
    return None if t is None else c_void_p(t.data_ptr())


def _dense(t, name: str):
    """Pointer of a tensor the library reads or writes as one dense block."""
    if t is None:
        return None
    if not t.is_contiguous():
        raise AeonError(1, f"{name} must be contiguous (the library is given a bare pointer)")
    return c_void_p(t.data_ptr())


def _rows(t, name: str):
    """Pointer of a 2-D tensor passed with its row stride: the columns must be adjacent."""
    if t.dim() != 2 or t.stride(1) != 1:
        raise AeonError(1, f"{name} must be 2-D with unit column stride (rows may be strided)")
    return c_void_p(t.data_ptr())


def _stream():
    import torch
    return c_void_p(torch.cuda.current_stream().cuda_stream)


class ExpertPool:
    """One device slab of `slots` expert payloads (the reference's UnifiedVRAMExpertPool)."""

    def __init__(self, cfg: MoeConfig, slots: int, device: int = 0):
        import torch
        self.cfg = cfg
        self.layout = expert_layout(cfg)
        self.slots = slots
        self.device = device
        self.payload_bytes = int(self.layout.payload_bytes)
        # torch owns the slab so its caching allocator sees the memory.
        self.slab = torch.empty(self.payload_bytes * slots, dtype=torch.uint8,
                                device=f"cuda:{device}")

    @property
    def base(self) -> int:
        return self.slab.data_ptr()

    def upload(self, slot: int, payload) -> None:
        import torch
        if not 0 <= slot < self.slots:
            raise AeonError(4, f"slot {slot} outside the pool's {self.slots} slots")
        t = torch.as_tensor(payload).view(torch.uint8)
        if t.numel() != self.payload_bytes:
            raise AeonError(1, "payload size does not match the pool's payload_bytes")
        self.slab[slot * self.payload_bytes:(slot + 1) * self.payload_bytes].copy_(t)

    def fill_synthetic(self, first_slot: int, count: int, seed: int, layer: int,
                       first_expert: int, scale_table) -> None:
        check(lib().aeon_b200_synth_fill_experts(
            ctypes.byref(self.cfg), c_void_p(self.base), first_slot, count, seed, layer,
            first_expert, _ptr(scale_table), scale_table.numel(), _stream()))


def synth_fill_dense16(out, seed: int, layer: int, stream_id: int, table) -> None:
    check(lib().aeon_b200_synth_fill_dense16(_ptr(out), out.numel(), seed, layer, stream_id,
                                             _ptr(table), table.numel(), _stream()))


class Context:
    """Device scratch + the kernel entry points for one layer shape."""

    def __init__(self, cfg: MoeConfig, device: int = 0, max_tokens: int = 128):
        self.cfg = cfg
        self.device = device
        self.max_tokens = max_tokens
        handle = c_void_p()
        check(lib().aeon_b200_ctx_create(ctypes.byref(cfg), device, max_tokens, ctypes.byref(handle)))
        self._h = handle

    def close(self) -> None:
        if getattr(self, "_h", None):
            lib().aeon_b200_ctx_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def scratch_bytes(self) -> int:
        return int(lib().aeon_b200_ctx_scratch_bytes(self._h))

    @property
    def launches(self) -> int:
        return int(lib().aeon_b200_ctx_launches(self._h))

    def check(self) -> None:
        check(lib().aeon_b200_ctx_check(self._h, _stream()))

    def set_pool_slots(self, slots: int) -> None:
        """Declares the slot count of the pools this context is used with: a slot table entry at or
        above it is reported by check() instead of being used as an address."""
        check(lib().aeon_b200_ctx_set_pool_slots(self._h, slots))

    def last_stats(self):
        distinct, entries = c_int32(), c_int32()
        check(lib().aeon_b200_ctx_last_stats(self._h, _stream(), ctypes.byref(distinct),
                                             ctypes.byref(entries)))
        return distinct.value, entries.value

    def set_timing(self, enabled: bool) -> None:
        check(lib().aeon_b200_ctx_set_timing(self._h, int(enabled)))

    def kernel_times(self):
        """((ms_w13, launches), (ms_w2, launches)) since the last call."""
        ms = (ctypes.c_double * 2)()
        n = (c_int64 * 2)()
        check(lib().aeon_b200_ctx_kernel_times(self._h, _stream(), ms, n))
        return (ms[0], n[0]), (ms[1], n[1])

    def router_topk(self, x, gate, bias=None, hash_table=None, token_ids=None, logits_out=None):
        import torch
        tokens = x.shape[0]
        k = self.cfg.top_k
        weights = torch.empty(tokens, k, dtype=torch.float32, device=x.device)
        ids = torch.empty(tokens, k, dtype=torch.int32, device=x.device)
        check(lib().aeon_b200_router_topk(self._h, _rows(x, "x"), x.stride(0), _dense(gate, "gate"),
                                          _dense(bias, "bias"), _dense(hash_table, "hash_table"),
                                          _dense(token_ids, "token_ids"), tokens, _ptr(weights),
                                          _ptr(ids), _dense(logits_out, "logits_out"), _stream()))
        return weights, ids

    def expert_permutation(self, ids, experts=None, weights=None):
        import torch
        tokens, slots = ids.shape
        experts = experts or self.cfg.experts
        dev = ids.device
        offsets = torch.empty(experts + 1, dtype=torch.int32, device=dev)
        token_idx = torch.full((tokens * slots,), -1, dtype=torch.int32, device=dev)
        draw_idx = torch.full((tokens * slots,), -1, dtype=torch.int32, device=dev)
        wpos = torch.zeros(tokens * slots, dtype=torch.float32, device=dev) if weights is not None else None
        check(lib().aeon_b200_expert_permutation(self._h, _dense(ids, "ids"), tokens, slots, experts,
                                                 _ptr(offsets), _ptr(token_idx), _ptr(draw_idx),
                                                 _dense(weights, "weights"), _ptr(wpos), _stream()))
        return offsets, token_idx, draw_idx, wpos

    def shared_expert(self, w1, w3, w2, x, moe_accum):
        check(lib().aeon_b200_shared_expert(self._h, _dense(w1, "w1"), _dense(w3, "w3"), _dense(w2, "w2"),
                                            _rows(x, "x"), x.stride(0), x.shape[0],
                                            _rows(moe_accum, "moe_accum"), moe_accum.stride(0), _stream()))

    def moe_decode(self, pool_base: int, slot_of_expert, x, ids, weights, moe_accum,
                   skip_absent: bool = False, defer_accumulate: bool = False, overwrite: bool = False):
        flags = ((DECODE_SKIP_ABSENT if skip_absent else 0) | (DECODE_DEFER_ACCUMULATE if defer_accumulate else 0) |
                 (DECODE_OVERWRITE if overwrite else 0))
        check(lib().aeon_b200_moe_decode(self._h, c_void_p(pool_base), _dense(slot_of_expert, "slot_of_expert"),
                                         _rows(x, "x"), x.stride(0), _dense(ids, "ids"),
                                         _dense(weights, "weights"), x.shape[0],
                                         _rows(moe_accum, "moe_accum"), moe_accum.stride(0), flags, _stream()))

    def moe_accumulate(self, slot_of_expert, ids, moe_accum, skip_absent: bool = False,
                       overwrite: bool = False):
        check(lib().aeon_b200_moe_accumulate(self._h, _dense(slot_of_expert, "slot_of_expert"),
                                             _dense(ids, "ids"), ids.shape[0],
                                             _rows(moe_accum, "moe_accum"), moe_accum.stride(0),
                                             (DECODE_SKIP_ABSENT if skip_absent else 0) |
                                             (DECODE_OVERWRITE if overwrite else 0), _stream()))


def hc_params_default() -> HcParams:
    out = HcParams()
    check(lib().aeon_b200_hc_params_default(ctypes.byref(out)))
    return out


def _hc_ffn_front(self, res_mid, hc_fn, hc_base, hc_scale3, norm_weight, params: HcParams | None = None):
    """res_mid [T, 4, H] 16-bit -> (ffn_norm [T, H] 16-bit, pre [T, 4], post [T, 4], comb [T, 16])."""
    import torch
    T, H = res_mid.shape[0], res_mid.shape[2]
    params = params or hc_params_default()
    ffn_norm = torch.empty(T, H, dtype=res_mid.dtype, device=res_mid.device)
    pre = torch.empty(T, 4, dtype=torch.float32, device=res_mid.device)
    post = torch.empty_like(pre)
    comb = torch.empty(T, 16, dtype=torch.float32, device=res_mid.device)
    check(lib().aeon_b200_hc_ffn_front(self._h, _ptr(res_mid), _ptr(hc_fn), _ptr(hc_base), _ptr(hc_scale3),
                                       _ptr(norm_weight), T, ctypes.byref(params), _ptr(ffn_norm),
                                       ffn_norm.stride(0), _ptr(pre), _ptr(post), _ptr(comb), _stream()))
    return ffn_norm, pre, post, comb


def _hc_post(self, moe_out, res_mid, post, comb):
    """res_out [T, 4, H] 16-bit = post * moe_out + comb^T . res_mid."""
    import torch
    res_out = torch.empty_like(res_mid)
    check(lib().aeon_b200_hc_post(self._h, _ptr(moe_out), moe_out.stride(0), _ptr(res_mid), _ptr(post),
                                  _ptr(comb), res_mid.shape[0], _ptr(res_out), _stream()))
    return res_out


def _moe_prefill(self, pool_base: int, slot_of_expert, x, ids, weights, moe_accum,
                 skip_absent: bool = False, overwrite: bool = False):
    check(lib().aeon_b200_moe_prefill(self._h, c_void_p(pool_base), _dense(slot_of_expert, "slot_of_expert"),
                                      _rows(x, "x"), x.stride(0), _dense(ids, "ids"),
                                      _dense(weights, "weights"), x.shape[0],
                                      _rows(moe_accum, "moe_accum"), moe_accum.stride(0),
                                      (DECODE_SKIP_ABSENT if skip_absent else 0) |
                                      (DECODE_OVERWRITE if overwrite else 0), _stream()))


Context.moe_prefill = _moe_prefill
Context.hc_ffn_front = _hc_ffn_front
Context.hc_post = _hc_post


def router_topk_noalloc(cfg: MoeConfig, x, gate, weights_out, ids_out, bias=None) -> None:
    """Router without a context and without any allocation: every buffer, outputs included,
    is the caller's; the logits scratch is built into the library (<= 64 tokens, <= 1024
    experts). For callers that cannot call cudaMalloc at the point of use."""
    check(lib().aeon_b200_router_topk_noalloc(ctypes.byref(cfg), _rows(x, "x"), x.stride(0), _dense(gate, "gate"),
                                              _dense(bias, "bias"), x.shape[0], _dense(weights_out, "weights_out"),
                                              _dense(ids_out, "ids_out"), _stream()))


def ep_combine(out, partials) -> None:
    """out[t, :] += sum_r partials[r, t, :] in rank order (fp32)."""
    ranks, tokens, hidden = partials.shape
    check(lib().aeon_b200_ep_combine(_rows(out, "out"), out.stride(0), _dense(partials, "partials"), ranks,
                                     tokens, hidden, _stream()))


GROUP_ID_BYTES = 128


def group_unique_id() -> bytes:
    """The 128-byte id one rank creates and hands to the others (any host channel)."""
    buf = ctypes.create_string_buffer(GROUP_ID_BYTES)
    check(lib().aeon_b200_group_unique_id(buf))
    return buf.raw


class Group:
    """This rank's membership of a multi-GPU group (the library's own NCCL communicator).

    The data-path collectives of expert / tensor / pipeline parallelism go through the C ABI,
    so a C++ host and this binding share one path. The methods named like torch.distributed's
    (all_gather_into_tensor, all_to_all_single, reduce_scatter_tensor, send, recv) let the
    protocol functions of aeon_b200.stack run over a Group or over a torch process group."""

    def __init__(self, unique_id: bytes, rank: int, world: int, device: int):
        if len(unique_id) != GROUP_ID_BYTES:
            raise AeonError(1, "a group id is 128 bytes")
        handle = c_void_p()
        check(lib().aeon_b200_group_create(unique_id, rank, world, device, ctypes.byref(handle)))
        self._h, self.rank, self.world, self.device = handle, rank, world, device

    @classmethod
    def from_process_group(cls, dist, device: int, group=None):
        """Bootstraps over an initialised torch.distributed group: rank 0's id is broadcast."""
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        box = [group_unique_id() if rank == 0 else None]
        src = 0 if group is None else dist.get_global_rank(group, 0)
        dist.broadcast_object_list(box, src=src, group=group)
        return cls(box[0], rank, world, device)

    def close(self) -> None:
        if getattr(self, "_h", None):
            check(lib().aeon_b200_group_destroy(self._h))
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def get_rank(self) -> int:
        return self.rank

    def get_world_size(self) -> int:
        return self.world

    # -- the C ABI calls ----------------------------------------------------------------------
    def ep_dispatch(self, x_local, x_all) -> None:
        row_bytes = x_local.shape[1] * x_local.element_size()
        check(lib().aeon_b200_ep_dispatch(self._h, _dense(x_local, "x_local"), x_local.shape[0], row_bytes,
                                          _dense(x_all, "x_all"), _stream()))

    def ep_dispatch_routed(self, x_local, x_all, ids_local, weights_local, ids_all, weights_all) -> None:
        """The dispatch plus the all-gather of the routing each rank computed for its own tokens."""
        row_bytes = x_local.shape[1] * x_local.element_size()
        check(lib().aeon_b200_ep_dispatch_routed(self._h, _dense(x_local, "x_local"), x_local.shape[0], row_bytes,
                                                 _dense(x_all, "x_all"), _dense(ids_local, "ids_local"),
                                                 _dense(weights_local, "weights_local"), ids_local.shape[1],
                                                 _dense(ids_all, "ids_all"), _dense(weights_all, "weights_all"),
                                                 _stream()))

    def ep_exchange(self, partial, recv) -> None:
        tl = partial.shape[0] // self.world
        check(lib().aeon_b200_ep_exchange(self._h, _dense(partial, "partial"), tl, partial.shape[1],
                                          _dense(recv, "recv"), _stream()))

    def tp_reduce(self, partial, out_local) -> None:
        check(lib().aeon_b200_tp_reduce(self._h, _dense(partial, "partial"), out_local.shape[0],
                                        out_local.shape[1], _dense(out_local, "out_local"), _stream()))

    # -- torch.distributed-shaped names, for the protocol functions ------------------------------
    def all_gather_into_tensor(self, out, inp, group=None) -> None:
        self.ep_dispatch(inp, out)

    def all_to_all_single(self, out, inp, group=None) -> None:
        self.ep_exchange(inp, out)

    def reduce_scatter_tensor(self, out, inp, group=None) -> None:
        self.tp_reduce(inp, out)

    def send(self, tensor, dst: int) -> None:
        check(lib().aeon_b200_pp_send(self._h, _dense(tensor, "tensor"), tensor.numel() * tensor.element_size(),
                                      dst, _stream()))

    def recv(self, tensor, src: int) -> None:
        check(lib().aeon_b200_pp_recv(self._h, _dense(tensor, "tensor"), tensor.numel() * tensor.element_size(),
                                      src, _stream()))


class _DevicePointer:
    """A device buffer owned by the library, seen through the CUDA array interface."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (int(ptr), False),
                                         "version": 2, "strides": None}


def _device_view(ptr: int, shape, typestr: str, device):
    import torch
    return torch.as_tensor(_DevicePointer(ptr, shape, typestr), device=device)


class PeerCombine:
    """Receive buffers of an expert-parallel group mapped between the ranks of one box (CUDA IPC),
    for the combine that is fused with the slot-order accumulate: push() is the second half of a
    deferred decode call and stores every finished row straight into its owner's buffer, combine()
    waits (bounded) for all ranks' rows and adds them in rank order. Creation is collective."""

    def __init__(self, group: Group, device: int, tokens_local_max: int, hidden: int):
        handle = c_void_p()
        check(lib().aeon_b200_ep_peer_create(group._h, device, tokens_local_max, hidden, ctypes.byref(handle)))
        self._h, self.group = handle, group

    def close(self) -> None:
        if getattr(self, "_h", None):
            check(lib().aeon_b200_ep_peer_destroy(self._h))
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_wait_budget(self, milliseconds: float) -> None:
        check(lib().aeon_b200_ep_peer_set_wait_budget(self._h, float(milliseconds)))

    def dispatch(self, ctx: Context, x_local, ids_local, weights_local):
        """Peer-memory dispatch: returns (x_all, ids_all, weights_all), views of this rank's gather
        buffers (overwritten by the next dispatch), filled once the stream reaches this point."""
        import torch
        tl, hidden = x_local.shape
        k = ids_local.shape[1]
        px, pi, pw = c_void_p(), c_void_p(), c_void_p()
        check(lib().aeon_b200_ep_peer_dispatch(ctx._h, self._h, _dense(x_local, "x_local"), tl,
                                               _dense(ids_local, "ids_local"), _dense(weights_local, "weights_local"),
                                               ctypes.byref(px), ctypes.byref(pi), ctypes.byref(pw), _stream()))
        key = (tl, hidden, k, x_local.dtype)
        if getattr(self, "_views_key", None) != key:
            tokens = tl * self.group.world
            dev = x_local.device
            x_all = _device_view(px.value, (tokens, hidden), "<i2", dev).view(x_local.dtype)
            ids_all = _device_view(pi.value, (tokens, k), "<i4", dev)
            weights_all = _device_view(pw.value, (tokens, k), "<f4", dev)
            self._views, self._views_key = (x_all, ids_all, weights_all), key
        return self._views

    def push(self, ctx: Context, slot_of_expert, ids, tokens_local: int) -> None:
        check(lib().aeon_b200_moe_accumulate_push(ctx._h, self._h, _dense(slot_of_expert, "slot_of_expert"),
                                                  _dense(ids, "ids"), tokens_local, _stream()))

    def combine(self, ctx: Context, out) -> None:
        check(lib().aeon_b200_ep_peer_combine(ctx._h, self._h, _rows(out, "out"), out.stride(0), out.shape[0],
                                              _stream()))
