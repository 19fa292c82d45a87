"""ctypes binding of the CPU oracle (oracle/liboracle.so). Test infrastructure only."""
from __future__ import annotations

import ctypes
import os
import subprocess
from ctypes import POINTER, c_double, c_int, c_int32, c_int64, c_uint16, c_uint32, c_uint64, c_void_p

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
LIB = os.path.join(ORACLE_DIR, "liboracle.so")


class LayoutArgs(ctypes.Structure):
    _fields_ = [(n, c_int) for n in ("hidden", "intermediate", "group", "w13_rpw", "w13_lpr",
                                      "w2_rpw", "w2_lpr")]


def _load():
    src_time = max(os.path.getmtime(os.path.join(ORACLE_DIR, f))
                   for f in ("aeon_oracle.hpp", "oracle_capi.cpp"))
    if not os.path.exists(LIB) or os.path.getmtime(LIB) < src_time:
        subprocess.run(["make", "-C", ORACLE_DIR, os.path.join(ORACLE_DIR, "liboracle.so")],
                       check=True, capture_output=True)
    L = ctypes.CDLL(LIB)
    L.ao_last_error.restype = ctypes.c_char_p
    L.ao_clamped_swiglu.restype = c_double
    L.ao_clamped_swiglu.argtypes = [c_double, c_double, c_double, c_int]
    L.ao_fnv1a.restype = c_uint64
    L.ao_fnv1a.argtypes = [c_void_p, c_uint64]
    return L


_L = _load()


def _chk(rc):
    if rc != 0:
        raise RuntimeError(_L.ao_last_error().decode())


def layout_args(cfg) -> LayoutArgs:
    return LayoutArgs(cfg.hidden, cfg.intermediate, cfg.group_size, cfg.w13_rpw, cfg.w13_lpr,
                      cfg.w2_rpw, cfg.w2_lpr)


def threads() -> int:
    return _L.ao_threads()


def set_threads(n: int) -> int:
    """Thread count of the oracle's parallel loops from now on; returns the count in force."""
    return _L.ao_set_threads(int(n))


def layout(la: LayoutArgs) -> dict:
    out = (c_uint64 * 22)()
    _chk(_L.ao_layout(ctypes.byref(la), out))
    d = {"payload_bytes": out[0]}
    for m, name in enumerate(("w1", "w2", "w3")):
        o = out[1 + 7 * m: 8 + 7 * m]
        d[name] = dict(packed_offset=o[0], scale_offset=o[1], rows=o[2], cols=o[3], rpw=o[4],
                       lpr=o[5], iters=o[6])
    return d


def swizzled_address(la, kind, row, col):
    out = (c_uint64 * 3)()
    _chk(_L.ao_swizzled_address(ctypes.byref(la), kind, row, col, out))
    return int(out[0]), int(out[1]), int(out[2])


def rng_fill(seed: int, scale: float, n: int) -> np.ndarray:
    out = np.empty(n, dtype=np.float64)
    _chk(_L.ao_rng_fill(c_uint64(seed), c_double(scale), c_uint64(n), out.ctypes.data_as(c_void_p)))
    return out


def rng_u64(seed: int, n: int) -> np.ndarray:
    out = np.empty(n, dtype=np.uint64)
    _chk(_L.ao_rng_u64(c_uint64(seed), c_uint64(n), out.ctypes.data_as(c_void_p)))
    return out


def half_bits_to_double(bits) -> np.ndarray:
    bits = np.ascontiguousarray(bits, dtype=np.uint16)
    out = np.empty(bits.shape, dtype=np.float64)
    _chk(_L.ao_half_bits_to_double(bits.ctypes.data_as(c_void_p), c_uint64(bits.size),
                                   out.ctypes.data_as(c_void_p)))
    return out


def double_to_half_bits(v) -> np.ndarray:
    v = np.ascontiguousarray(v, dtype=np.float64)
    out = np.empty(v.shape, dtype=np.uint16)
    _chk(_L.ao_double_to_half_bits(v.ctypes.data_as(c_void_p), c_uint64(v.size),
                                   out.ctypes.data_as(c_void_p)))
    return out


def synth_expert_payload(la, seed, layer, expert, table) -> np.ndarray:
    n = layout(la)["payload_bytes"]
    out = np.empty(n, dtype=np.uint8)
    table = np.ascontiguousarray(table, dtype=np.uint16)
    _chk(_L.ao_synth_expert_payload(ctypes.byref(la), out.ctypes.data_as(c_void_p), c_uint64(seed),
                                    c_uint32(layer), c_uint32(expert),
                                    table.ctypes.data_as(c_void_p), c_uint32(table.size)))
    return out


def synth_dense16(count, seed, layer, stream, table) -> np.ndarray:
    out = np.empty(count, dtype=np.uint16)
    table = np.ascontiguousarray(table, dtype=np.uint16)
    _chk(_L.ao_synth_dense16(out.ctypes.data_as(c_void_p), c_uint64(count), c_uint64(seed),
                             c_uint32(layer), c_uint32(stream), table.ctypes.data_as(c_void_p),
                             c_uint32(table.size)))
    return out


def decode_matrix(la, kind, payload, mode=0) -> np.ndarray:
    lay = layout(la)[("w1", "w2", "w3")[kind]]
    out = np.empty((lay["rows"], lay["cols"]), dtype=np.float64)
    payload = np.ascontiguousarray(payload, dtype=np.uint8)
    _chk(_L.ao_decode_matrix(ctypes.byref(la), kind, payload.ctypes.data_as(c_void_p), mode,
                             out.ctypes.data_as(c_void_p)))
    return out


def encode_matrix(la, kind, payload, w) -> None:
    w = np.ascontiguousarray(w, dtype=np.float64)
    _chk(_L.ao_encode_matrix(ctypes.byref(la), kind, payload.ctypes.data_as(c_void_p),
                             w.ctypes.data_as(c_void_p)))


def swizzle_from_source(la, kind, src_packed, src_scale, payload) -> None:
    src_packed = np.ascontiguousarray(src_packed, dtype=np.uint32)
    src_scale = np.ascontiguousarray(src_scale, dtype=np.uint16)
    _chk(_L.ao_swizzle_from_source(ctypes.byref(la), kind, src_packed.ctypes.data_as(c_void_p),
                                   src_scale.ctypes.data_as(c_void_p),
                                   payload.ctypes.data_as(c_void_p)))


def router_logits_f64(gate_bits, gate_dtype, x_bits, x_dtype) -> np.ndarray:
    gate_bits = np.ascontiguousarray(gate_bits, dtype=np.uint16)
    x_bits = np.ascontiguousarray(x_bits, dtype=np.uint16)
    E, H = gate_bits.shape
    T = x_bits.shape[0]
    out = np.empty((T, E), dtype=np.float64)
    _chk(_L.ao_router_logits_f64(gate_bits.ctypes.data_as(c_void_p), gate_dtype, E, H,
                                 x_bits.ctypes.data_as(c_void_p), x_dtype, T, x_bits.shape[1],
                                 out.ctypes.data_as(c_void_p)))
    return out


def router_logits_f32_ordered(gate_bits, gate_dtype, x_bits, x_dtype) -> np.ndarray:
    gate_bits = np.ascontiguousarray(gate_bits, dtype=np.uint16)
    x_bits = np.ascontiguousarray(x_bits, dtype=np.uint16)
    E, H = gate_bits.shape
    T = x_bits.shape[0]
    out = np.empty((T, E), dtype=np.float32)
    _chk(_L.ao_router_logits_f32_ordered(gate_bits.ctypes.data_as(c_void_p), gate_dtype, E, H,
                                         x_bits.ctypes.data_as(c_void_p), x_dtype, T,
                                         x_bits.shape[1], out.ctypes.data_as(c_void_p)))
    return out


def router_topk(logits, bias, top_k, scaling, score_fn, renormalize=True, bias_before_score=False):
    logits = np.ascontiguousarray(logits, dtype=np.float64)
    T, E = logits.shape
    ids = np.empty((T, top_k), dtype=np.int32)
    w = np.empty((T, top_k), dtype=np.float64)
    margin = np.empty(T, dtype=np.float64)
    b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float64)
    _chk(_L.ao_router_topk(logits.ctypes.data_as(c_void_p),
                           None if b is None else b.ctypes.data_as(c_void_p), T, E, top_k,
                           c_double(scaling), score_fn, int(renormalize), int(bias_before_score),
                           ids.ctypes.data_as(c_void_p), w.ctypes.data_as(c_void_p),
                           margin.ctypes.data_as(c_void_p)))
    return ids, w, margin


def router_hash(logits, table_row, scaling, score_fn):
    logits = np.ascontiguousarray(logits, dtype=np.float64)
    row = np.ascontiguousarray(table_row, dtype=np.int64)
    ids = np.empty(row.size, dtype=np.int32)
    w = np.empty(row.size, dtype=np.float64)
    _chk(_L.ao_router_hash(logits.ctypes.data_as(c_void_p), logits.size,
                           row.ctypes.data_as(c_void_p), row.size, c_double(scaling), score_fn,
                           ids.ctypes.data_as(c_void_p), w.ctypes.data_as(c_void_p)))
    return ids, w


def topk_indices(scores, k) -> np.ndarray:
    scores = np.ascontiguousarray(scores, dtype=np.float64)
    out = np.empty(k, dtype=np.int32)
    _chk(_L.ao_topk_indices(scores.ctypes.data_as(c_void_p), scores.size, k,
                            out.ctypes.data_as(c_void_p)))
    return out


def clamped_swiglu(gate, up, limit=10.0, mode=0) -> float:
    return _L.ao_clamped_swiglu(gate, up, limit, mode)


def expert_ffn(la, payload, x, limit=10.0, clamp_mode=0, want_pre=False):
    x = np.ascontiguousarray(x, dtype=np.float64)
    payload = np.ascontiguousarray(payload, dtype=np.uint8)
    out = np.empty(la.hidden, dtype=np.float64)
    hid = np.empty(la.intermediate, dtype=np.float64)
    gate = np.empty(la.intermediate, dtype=np.float64)
    up = np.empty(la.intermediate, dtype=np.float64)
    _chk(_L.ao_expert_ffn(ctypes.byref(la), payload.ctypes.data_as(c_void_p),
                          x.ctypes.data_as(c_void_p), c_double(limit), clamp_mode,
                          out.ctypes.data_as(c_void_p), hid.ctypes.data_as(c_void_p),
                          gate.ctypes.data_as(c_void_p), up.ctypes.data_as(c_void_p)))
    return (out, hid, gate, up) if want_pre else out


def expert_ffn_batch(la, payload, x, limit=10.0) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float64)
    payload = np.ascontiguousarray(payload, dtype=np.uint8)
    out = np.empty_like(x)
    _chk(_L.ao_expert_ffn_batch(ctypes.byref(la), payload.ctypes.data_as(c_void_p),
                                x.ctypes.data_as(c_void_p), x.shape[0], c_double(limit),
                                out.ctypes.data_as(c_void_p)))
    return out


def dense_ffn(w1, w3, w2, dtype, x, limit=10.0) -> np.ndarray:
    w1 = np.ascontiguousarray(w1, dtype=np.uint16)
    w3 = np.ascontiguousarray(w3, dtype=np.uint16)
    w2 = np.ascontiguousarray(w2, dtype=np.uint16)
    I, H = w1.shape
    x = np.ascontiguousarray(x, dtype=np.float64)
    out = np.empty(H, dtype=np.float64)
    _chk(_L.ao_dense_ffn(w1.ctypes.data_as(c_void_p), w3.ctypes.data_as(c_void_p),
                         w2.ctypes.data_as(c_void_p), dtype, I, H, x.ctypes.data_as(c_void_p),
                         c_double(limit), out.ctypes.data_as(c_void_p)))
    return out


def moe_combine(expert_out, weights, shared=None) -> np.ndarray:
    expert_out = np.ascontiguousarray(expert_out, dtype=np.float64)
    weights = np.ascontiguousarray(weights, dtype=np.float64)
    k, H = expert_out.shape
    out = np.empty(H, dtype=np.float64)
    sh = None if shared is None else np.ascontiguousarray(shared, dtype=np.float64)
    _chk(_L.ao_moe_combine(expert_out.ctypes.data_as(c_void_p), weights.ctypes.data_as(c_void_p),
                           k, H, None if sh is None else sh.ctypes.data_as(c_void_p),
                           out.ctypes.data_as(c_void_p)))
    return out


def compare(want, got, rel_floor=1e-3) -> dict:
    want = np.ascontiguousarray(want, dtype=np.float64).ravel()
    got = np.ascontiguousarray(got, dtype=np.float64).ravel()
    assert want.size == got.size
    stats = (c_double * 4)()
    _chk(_L.ao_compare(want.ctypes.data_as(c_void_p), got.ctypes.data_as(c_void_p),
                       c_uint64(want.size), c_double(rel_floor), stats))
    return dict(max_abs=stats[0], max_rel=stats[1], rms_abs=stats[2], rel_l2=stats[3])


def fnv1a(array) -> int:
    a = np.ascontiguousarray(array)
    return int(_L.ao_fnv1a(a.ctypes.data_as(c_void_p), a.nbytes))


def dense_ffn_f64(w1, w3, w2, x, limit=10.0) -> np.ndarray:
    w1 = np.ascontiguousarray(w1, dtype=np.float64)
    w3 = np.ascontiguousarray(w3, dtype=np.float64)
    w2 = np.ascontiguousarray(w2, dtype=np.float64)
    I, H = w1.shape
    x = np.ascontiguousarray(x, dtype=np.float64)
    out = np.empty(H, dtype=np.float64)
    _chk(_L.ao_dense_ffn_f64(w1.ctypes.data_as(c_void_p), w3.ctypes.data_as(c_void_p),
                             w2.ctypes.data_as(c_void_p), I, H, x.ctypes.data_as(c_void_p),
                             c_double(limit), out.ctypes.data_as(c_void_p)))
    return out


def ffn_front(res_mid, hc_fn, hc_base, hc_scale3, norm_weight=None, norm_eps=1e-6) -> dict:
    """Hyper-connection pre-mix + FFN RMSNorm: res_mid [hc, hidden] fp64, hc_fn fp32
    [hc*(hc+2), hc*hidden], hc_base fp32 [hc*(hc+2)], hc_scale3 fp32 [3]."""
    res_mid = np.ascontiguousarray(res_mid, dtype=np.float64)
    hc, hidden = res_mid.shape
    fn = np.ascontiguousarray(hc_fn, dtype=np.float32)
    base = np.ascontiguousarray(hc_base, dtype=np.float32)
    scale = np.ascontiguousarray(hc_scale3, dtype=np.float32)
    assert fn.shape == (hc * (hc + 2), hc * hidden) and base.shape == (hc * (hc + 2),) and scale.shape == (3,)
    w = None if norm_weight is None else np.ascontiguousarray(norm_weight, dtype=np.float64)
    out = dict(mixes=np.empty(hc * (hc + 2)), pre=np.empty(hc), post=np.empty(hc), comb=np.empty((hc, hc)),
               ffn_pre=np.empty(hidden), ffn_norm=np.empty(hidden))
    _chk(_L.ao_ffn_front(res_mid.ctypes.data_as(c_void_p), hidden, hc, fn.ctypes.data_as(c_void_p),
                         base.ctypes.data_as(c_void_p), scale.ctypes.data_as(c_void_p),
                         None if w is None else w.ctypes.data_as(c_void_p), c_double(norm_eps),
                         *[out[k].ctypes.data_as(c_void_p)
                           for k in ("mixes", "pre", "post", "comb", "ffn_pre", "ffn_norm")]))
    return out


def hc_post(layer_out, residual, post_mix, comb, transpose_comb=False) -> np.ndarray:
    """out[j][h] = post_mix[j] * layer_out[h] + sum_i comb[i][j] * residual[i][h]."""
    residual = np.ascontiguousarray(residual, dtype=np.float64)
    hc, hidden = residual.shape
    layer_out = np.ascontiguousarray(layer_out, dtype=np.float64)
    post_mix = np.ascontiguousarray(post_mix, dtype=np.float64)
    comb = np.ascontiguousarray(comb, dtype=np.float64)
    out = np.empty((hc, hidden))
    _chk(_L.ao_hc_post(layer_out.ctypes.data_as(c_void_p), residual.ctypes.data_as(c_void_p),
                       post_mix.ctypes.data_as(c_void_p), comb.ctypes.data_as(c_void_p), hidden, hc,
                       int(transpose_comb), out.ctypes.data_as(c_void_p)))
    return out
