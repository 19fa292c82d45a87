"""Helpers shared by the GPU parity tests (and the smoke check): seeded inputs as the
benchmark configurations describe them, device pools filled by the library's synthetic
generators, and the oracle evaluation of a routed batch."""
from __future__ import annotations

import numpy as np

import aeon_b200
from aeon_b200 import synth

TOL_MAX_ABS = 2e-2      # layer-output tolerance of the benchmark contract
TOL_REL_L2 = 1e-3


def torch_bits(bits: np.ndarray, dtype: int, device="cuda"):
    import torch
    t = torch.from_numpy(bits.view(np.int16).copy()).to(device)
    return t.view(torch.bfloat16 if dtype == aeon_b200.BF16 else torch.float16)


class SyntheticLayer:
    """One MoE layer's weights on the device, generated from (seed, layer)."""

    def __init__(self, cfg, experts_resident=None, seed=0, layer=0, device=0, with_shared=True):
        import torch
        self.cfg, self.seed, self.layer = cfg, seed, layer
        self.dev = f"cuda:{device}"
        E = cfg.experts
        self.resident = list(range(E)) if experts_resident is None else list(experts_resident)
        self.scale_table = synth.half_normal_table(0.02, 1e-4, 4096, dtype=aeon_b200.F16)
        self.d_scale_table = torch.from_numpy(self.scale_table.view(np.int16).copy()).to(self.dev)
        self.pool = aeon_b200.ExpertPool(cfg, len(self.resident), device)
        slot_of = np.full(E, -1, dtype=np.int32)
        # contiguous runs of expert ids are filled with one call each
        run_start = 0
        for i in range(1, len(self.resident) + 1):
            if i == len(self.resident) or self.resident[i] != self.resident[i - 1] + 1:
                self.pool.fill_synthetic(run_start, i - run_start, seed, layer,
                                         self.resident[run_start], self.d_scale_table)
                run_start = i
        for slot, e in enumerate(self.resident):
            slot_of[e] = slot
        self.slot_of = torch.from_numpy(slot_of).to(self.dev)
        rng = np.random.default_rng([seed, layer, 0x6A7E])
        self.gate_bits = synth.normal_bits(rng, (E, cfg.hidden), 0.01, cfg.act_dtype)
        self.gate = torch_bits(self.gate_bits, cfg.act_dtype, self.dev)
        self.shared = None
        if with_shared:
            self.dense_table = synth.half_normal_table(0.02, 0.0, 4096, dtype=cfg.act_dtype)
            d_table = torch.from_numpy(self.dense_table.view(np.int16).copy()).to(self.dev)
            n = cfg.hidden * cfg.intermediate
            bufs = []
            for stream_id in range(3):
                t = torch.empty(n, dtype=torch.int16, device=self.dev)
                aeon_b200.synth_fill_dense16(t, seed, layer, stream_id, d_table)
                bufs.append(t)
            self.shared = bufs   # w1 [I,H], w3 [I,H], w2 [H,I] as raw 16-bit

    def shared_bits(self, oracle):
        cfg = self.cfg
        n = cfg.hidden * cfg.intermediate
        w1 = oracle.synth_dense16(n, self.seed, self.layer, 0, self.dense_table).reshape(cfg.intermediate, cfg.hidden)
        w3 = oracle.synth_dense16(n, self.seed, self.layer, 1, self.dense_table).reshape(cfg.intermediate, cfg.hidden)
        w2 = oracle.synth_dense16(n, self.seed, self.layer, 2, self.dense_table).reshape(cfg.hidden, cfg.intermediate)
        return w1, w3, w2


def activations(cfg, tokens, seed=0, scale=1.0):
    rng = np.random.default_rng([seed, 0xAC7])
    return synth.normal_bits(rng, (tokens, cfg.hidden), scale, cfg.act_dtype)


def oracle_routed(oracle, layer: SyntheticLayer, x_bits, ids, weights, token_subset=None):
    """fp64 routed sum, slot order, for the chosen tokens: {token: vector[H]}."""
    cfg = layer.cfg
    la = oracle.layout_args(cfg)
    x = synth.from_bits16(x_bits, cfg.act_dtype)
    tokens = range(x.shape[0]) if token_subset is None else token_subset
    by_expert = {}
    for t in tokens:
        for slot in range(ids.shape[1]):
            by_expert.setdefault(int(ids[t, slot]), []).append((t, slot))
    outs = {}
    for e, uses in sorted(by_expert.items()):
        payload = oracle.synth_expert_payload(la, layer.seed, layer.layer, e, layer.scale_table)
        toks = sorted({t for t, _ in uses})
        y = oracle.expert_ffn_batch(la, payload, x[toks], cfg.swiglu_limit)
        for t, slot in uses:
            outs[(t, slot)] = y[toks.index(t)]
    result = {}
    for t in tokens:
        eo = np.stack([outs[(t, s)] for s in range(ids.shape[1])])
        result[t] = oracle.moe_combine(eo, weights[t])
    return result


def mirrored_oracle(oracle, layer, x_bits, ids, weights, tokens):
    """The oracle for the grouped (prefill) path: fp64 accumulation over the operands that path feeds
    its tensor-core MMAs -- weights fp16(q * scale), activations fp16, hidden vector rounded to fp16
    between the two GEMMs -- combined in slot order, for the chosen tokens: {token: vector[H]}.
    The reference gates its own grouped kernels the same way
    (tests/test_v4_grouped_wmma_oracle.cpp:63-73,219-228)."""
    cfg = layer.cfg
    la = oracle.layout_args(cfg)
    x16 = synth.from_bits16(x_bits, cfg.act_dtype).astype(np.float16).astype(np.float64)
    L = cfg.swiglu_limit
    cache = {}
    out = {}
    for t in tokens:
        acc = np.zeros(cfg.hidden)
        for s in range(ids.shape[1]):
            e = int(ids[t, s])
            if e not in cache:
                payload = oracle.synth_expert_payload(la, layer.seed, layer.layer, e, layer.scale_table)
                cache[e] = [oracle.decode_matrix(la, k, payload).astype(np.float16).astype(np.float64)
                            for k in (0, 2, 1)]
            w1, w3, w2 = cache[e]
            gate = np.minimum(w1 @ x16[t], L)
            up = np.clip(w3 @ x16[t], -L, L)
            h = (gate / (1.0 + np.exp(-gate)) * up).astype(np.float16).astype(np.float64)
            acc += float(weights[t, s]) * (w2 @ h)
        out[t] = acc
    return out


def assert_close(oracle, want, got, label="", tol_abs=TOL_MAX_ABS, tol_l2=TOL_REL_L2):
    s = oracle.compare(want, got)
    assert s["max_abs"] <= tol_abs and s["rel_l2"] <= tol_l2, (label, s)
    return s
