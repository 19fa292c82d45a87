import numpy as np
import pytest

import aeon_b200
from aeon_b200 import synth
import gpu_support as gs

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("preset,tokens", [("baseline", 1), ("baseline", 12), ("baseline", 16), ("ref_dsv4", 5),
                                           # above 16 tokens: the tensor-core form
                                           ("baseline", 17), ("baseline", 19), ("ref_dsv4", 45), ("baseline", 64),
                                           ("baseline", 100), ("ref_dsv4", 77),
                                           # more than one 256-token pass
                                           ("baseline", 300)])
def test_shared_expert_matches_dense_oracle(oracle, preset, tokens):
    import torch
    cfg = aeon_b200.preset(preset)
    layer = gs.SyntheticLayer(cfg, [0], seed=6, layer=3, with_shared=True)
    ctx = aeon_b200.Context(cfg, max_tokens=tokens)
    x_bits = gs.activations(cfg, tokens, seed=2, scale=2.0)
    out = torch.full((tokens, cfg.hidden), 123.0, dtype=torch.float32, device="cuda")
    ctx.shared_expert(layer.shared[0], layer.shared[1], layer.shared[2],
                      gs.torch_bits(x_bits, cfg.act_dtype), out)
    ctx.check()
    got = out.cpu().numpy().astype(np.float64)
    x = synth.from_bits16(x_bits, cfg.act_dtype)
    w1, w3, w2 = layer.shared_bits(oracle)
    for t in sorted({0, tokens // 2, tokens - 1, min(tokens - 1, 64), min(tokens - 1, 256)}):
        want = oracle.dense_ffn(w1, w3, w2, cfg.act_dtype, x[t], cfg.swiglu_limit)
        s = gs.assert_close(oracle, want, got[t], f"{preset} token {t}", tol_abs=1e-3, tol_l2=1e-5)
