import numpy as np
import pytest

import aeon_b200
from aeon_b200 import synth

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("preset", ["baseline", "ref_dsv4"])
def test_device_pool_is_byte_identical_to_oracle_payloads(oracle, preset):
    import torch
    cfg = aeon_b200.preset(preset)
    table = synth.half_normal_table(0.02, 1e-4, 4096, dtype=aeon_b200.F16)
    d_table = torch.from_numpy(table.view(np.int16).copy()).cuda()
    pool = aeon_b200.ExpertPool(cfg, 3)
    pool.slab.fill_(0xAB)
    pool.fill_synthetic(0, 3, seed=5, layer=2, first_expert=41, scale_table=d_table)
    torch.cuda.synchronize()
    la = oracle.layout_args(cfg)
    lay = oracle.layout(la)
    host = pool.slab.cpu().numpy().reshape(3, -1)
    for slot in range(3):
        want = oracle.synth_expert_payload(la, 5, 2, 41 + slot, table)
        for name in ("w1", "w2", "w3"):
            m = lay[name]
            nw = m["rows"] * m["cols"]
            for off, size in ((m["packed_offset"], nw // 2), (m["scale_offset"], nw // cfg.group_size * 2)):
                np.testing.assert_array_equal(host[slot, off:off + size], want[off:off + size])
    # scales follow the requested distribution: |N(0, 0.02)| + 1e-4
    m = lay["w1"]
    sc = host[0, m["scale_offset"]:m["scale_offset"] + 2 * 4096].view(np.float16).astype(np.float64)
    assert sc.min() >= 1e-4 and 0.012 < sc.mean() < 0.020
    nib = host[0, :65536]
    vals = np.concatenate([nib & 0xF, nib >> 4]).astype(np.int64) - 8
    assert vals.min() == -8 and vals.max() == 7 and abs(vals.mean() + 0.5) < 0.1


def test_dense_fill_matches_oracle(oracle):
    import torch
    table = synth.half_normal_table(0.02, 0.0, 4096, dtype=aeon_b200.BF16)
    d_table = torch.from_numpy(table.view(np.int16).copy()).cuda()
    out = torch.empty(100003, dtype=torch.int16, device="cuda")
    aeon_b200.synth_fill_dense16(out, 9, 1, 2, d_table)
    want = oracle.synth_dense16(100003, 9, 1, 2, table)
    np.testing.assert_array_equal(out.cpu().numpy().view(np.uint16), want)
    vals = synth.from_bits16(want, aeon_b200.BF16)
    assert abs(vals.mean()) < 5e-4 and 0.018 < vals.std() < 0.022
