"""The bounds-checked build of the library (make -C project-aeon_b200/csrc bounds): the same
sources with every run-time-derived index checked against its buffer and guard regions behind
the context's scratch buffers. It stands in for a memory checker: the small decode, prefill,
router and layer cases are run through it in a child process (the library path is chosen with
AEON_B200_LIBRARY before the binding loads) and must (1) report itself as the checked build,
(2) agree with the oracle like the normal build, (3) leave every guard region intact and raise no
index violation, and (4) report -- not use -- a slot-table entry beyond the declared pool size."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BOUNDS_LIB = os.path.join(ROOT, "project-aeon_b200", "lib_bounds", "libaeon_b200.so")

CHILD = r"""
import sys
import numpy as np
import torch
import aeon_b200
import gpu_support as gs
import oracle_py as oracle

assert aeon_b200.bounds_checked(), "the child must run the bounds-checked build"
cfg = aeon_b200.preset("baseline")
resident = list(range(8, 24))
layer = gs.SyntheticLayer(cfg, resident, seed=3, layer=1, with_shared=True)
rng = np.random.default_rng(5)

# decode: 11 tokens (an expert with more than one work entry), checked against the oracle
tokens = 11
ids = np.stack([rng.choice(resident, cfg.top_k, replace=False) for _ in range(tokens)]).astype(np.int32)
w = rng.random((tokens, cfg.top_k)).astype(np.float32) + 0.05
w /= w.sum(axis=1, keepdims=True)
x_bits = gs.activations(cfg, tokens, seed=2)
x = gs.torch_bits(x_bits, cfg.act_dtype)
ctx = aeon_b200.Context(cfg, max_tokens=tokens)
ctx.set_pool_slots(len(resident))
d_ids, d_w = torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda()
out = torch.zeros(tokens, cfg.hidden, dtype=torch.float32, device="cuda")
ctx.moe_decode(layer.pool.base, layer.slot_of, x, d_ids, d_w, out)
ctx.check()                                  # error flag clear, guard regions intact
want = gs.oracle_routed(oracle, layer, x_bits, ids, w.astype(np.float64), [0, tokens - 1])
for t in (0, tokens - 1):
    gs.assert_close(oracle, want[t], out[t].double().cpu().numpy(), f"bounds build decode token {t}")

# router + shared expert + prefill through the same context
weights, top = ctx.router_topk(x, layer.gate)
acc = torch.zeros(tokens, cfg.hidden, dtype=torch.float32, device="cuda")
ctx.shared_expert(layer.shared[0], layer.shared[1], layer.shared[2], x, acc)
pre = torch.zeros(tokens, cfg.hidden, dtype=torch.float32, device="cuda")
ctx.moe_prefill(layer.pool.base, layer.slot_of, x, d_ids, d_w, pre)
ctx.check()
mirrored = gs.mirrored_oracle(oracle, layer, x_bits, ids, w.astype(np.float64), [3])
gs.assert_close(oracle, mirrored[3], pre[3].double().cpu().numpy(), "bounds build prefill token 3")

# a slot table entry beyond the declared pool: reported by check(), never used as an address
bad_slots = layer.slot_of.clone()
bad_slots[resident[0]] = len(resident) + 5
out.zero_()
ctx.moe_decode(layer.pool.base, bad_slots, x, d_ids, d_w, out, skip_absent=True)
try:
    ctx.check()
    raise SystemExit("the out-of-range slot was not reported")
except aeon_b200.AeonError as e:
    assert e.status == 4, e
ctx.check()                                  # the flag was cleared by the report; the context is usable
out.zero_()
ctx.moe_decode(layer.pool.base, layer.slot_of, x, d_ids, d_w, out)
ctx.check()
gs.assert_close(oracle, want[0], out[0].double().cpu().numpy(), "after the report")
print("BOUNDS BUILD OK")
"""


def test_bounds_checked_build_runs_the_path_clean():
    if not os.path.exists(BOUNDS_LIB):
        subprocess.run(["make", "-C", os.path.join(ROOT, "project-aeon_b200", "csrc"), "-j", str(os.cpu_count() or 4),
                        "bounds"], check=True, capture_output=True)
    env = dict(os.environ, AEON_B200_LIBRARY=BOUNDS_LIB,
               PYTHONPATH=os.pathsep.join([os.path.join(ROOT, "project-aeon_b200"), os.path.join(ROOT, "tests")]))
    r = subprocess.run([sys.executable, "-c", CHILD], env=env, capture_output=True, text=True, timeout=900)
    print(r.stdout[-2000:])
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "BOUNDS BUILD OK" in r.stdout


def test_declared_pool_size_guards_the_slot_table_in_the_normal_build():
    """The slot-range report is part of every build, not only the checked one."""
    import numpy as np
    import torch
    import aeon_b200
    import gpu_support as gs
    cfg = aeon_b200.preset("baseline")
    resident = list(range(8))
    layer = gs.SyntheticLayer(cfg, resident, seed=3, layer=1, with_shared=False)
    ctx = aeon_b200.Context(cfg, max_tokens=2)
    ctx.set_pool_slots(len(resident))
    x = gs.torch_bits(gs.activations(cfg, 2, seed=2), cfg.act_dtype)
    ids = torch.arange(8, dtype=torch.int32, device="cuda").repeat(2, 1).contiguous()
    w = torch.full((2, 8), 0.125, dtype=torch.float32, device="cuda")
    out = torch.zeros(2, cfg.hidden, dtype=torch.float32, device="cuda")
    bad = layer.slot_of.clone()
    bad[3] = 1 << 20                                   # far outside the pool
    ctx.moe_decode(layer.pool.base, bad, x, ids, w, out, skip_absent=True)
    with pytest.raises(aeon_b200.AeonError) as e:
        ctx.check()
    assert e.value.status == 4
    ctx.moe_prefill(layer.pool.base, bad, x, ids, w, out, skip_absent=True)
    with pytest.raises(aeon_b200.AeonError) as e:
        ctx.check()
    assert e.value.status == 4
    ctx.check()
