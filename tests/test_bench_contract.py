"""The benchmark's output contract: one JSON line with the keys the driver reads. Checked on a
line recorded from a B200 run of `python bench.py --steps 20 --warmup 5`
(tests/golden/bench_line_b200_sample.json) and, live, on the CPU reference arm. The shape
literals the reference arm uses instead of the product library are checked against the
library's own preset."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

BASE_KEYS = {"metric": str, "value": (int, float), "unit": str, "n_gpus": int, "steps": int, "warmup": int,
             "ms_per_step": (int, float), "higher_is_better": bool, "scaling": str, "dtype": str,
             "data": str, "config": dict, "e2e": dict}


def check_base(line):
    for key, kind in BASE_KEYS.items():
        assert key in line and isinstance(line[key], kind), key
    assert "vs_baseline" in line and line["vs_baseline"] is None      # no published number for this metric
    assert "workload" in line["config"]
    for key in ("value", "unit", "h2d_bytes_per_step", "d2h_bytes_per_step"):
        assert key in line["e2e"], key
    assert line["value"] > 0 and line["ms_per_step"] > 0 and line["data"] == "synthetic"


def test_recorded_b200_line_has_the_contract_keys():
    line = json.loads(open(os.path.join(ROOT, "tests", "golden", "bench_line_b200_sample.json")).read())
    check_base(line)
    assert line["warmup"] >= 3 and line["gpu_launches"] > 0
    assert line["e2e"]["h2d_bytes_per_step"] > 0 and line["e2e"]["d2h_bytes_per_step"] > 0
    assert line["e2e"]["value"] < line["value"]                       # copies inside the timed region cost something
    roof = line["roofline"]
    for key in ("bound", "achieved", "peak", "unit", "frac", "traffic"):
        assert key in roof, key
    assert roof["bound"] == "hbm" and roof["unit"] == "GB/s"
    assert abs(roof["frac"] - roof["achieved"] / roof["peak"]) < 1e-9
    # ncu traffic within 2 % of the algorithmic bytes: every weight byte is read once
    assert 0.98 < roof["traffic"] / roof["algorithmic_bytes_per_launch"] < 1.02
    assert roof["kernel"] == "moe_w13_rows_kernel" and roof["second_kernel"]["kernel"] == "moe_w2_rows_kernel"
    assert 0.5 < roof["frac"] < 1.05 and 0.5 < roof["whole_step"]["frac"] < 1.0
    # the run checks itself on the box that timed it: identical routing, layer output within tolerance
    parity = line["parity"]
    assert parity["ok"] and parity["ids_equal"] and parity["ids_match_oracle"]
    assert parity["max_abs"] <= parity["tolerance"]["max_abs"] == 2e-2
    assert parity["rel_l2"] <= parity["tolerance"]["rel_l2"] == 1e-3
    assert line["launch_mode"] in ("cuda graph replay", "eager launches")
    cpu = line["cpu_baseline"]
    for key in ("value", "unit", "cores", "kind", "sample"):
        assert key in cpu, key
    assert cpu["kind"] in ("reference", "port") and cpu["cores"] >= 1
    clocks = line["clocks"]
    # at the clock limit, or below it with the power cap as the stated reason (1 kW part under a
    # memory-bound load); never below it for no reason (a leftover clock lock)
    assert clocks["sm_mhz"] > 0.9 * clocks["sm_max_mhz"] or "sw_power_cap" in clocks["reasons"]
    assert clocks["sm_mhz"] > 0.8 * clocks["sm_max_mhz"]
    assert not set(clocks["reasons"]) & {"hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown"}


def test_reference_arm_prints_one_contract_line():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                          "--warmup", "0"], capture_output=True, text=True, timeout=900, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.strip()]
    assert len(lines) == 1, lines
    line = json.loads(lines[0])
    check_base(line)
    assert line["impl"] == "reference" and line["n_gpus"] == 1
    assert line["e2e"] == {"value": line["value"], "unit": line["unit"], "h2d_bytes_per_step": 0,
                           "d2h_bytes_per_step": 0}
    assert line["cpu_baseline"]["value"] == line["value"] and line["cpu_baseline"]["kind"] == "port"


def test_reference_arm_shape_literals_match_the_library_preset():
    """bench.py's reference arm must not load the product library, so it carries the benchmark's
    shapes as literals; they have to be the library's `baseline` preset."""
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "project-aeon_b200"))
    import bench
    import aeon_b200
    cfg = aeon_b200.preset("baseline")
    for key, value in bench.BASELINE_SHAPE.items():
        assert getattr(cfg, key) == value, key
