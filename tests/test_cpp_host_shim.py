"""Builds and runs the C++ host-layer checks (tests/cpp/test_host_shim.cpp): the reference's
class names over the C ABI — topology, device-id parser, registry state machine, expert
container, format descriptors. Host only; links libaeon_b200.so for the geometry calls."""
import os
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def build(src, out, compiler="g++", extra=()):
    lib_dir = os.path.join(ROOT, "project-aeon_b200", "lib")
    cmd = [compiler, "-std=c++17", "-O1", src, "-o", out,
           "-I" + os.path.join(ROOT, "include"), "-I" + os.path.join(ROOT, "project-aeon_b200", "host"),
           "-L" + lib_dir, "-laeon_b200", *extra]
    if compiler == "g++":
        cmd += ["-Wl,-rpath," + lib_dir, "-Wall", "-Wextra"]
    else:
        cmd += ["-Xlinker", "-rpath," + lib_dir]
    subprocess.run(cmd, check=True, capture_output=True, text=True)


def write_python_model_dir(model_dir):
    """A small model directory from the Python converter, with the figures the C++ loader must
    find in it: both sides read the same files."""
    import numpy as np
    import aeon_b200
    from aeon_b200 import artifact
    import oracle_py
    cfg = aeon_b200.preset("baseline").copy(hidden=256, intermediate=2048, experts=32, top_k=4)
    rng = np.random.default_rng(11)

    def source_of(layer, expert):
        r = np.random.default_rng([layer, expert])
        return [r.integers(0, 2 ** 32, size=shape, dtype=np.uint64).astype(np.uint32) if i % 2 == 0
                else r.integers(0x2000, 0x2800, size=shape).astype(np.uint16)
                for i, shape in enumerate(aeon_b200.source_shapes(cfg))]

    fmt = artifact.write_expert_artifact(model_dir, cfg, 1, source_of, max_tensor_parallel=4)
    gate = rng.integers(0, 2 ** 16, size=(cfg.experts, cfg.hidden), dtype=np.uint16)
    artifact.write_dense_container(os.path.join(model_dir, artifact.DENSE_FILENAME),
                                   [("layers.0.ffn.gate.weight", "BF16", gate),
                                    ("layers.0.ffn.gate.bias", "F32", np.zeros(cfg.experts, np.float32))])
    art = artifact.ExpertArtifact(model_dir)
    with open(os.path.join(model_dir, "expected.txt"), "w") as f:
        f.write(f"{fmt.shard_count} {fmt.payload_bytes} {oracle_py.fnv1a(np.asarray(art.expert_data(0, 3)))} "
                f"{oracle_py.fnv1a(gate)} {art.rank_slice(0, 3, 2, 1)[0]}\n")


def test_host_shim(tmp_path):
    exe = str(tmp_path / "test_host_shim")
    build(os.path.join(ROOT, "tests", "cpp", "test_host_shim.cpp"), exe)
    model_dir = str(tmp_path / "py_model")
    write_python_model_dir(model_dir)
    r = subprocess.run([exe, str(tmp_path), model_dir], capture_output=True, text=True)
    print(r.stdout)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "ALL PASS" in r.stdout and "FAIL " not in r.stdout


def test_integration_example_compiles_with_override(tmp_path):
    """The executor of INTEGRATION.md overrides the seam's members as written (compile and link only)."""
    build(os.path.join(ROOT, "tests", "cpp", "integration_example.cpp"), str(tmp_path / "integration_example"))


import pytest


@pytest.mark.gpu
def test_executor_on_gpu(tmp_path):
    """tests/cpp/test_executor_gpu.cpp: the C++ executor over a small pool against the direct
    C-ABI call (bit-identical), chunk-wide dispatch, protocol errors, wrong-expert probe."""
    exe = str(tmp_path / "test_executor_gpu")
    build(os.path.join(ROOT, "tests", "cpp", "test_executor_gpu.cpp"), exe, compiler="nvcc")
    r = subprocess.run([exe, str(tmp_path)], capture_output=True, text=True)
    print(r.stdout)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "ALL PASS" in r.stdout
