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


def test_host_shim(tmp_path):
    exe = str(tmp_path / "test_host_shim")
    build(os.path.join(ROOT, "tests", "cpp", "test_host_shim.cpp"), exe)
    r = subprocess.run([exe, str(tmp_path)], capture_output=True, text=True)
    print(r.stdout)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "ALL PASS" in r.stdout and "FAIL " not in r.stdout


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
