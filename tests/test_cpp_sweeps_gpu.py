"""Builds and runs tests/cpp/kernel_sweeps.cc: the reference's operator unit tests (same graphs via
Scope + nn_ops, same sweeps) against the C++ runtime, with the CPU oracle as the expected value."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _build(tmp_path):
    from ogle_b200 import build
    from oracle import oracle
    build.build_all()
    oracle.build()
    exe = str(tmp_path / "kernel_sweeps")
    rt = os.path.join(ROOT, "ogle_b200", "csrc", "runtime")
    cmd = ["/usr/bin/g++", "-O2", "-std=c++17", os.path.join(ROOT, "tests", "cpp", "kernel_sweeps.cc"), "-o", exe,
           "-I", rt, "-I", os.path.join(ROOT, "include"), "-I", os.path.join(ROOT, "oracle"),
           "-L", os.path.join(ROOT, "ogle_b200"), "-logle_rt", "-logle_cuda",
           "-L", os.path.join(ROOT, "oracle"), "-loracle", "-L", "/usr/local/cuda/lib64", "-lcudart",
           "-Wl,-rpath," + os.path.join(ROOT, "ogle_b200"), "-Wl,-rpath," + os.path.join(ROOT, "oracle"),
           "-Wl,-rpath,/usr/local/cuda/lib64"]
    subprocess.run(cmd, check=True, capture_output=True)
    return exe


def test_kernel_sweeps_program_builds(tmp_path):
    """CPU: the program compiles and links against the runtime and the oracle."""
    assert os.path.exists(_build(tmp_path))


@pytest.mark.gpu
@pytest.mark.parametrize("math_mode,gemm_rtol", [("0", "1e-5"), ("2", "1e-4")])
def test_reference_kernel_sweeps(tmp_path, math_mode, gemm_rtol):
    """FP32 mode at the reference's tolerance; the default 3xTF32 mode with the gemm bound its
    truncating accumulator needs on all-positive inputs (conv, concat, transpose, clip unchanged)."""
    exe = _build(tmp_path)
    env = dict(os.environ, OGLE_MATH_MODE=math_mode)
    r = subprocess.run([exe, "256", gemm_rtol], capture_output=True, text=True, timeout=1500, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
    assert "PASSED" in r.stdout
