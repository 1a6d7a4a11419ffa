"""The exact integer helpers of the block norm (integer square root over 128 bits, the approximate-from-below reciprocal
and the floor division through it) run on the CPU: ``tests/host_norm_check.cu`` includes the kernels' own header and is
compiled for the host by nvcc.  Needs nvcc, no GPU."""
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def test_norm_helpers_on_the_host(tmp_path):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(nvcc).exists():
        pytest.skip("nvcc not found")
    exe = tmp_path / "host_norm_check"
    build = subprocess.run([nvcc, "-O2", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a",
                            "-I", str(ROOT / "integer_inference_engine_b200" / "csrc"), str(ROOT / "tests" / "host_norm_check.cu"),
                            "-o", str(exe)], capture_output=True, text=True, timeout=600)
    assert build.returncode == 0, build.stderr[-2000:]
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=600)
    assert run.returncode == 0 and run.stdout.startswith("ok "), run.stdout[-500:] + run.stderr[-500:]
