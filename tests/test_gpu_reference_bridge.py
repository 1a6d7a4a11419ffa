"""The reference's OWN bridge and its own CUDA differential tests, run against this repository's library.

``oracle/build.py::install_reference`` lays the unmodified ``nmc`` package (north-mini-code/src/nmc) and
``north-mini-code/tests/test_qk_cuda.py`` out under ``baseline/_ref/``.  With ``BONSAI_BIN_DIR`` pointing at
``integer_inference_engine_b200/lib`` the reference bridge loads ``libnmc_qk_cuda.so`` from there
(north-mini-code/src/nmc/qk_cuda.py:95-104), checks its ABI gate (qk_cuda.py:83-93) and every call of those tests goes
through the new kernels.  Skipped where ``baseline/_ref`` is absent.
"""
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]
REF = ROOT / "baseline" / "_ref" / "north-mini-code"
LIB_DIR = ROOT / "integer_inference_engine_b200" / "lib"


def _env(bin_dir=LIB_DIR):
    env = dict(os.environ)
    env["BONSAI_BIN_DIR"] = str(bin_dir)
    env["PYTHONPATH"] = os.pathsep.join([str(REF / "src"), str(REF)])
    env.pop("BONSAI_NOTARY_HOME", None)
    return env


@pytest.mark.skipif(not (REF / "tests" / "test_qk_cuda.py").exists(), reason="reference bridge not installed under baseline/_ref")
def test_reference_bridge_accepts_the_library_and_its_own_tests_pass(tmp_path):
    # the reference looks for its CPU kernel in the same directory (one of its tests compares the two producers): a
    # directory holding this repository's CUDA library beside the reference's own compiled CPU kernel
    (tmp_path / "libnmc_qk_cuda.so").symlink_to(LIB_DIR / "libnmc_qk_cuda.so")
    cpu_kernel = ROOT / "baseline" / "_ref" / "bin" / "libnmc_qk.so"
    if cpu_kernel.exists():
        (tmp_path / "libnmc_qk.so").symlink_to(cpu_kernel)
    probe = subprocess.run([sys.executable, "-c",
                            "from nmc import qk_cuda as q; import sys; l = q._lib(); "
                            "print(q._so_path()); sys.exit(0 if (l is not None and q.available()) else 3)"],
                           env=_env(tmp_path), cwd=str(REF), capture_output=True, text=True, timeout=300)
    assert probe.returncode == 0, f"the reference bridge refused the library: {probe.stdout} {probe.stderr}"
    assert str(tmp_path) in probe.stdout
    run = subprocess.run([sys.executable, "-m", "pytest", "tests/test_qk_cuda.py", "-q", "-x", "-p", "no:cacheprovider"],
                         env=_env(tmp_path), cwd=str(REF), capture_output=True, text=True, timeout=1500)
    tail = run.stdout[-3000:] + run.stderr[-1500:]
    assert run.returncode == 0, tail
    assert " passed" in run.stdout, tail
    if cpu_kernel.exists():
        assert "skipped" not in run.stdout.splitlines()[-1], tail   # every optional capability is present, nothing may skip
    print(run.stdout.splitlines()[-1])                      # the reference suite's own summary line


BONSAI = ROOT / "baseline" / "_ref" / "bonsai"

# The reference's GPU tests take their small model from a helper of another of its test modules, whose own imports need
# a signing package that is not installed here.  This stand-in provides that one helper with the same shape, through the
# reference's own generator.
_SMALL_MODEL_HELPER = """
from trinote.infer_int.reference_bonsai import random_bonsai_artifact


def _small_bonsai(seed=0):
    shape = {"dModel": 128, "nHeads": 4, "nHeadsKv": 2, "headDim": 32, "dFfn": 256, "vocab": 256, "nLayers": 2,
             "fpFracBits": 16, "ropeBase": 1_000_000, "ropeScalingType": "none"}
    return random_bonsai_artifact(shape, seq_len=32, seed=seed)
"""


@pytest.mark.skipif(not (BONSAI / "tests" / "test_bonsai_gpu.py").exists(), reason="reference 1-bit package not installed under baseline/_ref")
def test_reference_q1_bridge_and_its_own_gpu_tests_pass(tmp_path):
    """``trinote.infer_int.gpu_native`` (unmodified) loads ``libbonsai_q1_gpu.so`` from ``$BONSAI_BIN_DIR``
    (bonsai/src/trinote/notary_paths.py:154-164): a directory with this repository's library under that name beside the
    reference's compiled CPU kernel, then the reference's own parity file ``bonsai/tests/test_bonsai_gpu.py``."""
    bins = tmp_path / "bin"
    bins.mkdir()
    (bins / "libbonsai_q1_gpu.so").symlink_to(LIB_DIR / "libbonsai_q1_gpu.so")
    cpu_kernel = ROOT / "baseline" / "_ref" / "bin" / "libbonsai_q1_kernel.so"
    if cpu_kernel.exists():
        (bins / "libbonsai_q1_kernel.so").symlink_to(cpu_kernel)
    helpers = tmp_path / "helpers"
    helpers.mkdir()
    (helpers / "test_bonsai_smoke.py").write_text(_SMALL_MODEL_HELPER)
    env = dict(os.environ)
    env["BONSAI_BIN_DIR"] = str(bins)
    env["BONSAI_NOTARY_HOME"] = str(tmp_path / "home")
    env["PYTHONPATH"] = os.pathsep.join([str(BONSAI / "src"), str(helpers)])
    for name in ("TRINOTE_GPU", "TRINOTE_GPU_FULL"):
        env.pop(name, None)
    probe = subprocess.run([sys.executable, "-c", "from trinote.infer_int import gpu_native as g; import sys; "
                            "print(g._load_lib()._name); sys.exit(0 if g.gpu_available() and g.monolith_available() else 3)"],
                           env=env, cwd=str(BONSAI), capture_output=True, text=True, timeout=300)
    assert probe.returncode == 0, f"the reference bridge refused the library: {probe.stdout} {probe.stderr}"
    assert str(bins) in probe.stdout
    run = subprocess.run([sys.executable, "-m", "pytest", "tests/test_bonsai_gpu.py", "-q", "-p", "no:cacheprovider", "-rs"],
                         env=env, cwd=str(BONSAI), capture_output=True, text=True, timeout=1500)
    tail = run.stdout[-5000:] + run.stderr[-1500:]
    assert run.returncode == 0, tail
    assert " passed" in run.stdout, tail
    print(run.stdout.splitlines()[-1])
    print("\n".join(line for line in run.stdout.splitlines() if line.startswith("SKIPPED")))
