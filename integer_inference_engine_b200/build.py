"""In-tree build of the CUDA library: ``python -m integer_inference_engine_b200.build``.

Compiles every ``csrc/*.cu`` for sm_100a with nvcc into ``lib/libnmc_qk_cuda.so`` (the file name the
reference bridge looks for in ``BONSAI_BIN_DIR``, north-mini-code/src/nmc/qk_cuda.py:95-104) and copies it to
``lib/libbonsai_q1_gpu.so``, the name the Q1_0 bridge loads from the same directory
(bonsai/src/trinote/infer_int/gpu_native.py:27-45); one binary carries both symbol sets.  No fast-math:
the half->fixed conversion and every integer identity must be exact.
"""
from __future__ import annotations

import os
import shutil
import subprocess
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB_DIR = PKG / "lib"
LIB = LIB_DIR / "libnmc_qk_cuda.so"
LIB_Q1 = LIB_DIR / "libbonsai_q1_gpu.so"

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--cudart", "static",
              "-Xcompiler", "-fPIC", "-shared"]


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _stale() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + \
        list((PKG.parent / "include").glob("*.h"))
    return any(p.stat().st_mtime > t for p in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile the library if any source is newer than it.  Raises on compiler failure."""
    if not force and not _stale() and LIB_Q1.exists():
        return LIB
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(nvcc).exists():
        raise RuntimeError("nvcc not found: cannot build libnmc_qk_cuda.so")
    LIB_DIR.mkdir(exist_ok=True)
    cmd = [nvcc, *NVCC_FLAGS, *(["-Xptxas", "-v"] if verbose else []), *map(str, sources()), "-o", str(LIB)]
    env = dict(os.environ)
    subprocess.run(cmd, check=True, cwd=str(CSRC), env=env)
    shutil.copyfile(LIB, LIB_Q1)
    return LIB


if __name__ == "__main__":
    print(build(force=True, verbose=bool(os.environ.get("IIE_BUILD_VERBOSE"))))
