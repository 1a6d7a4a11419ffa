"""In-tree build of the CUDA library: ``python -m integer_inference_engine_b200.build``.

``--changed`` recompiles only the sources that changed.  Compiles every ``csrc/*.cu`` for sm_100a with nvcc into ``lib/libnmc_qk_cuda.so`` (the file name the
reference bridge looks for in ``BONSAI_BIN_DIR``, north-mini-code/src/nmc/qk_cuda.py:95-104) and copies it to
``lib/libbonsai_q1_gpu.so``, the name the Q1_0 bridge loads from the same directory
(bonsai/src/trinote/infer_int/gpu_native.py:27-45); one binary carries both symbol sets.  No fast-math:
the half->fixed conversion and every integer identity must be exact.
"""
from __future__ import annotations

import os
import shutil
import subprocess
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB_DIR = PKG / "lib"
LIB = LIB_DIR / "libnmc_qk_cuda.so"
LIB_Q1 = LIB_DIR / "libbonsai_q1_gpu.so"

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC"]
OBJ_DIR = LIB_DIR / "obj"


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _headers() -> list[Path]:
    return list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list((PKG.parent / "include").glob("*.h"))


def _stale() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    return any(p.stat().st_mtime > t for p in sources() + _headers())


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile the library if any source is newer than it: every ``.cu`` to an object file (in parallel, only those
    older than their source or any header), then one link.  Raises on compiler failure."""
    if not force and not _stale() and LIB_Q1.exists():
        return LIB
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(nvcc).exists():
        raise RuntimeError("nvcc not found: cannot build libnmc_qk_cuda.so")
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    newest_header = max(p.stat().st_mtime for p in _headers())
    jobs = []
    for src in sources():
        obj = OBJ_DIR / (src.stem + ".o")
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, newest_header):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        cmd = [nvcc, *NVCC_FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-c", str(src), "-o", str(obj)]
        return subprocess.run(cmd, cwd=str(CSRC), env=dict(os.environ), capture_output=True, text=True), src

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        for res, src in pool.map(compile_one, jobs):
            if verbose or res.returncode != 0:
                print(res.stdout + res.stderr, flush=True)
            if res.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src.name}")
    objs = [str(OBJ_DIR / (src.stem + ".o")) for src in sources()]
    subprocess.run([nvcc, "-shared", "--cudart", "static", "-gencode", "arch=compute_100a,code=sm_100a", *objs, "-o", str(LIB)],
                   check=True, cwd=str(CSRC))
    shutil.copyfile(LIB, LIB_Q1)
    return LIB


if __name__ == "__main__":
    print(build(force="--changed" not in os.sys.argv, verbose=bool(os.environ.get("IIE_BUILD_VERBOSE"))))
