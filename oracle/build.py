"""Build recipes for the CPU checkers.  TEST INFRASTRUCTURE ONLY.

``build_oracle()`` compiles this directory's C restatement into ``oracle/_build/liborc.so``.
``build_ref()`` compiles the reference project's own CPU kernels, from the sources where they lie
in a mounted reference tree, into ``oracle/_ref/`` (nothing is copied into this repository); it is a
no-op returning False when the reference tree is not mounted.  Both outputs are git-ignored and
travel to a GPU machine as prebuilt files.

``install_reference()`` lays the reference's own Python bridge, its CUDA test files and its own CUDA producer (built for
sm_100a with the flags of its build script) out under the git-ignored ``baseline/_ref/``: the reference arm and the
drop-in test run that unmodified code; nothing of it enters this repository's history.

Commands (the same ones the reference's build scripts use for these two files):
  gcc -O3 -fopenmp -fPIC -shared <ref>/north-mini-code/tools/nmc_qk_kernel.c -o oracle/_ref/libnmc_qk.so -lm
  gcc -O3 -march=x86-64-v2 -mtune=generic -fwrapv -fno-strict-overflow -fPIC -shared -fopenmp \
      <ref>/bonsai/tools/bonsai_q1_kernel.c -o oracle/_ref/libbonsai_q1_kernel.so
"""
from __future__ import annotations

import os
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
# where the reference checkout is mounted: IIE_REFERENCE_ROOT, else a checkout named "reference" beside this
# repository; with neither, nothing is built from it
_beside = HERE.parent.parent / "reference"
REFERENCE_ROOT = Path(os.environ["IIE_REFERENCE_ROOT"]) if os.environ.get("IIE_REFERENCE_ROOT") else \
    (_beside if (_beside / "north-mini-code").is_dir() else None)
BASELINE_REF = HERE.parent / "baseline" / "_ref"


def _stale(target: Path, *sources: Path) -> bool:
    return not target.exists() or any(s.stat().st_mtime > target.stat().st_mtime for s in sources)


def build_oracle(force: bool = False) -> Path:
    src, out = HERE / "qk_oracle.c", HERE / "_build" / "liborc.so"
    if force or _stale(out, src):
        out.parent.mkdir(exist_ok=True)
        subprocess.run(["gcc", "-O3", "-march=x86-64-v2", "-fopenmp", "-fPIC", "-shared", str(src), "-o", str(out)],
                       check=True)
    return out


def build_ref(force: bool = False) -> bool:
    if REFERENCE_ROOT is None:
        return False
    nmc = REFERENCE_ROOT / "north-mini-code" / "tools" / "nmc_qk_kernel.c"
    q1 = REFERENCE_ROOT / "bonsai" / "tools" / "bonsai_q1_kernel.c"
    if not nmc.exists():
        return False
    out_dir = HERE / "_ref"
    out_dir.mkdir(exist_ok=True)
    out = out_dir / "libnmc_qk.so"
    if force or _stale(out, nmc):
        subprocess.run(["gcc", "-O3", "-fopenmp", "-fPIC", "-shared", str(nmc), "-o", str(out), "-lm"], check=True)
    out1 = out_dir / "libbonsai_q1_kernel.so"
    if q1.exists() and (force or _stale(out1, q1)):
        subprocess.run(["gcc", "-O3", "-march=x86-64-v2", "-mtune=generic", "-fwrapv", "-fno-strict-overflow",
                        "-fPIC", "-shared", "-fopenmp", str(q1), "-o", str(out1)], check=True)
    return True


def install_reference(force: bool = False) -> bool:
    """``baseline/_ref/north-mini-code/{src/nmc, tests/test_qk_*.py}`` = the reference's bridge package and its CUDA
    differential tests, unmodified; ``baseline/_ref/bin/libnmc_qk_cuda.so`` = the reference's own CUDA producer compiled
    for sm_100a (north-mini-code/tools/build_nmc_cuda.sh: nvcc -O3 -arch=<sm> --cudart static -Xcompiler -fPIC -shared),
    with its CPU kernel ``libnmc_qk.so`` beside it; and the same for the 1-bit decoder (``baseline/_ref/bonsai``, see below).
    Returns False when no reference checkout is mounted."""
    import shutil
    if REFERENCE_ROOT is None or not (REFERENCE_ROOT / "north-mini-code" / "src" / "nmc").exists():
        return False
    root = REFERENCE_ROOT / "north-mini-code"
    dst = BASELINE_REF / "north-mini-code"
    if force and dst.exists():
        shutil.rmtree(dst)
    if not (dst / "src" / "nmc").exists():
        shutil.copytree(root / "src" / "nmc", dst / "src" / "nmc", ignore=shutil.ignore_patterns("__pycache__"))
    (dst / "tests").mkdir(parents=True, exist_ok=True)
    for name in ("test_qk_cuda.py", "test_qk_cuda_api.py", "test_qk_codec.py"):
        if (root / "tests" / name).exists():
            shutil.copyfile(root / "tests" / name, dst / "tests" / name)
    bin_dir = BASELINE_REF / "bin"
    bin_dir.mkdir(parents=True, exist_ok=True)
    cu, out = root / "tools" / "nmc_qk_cuda.cu", bin_dir / "libnmc_qk_cuda.so"
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if cu.exists() and Path(nvcc).exists() and (force or _stale(out, cu)):
        subprocess.run([nvcc, "-O3", "-arch=sm_100a", "--cudart", "static", "-Xcompiler", "-fPIC", "-shared", str(cu), "-o", str(out)],
                       check=True)
    cpu = root / "tools" / "nmc_qk_kernel.c"
    if cpu.exists() and (force or _stale(bin_dir / "libnmc_qk.so", cpu)):
        subprocess.run(["gcc", "-O3", "-fopenmp", "-fPIC", "-shared", str(cpu), "-o", str(bin_dir / "libnmc_qk.so"), "-lm"], check=True)
    # the 1-bit decoder: the reference's package ``trinote`` and its GPU parity tests, its CPU kernel, and its own CUDA
    # library compiled for sm_100a under another name (bonsai/tools/build_bonsai_q1_gpu.sh: nvcc -O3 -arch=<sm>
    # -Xcompiler -fPIC -shared; bonsai/tools/build_bonsai_q1_kernel.sh for the C kernel)
    broot, bdst = REFERENCE_ROOT / "bonsai", BASELINE_REF / "bonsai"
    if (broot / "src" / "trinote").exists():
        if force and bdst.exists():
            shutil.rmtree(bdst)
        if not (bdst / "src" / "trinote").exists():
            shutil.copytree(broot / "src" / "trinote", bdst / "src" / "trinote", ignore=shutil.ignore_patterns("__pycache__"))
        (bdst / "tests").mkdir(parents=True, exist_ok=True)
        for name in ("test_bonsai_gpu.py", "test_q1_oracle_subset.py"):
            if (broot / "tests" / name).exists():
                shutil.copyfile(broot / "tests" / name, bdst / "tests" / name)
        q1c, q1cu = broot / "tools" / "bonsai_q1_kernel.c", broot / "tools" / "bonsai_q1_gpu.cu"
        if q1c.exists() and (force or _stale(bin_dir / "libbonsai_q1_kernel.so", q1c)):
            subprocess.run(["gcc", "-O3", "-march=x86-64-v2", "-mtune=generic", "-fwrapv", "-fno-strict-overflow", "-fPIC", "-shared",
                            "-fopenmp", str(q1c), "-o", str(bin_dir / "libbonsai_q1_kernel.so")], check=True)
        ref_gpu = bin_dir / "reference_libbonsai_q1_gpu.so"
        if q1cu.exists() and Path(nvcc).exists() and (force or _stale(ref_gpu, q1cu)):
            subprocess.run([nvcc, "-O3", "-arch=sm_100a", "-Xcompiler", "-fPIC", "-shared", str(q1cu), "-o", str(ref_gpu)], check=True)
    return True


if __name__ == "__main__":
    print(build_oracle(force=True))
    print("reference CPU kernels built:", build_ref(force=True))
    print("reference bridge, tests and CUDA producer installed:", install_reference(force=True))
