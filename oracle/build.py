"""Build recipes for the CPU checkers.  TEST INFRASTRUCTURE ONLY.

``build_oracle()`` compiles this directory's C restatement into ``oracle/_build/liborc.so``.
``build_ref()`` compiles the reference project's own CPU kernels, from the sources where they lie
in a mounted reference tree, into ``oracle/_ref/`` (nothing is copied into this repository); it is a
no-op returning False when the reference tree is not mounted.  Both outputs are git-ignored and
travel to a GPU machine as prebuilt files.

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
REFERENCE_ROOT = Path(os.environ.get("IIE_REFERENCE_ROOT", "/root/reference"))


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


if __name__ == "__main__":
    print(build_oracle(force=True))
    print("reference CPU kernels built:", build_ref(force=True))
