"""The kernels' fixed-point helpers (power of two, sigmoid, SiLU, the single-precision floor division, balanced digits) run
on the CPU: ``tests/host_fixed_check.cu`` includes the kernels' own header and nvcc compiles it for the host; every function
is compared with the NumPy checker over boundary and random operands.  Needs nvcc, no GPU."""
import ctypes
import shutil
import subprocess
from pathlib import Path

import numpy as np
import pytest

from oracle import qk_oracle as o

ROOT = Path(__file__).resolve().parents[1]
I64, U64 = ctypes.POINTER(ctypes.c_int64), ctypes.POINTER(ctypes.c_uint64)


@pytest.fixture(scope="module")
def lib(tmp_path_factory):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(nvcc).exists():
        pytest.skip("nvcc not found")
    so = tmp_path_factory.mktemp("host_fixed") / "libhost_fixed.so"
    build = subprocess.run([nvcc, "-O2", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-Xcompiler", "-fPIC",
                            "-I", str(ROOT / "integer_inference_engine_b200" / "csrc"), str(ROOT / "tests" / "host_fixed_check.cu"),
                            "-o", str(so)], capture_output=True, text=True, timeout=600)
    assert build.returncode == 0, build.stderr[-2000:]
    return ctypes.CDLL(str(so))


def _p(a, t):
    return a.ctypes.data_as(t)


def _operands(fa, rng, n=400_000):
    clip = ((fa + 2) << (2 * fa)) // int(o._scaled_log2e(fa))
    edges = [0, 1, -1, 2, -2, clip - 1, clip, clip + 1, -clip + 1, -clip, -clip - 1, (1 << fa), -(1 << fa), (1 << 40), -(1 << 40),
             (1 << 62), -(1 << 62), np.iinfo(np.int64).max, np.iinfo(np.int64).min + 1]       # not INT64_MIN itself: its negation wraps and the power then shifts by a negative count, which the host compiler and the GPU resolve differently
    parts = [np.array(edges, np.int64)]
    for bits in (8, fa, fa + 3, fa + 6, 2 * fa + 4, 48, 62):
        parts.append(rng.integers(-(1 << bits), 1 << bits, size=n // 7, dtype=np.int64))
    return np.ascontiguousarray(np.concatenate(parts))


@pytest.mark.parametrize("fa", [16, 12, 20, 23])
def test_sigmoid_silu_and_power_of_two(lib, fa):
    rng = np.random.default_rng(100 + fa)
    x = _operands(fa, rng)
    y = np.empty_like(x)
    lib.h_sigmoid(_p(x, I64), _p(y, I64), ctypes.c_longlong(x.size), fa)
    assert np.array_equal(y, o.sigmoid_fixed(x, fa))
    small = x[np.abs(x) < (1 << 50)]                               # x * sigmoid(x) is exact in the checker's Python integers anyway
    ys = np.empty_like(small)
    lib.h_silu(_p(small, I64), _p(ys, I64), ctypes.c_longlong(small.size), fa)
    assert np.array_equal(ys, o.silu_int(small, fa))
    u = np.ascontiguousarray(np.concatenate([np.arange(0, 4096, dtype=np.int64), rng.integers(0, 1 << (fa + 7), size=200_000, dtype=np.int64),
                                             rng.integers(0, 1 << 40, size=50_000, dtype=np.int64)]))
    yu = np.empty_like(u)
    lib.h_exp2_neg(_p(u, I64), _p(yu, I64), ctypes.c_longlong(u.size), fa)
    assert np.array_equal(yu, o.exp2_neg_fixed(u, fa))


def test_single_precision_floor_division(lib):
    rng = np.random.default_rng(7)
    z = np.concatenate([rng.integers(1, 1 << b, size=60_000, dtype=np.int64) for b in (4, 12, 17, 24, 30, 31)]).astype(np.uint32)
    q_true = np.concatenate([rng.integers(0, 1 << b, size=z.size // 4, dtype=np.int64) for b in (3, 16, 24, 31)])[:z.size]
    rem = (rng.random(z.size) * z).astype(np.int64)
    rem[::5] = 0                                                   # exact multiples
    rem[1::5] = z[1::5].astype(np.int64) - 1                       # just below the next quotient
    num = (q_true * z.astype(np.int64) + rem).astype(np.uint64)
    keep = num < np.uint64(1 << 60)
    num, z, want = np.ascontiguousarray(num[keep]), np.ascontiguousarray(z[keep]), (q_true + rem // z.astype(np.int64))[keep]
    got = np.empty(num.size, np.uint64)
    lib.h_udiv(_p(num, U64), z.ctypes.data_as(ctypes.POINTER(ctypes.c_uint32)), _p(got, U64), ctypes.c_longlong(num.size))
    assert np.array_equal(got.astype(np.int64), want)


def test_balanced_digits(lib):
    rng = np.random.default_rng(11)
    cap = o.balanced_capacity(8)
    x = np.concatenate([np.array([0, 1, -1, 127, 128, -128, -129, cap, cap - 1, -cap, -cap - 1, cap + 1, np.iinfo(np.int64).max,
                                  np.iinfo(np.int64).min, 2139062143, 2139062144, -2147483648], np.int64)] +
                       [rng.integers(-(1 << b), 1 << b, size=50_000, dtype=np.int64) for b in (7, 15, 31, 47, 62)])
    x = np.ascontiguousarray(x)
    d, ok = np.empty(x.size, np.uint64), np.empty(x.size, np.uint8)
    lib.h_digits8(_p(x, I64), _p(d, U64), ok.ctypes.data_as(ctypes.POINTER(ctypes.c_uint8)), ctypes.c_longlong(x.size))
    assert np.array_equal(ok.astype(bool), x <= cap)              # every negative int64 fits eight digits
    fits = ok.astype(bool)
    digits = d[fits].view(np.int8).reshape(-1, 8).T                # little endian: byte l = digit l
    assert np.array_equal(digits, o.balanced_limbs(x[fits], 8))
