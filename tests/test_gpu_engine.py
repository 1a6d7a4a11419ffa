"""The reference's own ``Engine`` driving this repository's library, and this repository's decoder loading the same file.

The golden ids (tests/golden/engine_generate.npz) were produced by the reference ``Engine.generate`` on its CPU backend for
the synthetic checkpoint ``gguf.write_synthetic_model`` writes with ``oracle.qk_oracle.ENGINE_CASE``.  Here
(a) ``Decoder.from_gguf(...).generate`` must give the same ids, and
(b) the unmodified reference engine (installed under baseline/_ref) with ``NMC_BACKEND=cuda-resident`` and ``BONSAI_BIN_DIR``
    pointing at this repository's library (every product, the attention bank and the expert stages then run on the new
    kernels, north-mini-code/src/nmc/engine.py:449-597) must give them too.
"""
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from oracle import qk_oracle as o

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]
REF = ROOT / "baseline" / "_ref" / "north-mini-code"


def _checkpoint(tmp_path):
    from integer_inference_engine_b200 import gguf
    shape = gguf.write_synthetic_model(tmp_path / "m.gguf", **o.ENGINE_CASE["model"])
    gguf.write_stub_tokenizer(tmp_path / "tok", shape["vocab"])
    return tmp_path / "m.gguf", tmp_path / "tok"


def test_decoder_loaded_from_the_checkpoint_generates_the_reference_ids(tmp_path, golden_dir):
    from integer_inference_engine_b200 import device, qk_cuda as qk
    from integer_inference_engine_b200.model import Decoder
    qk.free_all()
    blob, _ = _checkpoint(tmp_path)
    dec = Decoder.from_gguf(blob)
    got = dec.generate(o.ENGINE_CASE["prompt"], o.ENGINE_CASE["n_new"])
    assert device.read_flags() == 0
    assert got == [int(t) for t in np.load(golden_dir / "engine_generate.npz")["ids"]]
    qk.free_all()


@pytest.mark.skipif(not (REF / "src" / "nmc" / "engine.py").exists(), reason="reference engine not installed under baseline/_ref")
@pytest.mark.parametrize("resident_attention", [True, False], ids=["attention-bank", "host-attention"])
def test_reference_engine_generates_through_this_library(tmp_path, golden_dir, resident_attention):
    blob, tok = _checkpoint(tmp_path)
    code = (
        "import json, sys\n"
        "from nmc.engine import Engine\n"
        "eng = Engine(sys.argv[1], sys.argv[2], backend='cuda-resident', resident_attention=bool(int(sys.argv[5])))\n"
        "assert eng.bname == 'cuda-resident', eng.bname\n"
        "ids = eng.generate(json.loads(sys.argv[3]), int(sys.argv[4]), stop_eos=False)\n"
        "eng.free()\n"
        "print(json.dumps(ids))\n")
    env = dict(os.environ)
    env["BONSAI_BIN_DIR"] = str(ROOT / "integer_inference_engine_b200" / "lib")
    env["PYTHONPATH"] = str(REF / "src")
    env.pop("BONSAI_NOTARY_HOME", None)
    env.pop("NMC_BACKEND", None)
    run = subprocess.run([sys.executable, "-c", code, str(blob), str(tok), json.dumps(list(o.ENGINE_CASE["prompt"])),
                          str(o.ENGINE_CASE["n_new"]), "1" if resident_attention else "0"],
                         env=env, cwd=str(tmp_path), capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stdout[-1500:] + run.stderr[-3000:]
    ids = json.loads(run.stdout.strip().splitlines()[-1])
    assert ids == [int(t) for t in np.load(golden_dir / "engine_generate.npz")["ids"]]
