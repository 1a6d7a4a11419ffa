"""CPU suite: the synthetic GGUF writer produces what its reader (and the reference's reader, whose layout it follows)
expects: key/value pairs, tensor index, aligned offsets, per-expert slices."""
import numpy as np

from integer_inference_engine_b200 import gguf
from oracle import qk_oracle as o


def test_written_checkpoint_reads_back(tmp_path):
    shape = gguf.write_synthetic_model(tmp_path / "m.gguf", **o.ENGINE_CASE["model"])
    g = gguf.GGUFFile(tmp_path / "m.gguf")
    A = gguf.ARCH
    assert g.kv["general.architecture"] == A and g.kv[f"{A}.block_count"] == shape["n_layers"]
    assert g.kv[f"{A}.expert_used_count"] == shape["top_k"] and abs(g.kv[f"{A}.rope.freq_base"] - 50000.0) < 1e-3
    assert g.data_start % 32 == 0 and all(t["offset"] % 32 == 0 for t in g.tensors.values())
    d, E, eff, vocab = shape["d_model"], shape["n_experts"], shape["e_ffn"], shape["vocab"]
    assert g.tensors["token_embd.weight"]["dims"] == [d, vocab] and g.tensors["token_embd.weight"]["nbytes"] == vocab * d // 256 * 210
    assert g.tensors["blk.1.ffn_down_exps.weight"]["dims"] == [eff, d, E]
    assert g.f32("blk.0.ffn_gate_inp.weight").shape == (E, d) and g.f32("output_norm.weight").shape == (d,)
    # an expert slice is a contiguous [out, in] block matrix: the slices tile the tensor exactly
    whole = g.raw("blk.0.ffn_gate_exps.weight")
    assert b"".join(g.expert("blk.0.ffn_gate_exps.weight", e) for e in range(E)) == whole
    # the blocks decode with the oracle's codec (any byte pattern is a valid block; fp16 scales are finite and small)
    w = o.dequant(g.expert("blk.0.ffn_down_exps.weight", 3), d, eff // 256, o.Q6_K, 24)
    assert w.shape == (d, eff) and int(np.abs(w).max()) < (1 << 40)


def test_stub_tokenizer_files(tmp_path):
    import json
    gguf.write_stub_tokenizer(tmp_path / "tok", 17)
    assert len(json.loads((tmp_path / "tok" / "vocab.json").read_text())) == 17
    assert json.loads((tmp_path / "tok" / "merges.json").read_text()) == []
    assert "eos_token_id" in json.loads((tmp_path / "tok" / "meta.json").read_text())
