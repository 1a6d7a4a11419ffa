"""GGUF files of the north-mini-code layout: a writer for synthetic checkpoints, a reader, and stub tokenizer files.

The reference's engine loads a model from one GGUF file plus a tokenizer directory (north-mini-code/src/nmc/engine.py:49-66;
the reader it uses is north-mini-code/src/nmc/gguf.py:27-46,116-122; the tokenizer wants vocab.json, merges.json and meta.json,
tokenizer.py:82-86).  No real checkpoint travels with this repository, so :func:`write_synthetic_model` produces a small
one with the same keys, tensor names, shapes and block formats: architecture ``cohere2moe``; per block ``attn_norm`` (F32),
``attn_q / attn_k / attn_v / attn_output`` (Q4_K), the dense router ``ffn_gate_inp`` (F32), ``ffn_gate_exps / ffn_up_exps``
(Q4_K, all experts in one 3-D tensor) and ``ffn_down_exps`` (Q6_K); ``output_norm`` (F32) and the tied ``token_embd`` (Q6_K).
With it the reference's own ``Engine.generate`` can drive this repository's library (``NMC_BACKEND=cuda-resident``), and
:meth:`integer_inference_engine_b200.model.Decoder.from_gguf` can load the same file without the reference.

File layout written here (GGUF version 3, little endian): magic, version, tensor count, key/value count, the key/value pairs,
the tensor index (name, dimensions with the fastest first, type id, offset), padding to ``general.alignment``, the tensor data,
every tensor starting on an aligned offset.
"""
from __future__ import annotations

import json
import struct
from pathlib import Path

import numpy as np

F32, Q4_K, Q6_K = 0, 12, 14                    # GGML tensor type ids
_BLOCK = {Q4_K: 144, Q6_K: 210}
_U32, _F32, _STR = 4, 6, 8                     # GGUF value type ids
ARCH = "cohere2moe"


def _s(text: str) -> bytes:
    raw = text.encode("utf-8")
    return struct.pack("<Q", len(raw)) + raw


def write_gguf(path, kv: dict, tensors: list, alignment: int = 32) -> None:
    """``kv``: name -> int (u32), float (f32) or str.  ``tensors``: (name, dims fastest-first, type id, bytes)."""
    kv = dict(kv)
    kv.setdefault("general.alignment", alignment)
    head = [b"GGUF", struct.pack("<IQQ", 3, len(tensors), len(kv))]
    for key, val in kv.items():
        if isinstance(val, str):
            head.append(_s(key) + struct.pack("<I", _STR) + _s(val))
        elif isinstance(val, float):
            head.append(_s(key) + struct.pack("<If", _F32, val))
        else:
            head.append(_s(key) + struct.pack("<II", _U32, int(val)))
    offset, placed = 0, []
    for name, dims, ttype, data in tensors:
        placed.append((offset, data))
        head.append(_s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", int(n)) for n in dims) +
                    struct.pack("<IQ", ttype, offset))
        offset += (len(data) + alignment - 1) // alignment * alignment
    blob = b"".join(head)
    with open(path, "wb") as f:
        f.write(blob)
        f.write(b"\0" * (-len(blob) % alignment))
        for off, data in placed:
            f.write(bytes(data))
            f.write(b"\0" * (-len(data) % alignment))


class GGUFFile:
    """Key/value pairs and the tensor index of a GGUF file; tensor bytes are read on demand."""

    def __init__(self, path):
        self.path = str(path)
        with open(self.path, "rb") as f:
            if f.read(4) != b"GGUF":
                raise ValueError(f"{path} is not a GGUF file")
            self.version, n_tensors, n_kv = struct.unpack("<IQQ", f.read(20))
            rd = lambda fmt: struct.unpack("<" + fmt, f.read(struct.calcsize("<" + fmt)))[0]
            string = lambda: f.read(rd("Q")).decode("utf-8")
            scalar = {0: "B", 1: "b", 2: "H", 3: "h", 4: "I", 5: "i", 6: "f", 7: "B", 10: "Q", 11: "q", 12: "d"}

            def value(t):
                if t == 8:
                    return string()
                if t == 9:
                    et, n = rd("I"), rd("Q")
                    return [value(et) for _ in range(n)]
                return rd(scalar[t])
            self.kv = {}
            for _ in range(n_kv):
                key = string()
                self.kv[key] = value(rd("I"))
            self.tensors = {}
            for _ in range(n_tensors):
                name = string()
                dims = [rd("Q") for _ in range(rd("I"))]
                ttype, off = rd("I"), rd("Q")
                n = int(np.prod(dims))
                nbytes = n * 4 if ttype == F32 else n // 256 * _BLOCK[ttype]
                self.tensors[name] = {"dims": dims, "type": ttype, "offset": off, "nbytes": nbytes}
            align = int(self.kv.get("general.alignment", 32))
            self.data_start = (f.tell() + align - 1) // align * align

    def raw(self, name: str, start: int = 0, nbytes: "int | None" = None) -> bytes:
        t = self.tensors[name]
        with open(self.path, "rb") as f:
            f.seek(self.data_start + t["offset"] + start)
            return f.read(t["nbytes"] - start if nbytes is None else nbytes)

    def f32(self, name: str) -> np.ndarray:
        t = self.tensors[name]
        return np.frombuffer(self.raw(name), dtype="<f4").reshape(t["dims"][::-1]).astype(np.float64)

    def expert(self, name: str, e: int) -> bytes:
        """Expert ``e`` of a 3-D tensor [in, out, experts]: a contiguous [out, in] block matrix."""
        t = self.tensors[name]
        per = t["dims"][0] * t["dims"][1] // 256 * _BLOCK[t["type"]]
        return self.raw(name, e * per, per)


def write_stub_tokenizer(directory, vocab: int) -> None:
    """The three files the reference's tokenizer loads, for a model that is only ever driven with token ids."""
    d = Path(directory)
    d.mkdir(parents=True, exist_ok=True)
    (d / "vocab.json").write_text(json.dumps([f"<t{i}>" for i in range(vocab)]))
    (d / "merges.json").write_text("[]")
    (d / "meta.json").write_text(json.dumps({"bos_token_id": None, "eos_token_id": None, "add_bos_token": False}))


def write_synthetic_model(path, *, n_layers: int = 2, d_model: int = 256, n_heads: int = 4, n_kv: int = 2, head_dim: int = 64,
                          e_ffn: int = 256, n_experts: int = 8, top_k: int = 2, vocab: int = 96, window: int = 8,
                          context: int = 64, rope_base: float = 50000.0, seed: int = 0) -> dict:
    """A seeded random checkpoint of the north-mini-code architecture (every block a MoE block).  Quantised tensors are
    uniform block bytes with fp16 scales |N(0,1)| * 0.01, norm gains |N(0,1)| + 0.5, routers N(0,1) * 0.05.
    Returns the shape as a dict."""
    rng = np.random.default_rng(seed)

    def q4k(out_f, in_f, experts=1):
        n = experts * out_f * in_f // 256
        blk = rng.integers(0, 256, size=(n, 144), dtype=np.uint8)
        blk[:, 0:4] = np.abs(rng.standard_normal((n, 2)) * 0.01).astype("<f2").view(np.uint8).reshape(n, 4)
        return blk.tobytes()

    def q6k(out_f, in_f, experts=1):
        n = experts * out_f * in_f // 256
        blk = rng.integers(0, 256, size=(n, 210), dtype=np.uint8)
        blk[:, 208:210] = np.abs(rng.standard_normal(n) * 0.01).astype("<f2").view(np.uint8).reshape(n, 2)
        return blk.tobytes()

    f32 = lambda a: np.ascontiguousarray(a, dtype="<f4").tobytes()
    qd, kd = n_heads * head_dim, n_kv * head_dim
    tensors = [("token_embd.weight", [d_model, vocab], Q6_K, q6k(vocab, d_model)),
               ("output_norm.weight", [d_model], F32, f32(np.abs(rng.standard_normal(d_model)) + 0.5))]
    for li in range(n_layers):
        p = f"blk.{li}."
        tensors += [
            (p + "attn_norm.weight", [d_model], F32, f32(np.abs(rng.standard_normal(d_model)) + 0.5)),
            (p + "attn_q.weight", [d_model, qd], Q4_K, q4k(qd, d_model)),
            (p + "attn_k.weight", [d_model, kd], Q4_K, q4k(kd, d_model)),
            (p + "attn_v.weight", [d_model, kd], Q4_K, q4k(kd, d_model)),
            (p + "attn_output.weight", [qd, d_model], Q4_K, q4k(d_model, qd)),
            (p + "ffn_gate_inp.weight", [d_model, n_experts], F32, f32(rng.standard_normal((n_experts, d_model)) * 0.05)),
            (p + "ffn_gate_exps.weight", [d_model, e_ffn, n_experts], Q4_K, q4k(e_ffn, d_model, n_experts)),
            (p + "ffn_up_exps.weight", [d_model, e_ffn, n_experts], Q4_K, q4k(e_ffn, d_model, n_experts)),
            (p + "ffn_down_exps.weight", [e_ffn, d_model, n_experts], Q6_K, q6k(d_model, e_ffn, n_experts)),
        ]
    A = ARCH
    kv = {"general.architecture": A, f"{A}.embedding_length": d_model, f"{A}.attention.head_count": n_heads,
          f"{A}.attention.head_count_kv": n_kv, f"{A}.attention.key_length": head_dim, f"{A}.feed_forward_length": e_ffn,
          f"{A}.vocab_size": vocab, f"{A}.attention.sliding_window": window, f"{A}.expert_count": n_experts,
          f"{A}.expert_used_count": top_k, f"{A}.expert_feed_forward_length": e_ffn, f"{A}.rope.freq_base": float(rope_base),
          f"{A}.block_count": n_layers, f"{A}.leading_dense_block_count": 0, f"{A}.context_length": context}
    write_gguf(path, kv, tensors)
    return dict(n_layers=n_layers, d_model=d_model, n_heads=n_heads, n_kv=n_kv, head_dim=head_dim, e_ffn=e_ffn, n_experts=n_experts,
                top_k=top_k, vocab=vocab, window=window, context=context, rope_base=rope_base)
