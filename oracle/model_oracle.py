"""CPU checker for one decode step of the whole synthetic decoder.  TEST INFRASTRUCTURE ONLY.

Restates north-mini-code/src/nmc/cohere2.py:357-376 (block_cached, m = 1) and :201-204 (tied head) on top of
the functions of ``oracle/qk_oracle.py`` and the compiled linear / MoE checkers of ``oracle/native.py``.  The
caller hands in the raw weight bytes exported from the device and host copies of the KV caches.
"""
from __future__ import annotations

import numpy as np

from . import native as onat
from . import qk_oracle as o


def decode_token(token: int, pos: int, layers, embd_raw: bytes, out_gain, cfg, cos, sin):
    """layers[i] = dict(gain, wq, wk, wv, wo (raw Q4_K bytes), k, v (int64 caches [Hkv, rows, hd], row `pos` is written
    here), full (bool), moe=(router_raw, gate_raws, up_raws, down_raws)).  cfg = dict(d, H, Hkv, hd, eff, E, k, vocab,
    window, fa, fw).  Returns (next_token, x_after_each_layer [L+1, d], logits)."""
    d, H, Hkv, hd, fa, fw = cfg["d"], cfg["H"], cfg["Hkv"], cfg["hd"], cfg["fa"], cfg["fw"]
    nb = d // 256
    table_row = o.dequant(_rows(embd_raw, token, nb, 210), 1, nb, o.Q6_K, fa)
    x = table_row.reshape(1, d).astype(np.int64)
    trace = [x.copy()]
    for L in layers:
        h = o.rmsnorm_fixed(x, fa, 1, L["gain"])
        q = onat.qk_linear(L["wq"], h, H * hd, nb, fw, o.Q4_K).reshape(1, H, hd)
        k = onat.qk_linear(L["wk"], h, Hkv * hd, nb, fw, o.Q4_K).reshape(1, Hkv, hd)
        v = onat.qk_linear(L["wv"], h, Hkv * hd, nb, fw, o.Q4_K).reshape(1, Hkv, hd)
        if not L["full"]:
            rot = lambda t: o.rope_fixed(np.transpose(t, (1, 0, 2)), cos[pos:pos + 1], sin[pos:pos + 1], fa).transpose(1, 0, 2)
            q, k = rot(q), rot(k)
        L["k"][:, pos] = k[0]
        L["v"][:, pos] = v[0]
        att = o.attention_cached(q, L["k"][:, :pos + 1], L["v"][:, :pos + 1], pos, H, Hkv, fa, None if L["full"] else cfg["window"])
        ao = onat.qk_linear(L["wo"], att, d, H * hd // 256, fw, o.Q4_K)
        router, gate, up, down = L["moe"]
        moe = onat.moe_block(router, o.Q4_K, gate, up, down, o.Q4_K, o.Q6_K, cfg["k"], h, d, cfg["eff"], fa, fw)[2]
        x = x + ao + moe
        trace.append(x.copy())
    hn = o.rmsnorm_fixed(x, fa, 1, out_gain)
    logits = onat.qk_linear(embd_raw, hn, cfg["vocab"], nb, fw, o.Q6_K)[0]
    best = int(np.flatnonzero(logits == logits.max())[0])
    return best, np.concatenate(trace), logits


def _rows(raw: bytes, row: int, nb: int, block_bytes: int) -> bytes:
    return bytes(raw[row * nb * block_bytes:(row + 1) * nb * block_bytes])


def q1_rows(bits, scale, row: int) -> np.ndarray:
    """Row `row` of a Q1_0 matrix as int64: +scale where the bit is set, -scale elsewhere
    (bonsai/src/trinote/infer_int/reference_bonsai.py:138-146 q1_rows_fp)."""
    signs = o.q1_unpack_signs(np.asarray(bits)[row:row + 1]).astype(np.int64)          # [1, nb, 128] of +-1
    return (signs * np.asarray(scale, np.int64)[row:row + 1, :, None]).reshape(1, -1)


def q1_swiglu(gate, up, frac: int) -> np.ndarray:
    """((gate * sigmoid(gate)) >> frac) * up >> frac with NumPy's wrapping int64 products
    (reference_bonsai.py:245-262 fixed_point_silu, 611-614 _ffn_ref)."""
    gate, up = np.asarray(gate, np.int64), np.asarray(up, np.int64)
    with np.errstate(over="ignore"):
        silu = (gate * o.sigmoid_fixed(gate, frac)) >> frac
        return (silu * up) >> frac


def q1_decode_token(token: int, pos: int, layers, top, cfg, cos, sin):
    """One decode token of the 1-bit decoder (reference_bonsai.py:941-966 _run_layers with one new id, 656-720
    _attention_with_cache_bonsai, 603-615 _ffn_ref, 812-826 greedy head).  layers[i] = dict(n1, n2, qn, kn (int64 gains),
    wqkv, wo, w1u, w2 ((bits, scale) pairs; wqkv = Wq,Wk,Wv rows stacked, w1u = gate rows then up rows), k, v (int64
    caches [Hkv, rows, hd], row `pos` is written here)).  top = dict(embed, head, out_gain).
    cfg = dict(d, H, Hkv, hd, ffn, frac).  Returns (next_token, x_after_each_layer [L+1, d], logits)."""
    d, H, Hkv, hd, ffn, f = cfg["d"], cfg["H"], cfg["Hkv"], cfg["hd"], cfg["ffn"], cfg["frac"]
    qd, kd = H * hd, Hkv * hd
    lin = lambda x, w: onat.q1_linear(x, w[0], w[1], f)
    x = q1_rows(*top["embed"], token)
    trace = [x.copy()]
    for L in layers:
        h = o.rmsnorm_fixed(x, f, 1, L["n1"])
        qkv = lin(h, L["wqkv"])
        q = o.rmsnorm_fixed(qkv[0, :qd].reshape(H, hd), f, 1, L["qn"]).reshape(H, 1, hd)
        k = o.rmsnorm_fixed(qkv[0, qd:qd + kd].reshape(Hkv, hd), f, 1, L["kn"]).reshape(Hkv, 1, hd)
        q = o.rope_fixed(q, cos[pos:pos + 1], sin[pos:pos + 1], f, neox=True)
        k = o.rope_fixed(k, cos[pos:pos + 1], sin[pos:pos + 1], f, neox=True)
        L["k"][:, pos] = k[:, 0]
        L["v"][:, pos] = qkv[0, qd + kd:].reshape(Hkv, hd)
        att = o.attention_cached(q.transpose(1, 0, 2), L["k"][:, :pos + 1], L["v"][:, :pos + 1], pos, H, Hkv, f)
        x = x + lin(att, L["wo"])
        h = o.rmsnorm_fixed(x, f, 1, L["n2"])
        gu = lin(h, L["w1u"])
        x = x + lin(q1_swiglu(gu[:, :ffn], gu[:, ffn:], f), L["w2"])
        trace.append(x.copy())
    logits = lin(o.rmsnorm_fixed(x, f, 1, top["out_gain"]), top["head"])[0]
    return int(np.flatnonzero(logits == logits.max())[0]), np.concatenate(trace), logits
