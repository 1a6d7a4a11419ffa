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
