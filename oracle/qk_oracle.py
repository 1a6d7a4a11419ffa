"""CPU oracle for the integer MoE block and the fused-dequant integer matmul.  TEST INFRASTRUCTURE ONLY.

This module is the checker, never the product: only the test-suite, the smoke entry and the
benchmark's CPU-baseline leg may import it.  It restates, in plain NumPy, the arithmetic of the
reference project's CPU integer oracle so that CUDA results can be compared byte for byte on a box
where the reference tree is not present.

Parity pin: every function here is compared with the reference's own Python implementation by
``tests/golden/make_golden.py`` (run where the reference tree is mounted); the resulting vectors are
committed under ``tests/golden/`` and re-checked by ``tests/test_oracle_golden.py``.

Reference anchors (paths inside the reference project):
  * north-mini-code/src/nmc/qk_codec.py:28-35      6-bit scale/min unpack
  * north-mini-code/src/nmc/qk_codec.py:158-206    whole-tensor Q4_K / Q6_K integer dequant
  * north-mini-code/src/nmc/cohere2.py:97-111      to_fixed, linear, silu_int
  * north-mini-code/src/nmc/cohere2.py:162-188     _topk_lowidx, moe_layer_int
  * north-mini-code/src/nmc/_bonsai/fixedpoint.py:32-72,74-96,136-163   rmsnorm, exp2, sigmoid
  * north-mini-code/tools/nmc_qk_kernel.c:16-39    half -> fixed conversion
  * bonsai/src/trinote/infer_int/reference_bonsai.py:118-128,149-219   Q1_0 linear
"""
from __future__ import annotations

import math

import numpy as np

QK_K = 256
Q4_K, Q6_K = 0, 1
BLOCK_BYTES = {Q4_K: 144, Q6_K: 210}
Q1_GROUP = 128

_LOG2E_Q16 = 94548
_POLY_Q16 = (65536, 45426, 15743, 3638)


# ------------------------------------------------------------------------------------------------
# half -> fixed point
# ------------------------------------------------------------------------------------------------
def half_bits_to_fixed(bits, frac: int) -> np.ndarray:
    """round_half_even(float16(bits) * 2**frac) as int64, using integers only.

    Follows nmc_qk_kernel.c:16-39 (exact half->double, then llrint under round-to-nearest-even)
    and qk_codec.py:57-58 (Python ``round``).  A finite half is ``m * 2**e`` with an 11-bit
    integer ``m``; multiplying by 2**frac is a shift, and a right shift rounds half to even.
    """
    b = np.asarray(bits, dtype=np.uint16).astype(np.int64)
    sign = (b >> 15) & 1
    exp = (b >> 10) & 0x1F
    mant = b & 0x3FF
    m = np.where(exp == 0, mant, mant | 0x400)
    e = np.where(exp == 0, -24, exp - 25) + int(frac)
    out = np.empty(b.shape, dtype=np.int64)
    pos = e >= 0
    out[pos] = m[pos] << e[pos]
    if (~pos).any():
        s = (-e[~pos]).astype(np.int64)
        s = np.minimum(s, 40)                       # m < 2**11: any shift > 12 already yields 0
        mm = m[~pos]
        q = mm >> s
        rem = mm & ((np.int64(1) << s) - 1)
        half = np.int64(1) << (s - 1)
        up = (rem > half) | ((rem == half) & ((q & 1) == 1))
        out[~pos] = q + up.astype(np.int64)
    return np.where(sign == 1, -out, out)


# ------------------------------------------------------------------------------------------------
# block codecs (raw GGUF bytes -> int64 weights at scale 2**frac)
# ------------------------------------------------------------------------------------------------
def unpack_q4k_scales(scales: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """[nb,12] packed bytes -> (sc [nb,8], mn [nb,8]) 6-bit values (qk_codec.py:28-35)."""
    s = np.asarray(scales, dtype=np.int64)
    sc = np.empty(s.shape[:-1] + (8,), np.int64)
    mn = np.empty_like(sc)
    sc[..., :4] = s[..., 0:4] & 63
    mn[..., :4] = s[..., 4:8] & 63
    sc[..., 4:] = (s[..., 8:12] & 0xF) | ((s[..., 0:4] >> 6) << 4)
    mn[..., 4:] = (s[..., 8:12] >> 4) | ((s[..., 4:8] >> 6) << 4)
    return sc, mn


def dequant_q4k(raw, n_blocks_total: int, frac: int) -> np.ndarray:
    """Raw Q4_K bytes -> int64 [n_blocks_total*256]: w = d_q*sc_j*q - dmin_q*m_j (qk_codec.py:158-181).

    Block layout: d(fp16) dmin(fp16) scales[12] qs[128]; group g of 64 weights takes the low
    nibbles of qs[32g..32g+31] for its first 32 weights and the high nibbles for the next 32.
    """
    b = np.frombuffer(raw, np.uint8, n_blocks_total * 144).reshape(n_blocks_total, 144)
    dq = half_bits_to_fixed(b[:, 0:2].copy().view(np.uint16).reshape(-1), frac)[:, None, None]
    dmq = half_bits_to_fixed(b[:, 2:4].copy().view(np.uint16).reshape(-1), frac)[:, None, None]
    sc, mn = unpack_q4k_scales(b[:, 4:16])
    qs = b[:, 16:144].astype(np.int64).reshape(n_blocks_total, 4, 32)
    q = np.stack([qs & 0xF, qs >> 4], axis=2).reshape(n_blocks_total, 8, 32)   # sub-block j = 2g + hi
    w = dq * sc[:, :, None] * q - dmq * mn[:, :, None]
    return w.reshape(-1)


def dequant_q6k(raw, n_blocks_total: int, frac: int) -> np.ndarray:
    """Raw Q6_K bytes -> int64 [n_blocks_total*256]: w = d_q*sc*(q-32) (qk_codec.py:184-206).

    Block layout: ql[128] qh[64] scales[16](int8) d(fp16).  Within each 128-weight half, weight
    32k+l (k=0..3, l=0..31) takes its low 4 bits from ql[(k&1)*32+l] (low nibble for k<2, high
    nibble for k>=2), its high 2 bits from bits 2k..2k+1 of qh[l], and scale index 2k + l//16.
    """
    nb = n_blocks_total
    b = np.frombuffer(raw, np.uint8, nb * 210).reshape(nb, 210)
    ql = b[:, 0:128].astype(np.int64).reshape(nb, 2, 2, 32)       # [blk, half, k&1, l]
    qh = b[:, 128:192].astype(np.int64).reshape(nb, 2, 32)        # [blk, half, l]
    sca = b[:, 192:208].copy().view(np.int8).astype(np.int64).reshape(nb, 2, 8)
    dq = half_bits_to_fixed(b[:, 208:210].copy().view(np.uint16).reshape(-1), frac)
    w = np.empty((nb, 2, 4, 32), np.int64)
    for k in range(4):
        nib = (ql[:, :, k & 1, :] & 0xF) if k < 2 else (ql[:, :, k & 1, :] >> 4)
        q = (nib | (((qh >> (2 * k)) & 3) << 4)) - 32
        s = np.repeat(sca[:, :, 2 * k:2 * k + 2], 16, axis=2)    # [nb, 2, 32]: l//16 picks the scale
        w[:, :, k, :] = dq[:, None, None] * s * q
    return w.reshape(-1)


def dequant(raw, out_f: int, n_blocks: int, qtype: int, frac: int) -> np.ndarray:
    fn = dequant_q4k if qtype == Q4_K else dequant_q6k
    return fn(raw, out_f * n_blocks, frac).reshape(out_f, n_blocks * QK_K)


# ------------------------------------------------------------------------------------------------
# integer building blocks
# ------------------------------------------------------------------------------------------------
def to_fixed(x, frac: int) -> np.ndarray:
    """Activation quantiser: round-half-even(x * 2**frac) as int64 (cohere2.py:97)."""
    return np.round(np.asarray(x, np.float64) * (1 << frac)).astype(np.int64)


def linear(x_int, w_fixed, fw: int) -> np.ndarray:
    """y = floor((x @ W^T) / 2**fw) with an unbounded accumulator (cohere2.py:102-106)."""
    x = np.atleast_2d(np.asarray(x_int)).astype(object)
    w = np.asarray(w_fixed).astype(object)
    return ((x @ w.T) >> fw).astype(np.int64)


def qk_linear(raw, x_int, out_f: int, n_blocks: int, fw: int, qtype: int) -> np.ndarray:
    """Fused form of dequant + linear on raw block bytes (nmc_qk_kernel.c:85-120)."""
    return linear(x_int, dequant(raw, out_f, n_blocks, qtype, fw), fw)


def _scaled_log2e(frac: int) -> int:
    s = 16 - frac
    return _LOG2E_Q16 >> s if s >= 0 else _LOG2E_Q16 << -s


def exp2_neg_fixed(u, frac: int) -> np.ndarray:
    """2**(-u / 2**frac) at scale 2**frac for u >= 0: cubic in the fraction, shifted by the
    integer part (fixedpoint.py:74-96)."""
    u = np.asarray(u, np.int64)
    s = 16 - frac
    c = [(v >> s) if s >= 0 else (v << -s) for v in _POLY_Q16]
    k = u >> frac
    f = u & ((1 << frac) - 1)
    f2 = (f * f) >> frac
    f3 = (f2 * f) >> frac
    poly = c[0] - ((c[1] * f) >> frac) + ((c[2] * f2) >> frac) - ((c[3] * f3) >> frac)
    poly = np.maximum(poly, 0)
    return poly >> np.minimum(k, 63)


def sigmoid_fixed(x, frac: int = 16) -> np.ndarray:
    """Integer sigmoid = second entry of the two-term fixed-point softmax of [0, x]
    (fixedpoint.py:136-163)."""
    assert 1 <= frac <= 29
    x = np.asarray(x, np.int64)
    log2e = _scaled_log2e(frac)
    clip = np.int64(((frac + 2) << (2 * frac)) // log2e)
    m = np.maximum(x, 0)
    d0 = np.minimum(m, clip)
    d1 = np.minimum(m - x, clip)
    e0 = exp2_neg_fixed((d0 * log2e) >> frac, frac)
    e1 = exp2_neg_fixed((d1 * log2e) >> frac, frac)
    z = e0 + e1
    out = np.zeros(x.shape, np.int64)
    nz = z != 0
    out[nz] = (e1[nz] << frac) // z[nz]
    return out


def silu_int(x, fa: int) -> np.ndarray:
    """(x * sigmoid(x)) >> fa with an exact product (cohere2.py:109-111)."""
    x = np.asarray(x, np.int64)
    sig = sigmoid_fixed(x, fa)
    return ((x.astype(object) * sig.astype(object)) >> fa).astype(np.int64)


def mul_shift(a, b, fa: int) -> np.ndarray:
    """(a * b) >> fa with an exact product (cohere2.py:185)."""
    return ((np.asarray(a).astype(object) * np.asarray(b).astype(object)) >> fa).astype(np.int64)


def topk_lowidx(logits_row, k: int) -> np.ndarray:
    """Indices of the k largest values, descending, lowest index first among equals
    (cohere2.py:162-165)."""
    v = np.asarray(logits_row, np.int64)
    order = sorted(range(v.shape[0]), key=lambda i: (-int(v[i]), i))
    return np.asarray(order[:k], dtype=np.int64)


def rmsnorm_fixed(x, frac: int = 16, eps: int = 1, gain=None) -> np.ndarray:
    """Integer RMSNorm: (x << f) // isqrt(sum(x^2)//n + eps), then (* gain) >> f
    (fixedpoint.py:32-72)."""
    x = np.atleast_2d(np.asarray(x, np.int64))
    out = np.empty_like(x)
    n = x.shape[1]
    for r in range(x.shape[0]):
        row = [int(v) for v in x[r]]
        rms = math.isqrt(sum(v * v for v in row) // n + eps)
        out[r] = [(v << frac) // rms for v in row]
    if gain is not None:
        g = np.asarray(gain, np.int64)
        out = ((out.astype(object) * g.astype(object)) >> frac).astype(np.int64)
    return out


# ------------------------------------------------------------------------------------------------
# the MoE block (router -> top-k -> expert SwiGLU -> weighted combine)
# ------------------------------------------------------------------------------------------------
def route(h_int, router_fixed, k: int, fa: int, fw: int):
    """Router logits, selected expert ids (rank order) and sigmoid gate weights
    (cohere2.py:176-180)."""
    logits = linear(h_int, router_fixed, fw)
    ids = np.stack([topk_lowidx(r, k) for r in logits]).astype(np.int32)
    gates = np.stack([sigmoid_fixed(logits[t][ids[t]], fa) for t in range(logits.shape[0])])
    return logits, ids, gates


def expert_ffn(h_row, gate_w, up_w, down_w, fa: int, fw: int) -> np.ndarray:
    """One expert on one token: down((silu(gate h) * up h) >> fa)  (cohere2.py:183-186)."""
    g = silu_int(linear(h_row, gate_w, fw), fa)
    u = linear(h_row, up_w, fw)
    return linear(mul_shift(g, u, fa), down_w, fw)[0]


def moe_layer(h_int, router_fixed, experts, k: int, fa: int, fw: int):
    """Full MoE FFN on [T, d] tokens.  ``experts(e)`` returns (gate, up, down) int64 matrices.
    out[t] = sum_j ((expert_{sel_j}(h_t) * gate_j) >> fa): one floor per selected expert, then an
    exact sum (cohere2.py:168-188).  Returns (ids, gates, out)."""
    h = np.atleast_2d(np.asarray(h_int, np.int64))
    _, ids, gates = route(h, router_fixed, k, fa, fw)
    out = np.zeros((h.shape[0], h.shape[1]), dtype=object)
    for t in range(h.shape[0]):
        for j in range(k):
            gw, uw, dw = experts(int(ids[t, j]))
            eo = expert_ffn(h[t:t + 1], gw, uw, dw, fa, fw).astype(object)
            out[t] += (eo * int(gates[t, j])) >> fa
    return ids, gates, out.astype(np.int64)


# ------------------------------------------------------------------------------------------------
# attention sublayer: RoPE tables, rotation, softmax, KV-cached GQA attention
# ------------------------------------------------------------------------------------------------
def build_rope_tables(seq_len: int, head_dim: int, base: float = 10000.0, frac: int = 16):
    """cos/sin at scale 2**frac, shape [seq_len, head_dim // 2]: round(cos(p * base**(-2i/d)) * 2**frac)
    (_bonsai/rope.py:42-66)."""
    import math
    half = head_dim // 2
    inv = [base ** (-(2 * i) / head_dim) for i in range(half)]
    cos = np.empty((seq_len, half), np.int64)
    sin = np.empty((seq_len, half), np.int64)
    for p in range(seq_len):
        for i in range(half):
            cos[p, i] = round(math.cos(p * inv[i]) * (1 << frac))
            sin[p, i] = round(math.sin(p * inv[i]) * (1 << frac))
    return cos, sin


def rope_fixed(x, cos, sin, frac: int = 16, neox: bool = False) -> np.ndarray:
    """x [..., seq, hd] rotated with table rows 0..seq-1.  Interleaved pairs (2i, 2i+1)
    (_bonsai/rope.py:79-100) or rotate-half pairs (i, i + hd/2) (_bonsai/rope_v2.py:92-117):
    out0 = (x0 c - x1 s) >> frac, out1 = (x0 s + x1 c) >> frac."""
    x = np.asarray(x, np.int64)
    seq, hd = x.shape[-2], x.shape[-1]
    c, s = cos[:seq], sin[:seq]
    out = np.empty_like(x)
    if neox:
        x0, x1 = x[..., :hd // 2], x[..., hd // 2:]
        out[..., :hd // 2] = (x0 * c - x1 * s) >> frac
        out[..., hd // 2:] = (x0 * s + x1 * c) >> frac
    else:
        x0, x1 = x[..., 0::2], x[..., 1::2]
        out[..., 0::2] = (x0 * c - x1 * s) >> frac
        out[..., 1::2] = (x0 * s + x1 * c) >> frac
    return out


def softmax_fixed(z, frac: int = 16) -> np.ndarray:
    """Row softmax in integers: d = min(max - z, clip); e = 2**-(d log2e); p = (e << frac) // sum(e)
    (_bonsai/fixedpoint.py:99-133)."""
    z = np.atleast_2d(np.asarray(z, np.int64))
    log2e = _scaled_log2e(frac)
    clip = min(((frac + 2) << (2 * frac)) // log2e, (1 << 62) // log2e)
    out = np.empty_like(z)
    for r in range(z.shape[0]):
        d = np.minimum(int(z[r].max()) - z[r], clip)
        e = exp2_neg_fixed((d * log2e) >> frac, frac)
        tot = int(e.sum())
        out[r] = 0 if tot == 0 else (e << frac) // tot
    return out


def attention_cached(q, ck, cv, start: int, n_heads: int, n_kv: int, fa: int = 16, window=None, inv_sqrt=None):
    """m queries q [m, H, hd] at absolute positions start.. over the cache ck/cv [Hkv, Lc, hd] (Lc = start + m):
    scores = ((q k^T) >> fa) * inv_sqrt >> fa, causal + sliding-window mask with -(2**(fa+30)), integer softmax,
    out = (p v) >> fa  ->  [m, H*hd]  (cohere2.py:324-354)."""
    import math
    q = np.asarray(q, np.int64)
    m, H, hd = q.shape
    Lc = ck.shape[1]
    rep = n_heads // n_kv
    if inv_sqrt is None:
        inv_sqrt = int(round((1.0 / math.sqrt(hd)) * (1 << fa)))
    neg = -(1 << (fa + 30))
    out = np.empty((m, H, hd), np.int64)
    for h in range(H):
        kh, vh = np.asarray(ck[h // rep], np.int64), np.asarray(cv[h // rep], np.int64)
        scores = ((q[:, h, :] @ kh.T) >> fa)
        scores = (scores * inv_sqrt) >> fa
        for i in range(m):
            p = start + i
            scores[i, p + 1:] = neg
            if window is not None and p - window >= 0:
                scores[i, :p - window + 1] = neg
        out[:, h, :] = (softmax_fixed(scores, fa) @ vh) >> fa
    return out.reshape(m, H * hd)


# ------------------------------------------------------------------------------------------------
# balanced base-256 limbs (the decomposition the tensor/dp4a style kernels rely on)
# ------------------------------------------------------------------------------------------------
def balanced_capacity(n_limbs: int) -> int:
    """Largest |x| that n balanced digits in [-128,127] represent: 127*(256**n-1)/255
    (qk_cuda.py:973-976)."""
    return 127 * ((256 ** n_limbs - 1) // 255)


def limbs_needed(maxabs: int) -> int:
    """Smallest digit count in 1..8 covering +-maxabs, OverflowError beyond 8 (qk_cuda.py:979-992)."""
    m = int(maxabs)
    for n in range(1, 9):
        if m <= balanced_capacity(n):
            return n
    raise OverflowError(f"|x| max {m} exceeds 8 balanced base-256 digits")


def balanced_limbs(x, n_limbs: int) -> np.ndarray:
    """int64 [n] -> int8 [n_limbs, n]: signed low byte, subtract, shift, repeat."""
    v = np.asarray(x, np.int64).copy()
    out = np.empty((n_limbs,) + v.shape, np.int8)
    for l in range(n_limbs):
        out[l] = v.astype(np.int8)
        v = (v >> 8) + ((v >> 7) & 1)               # (v - digit) / 256 without leaving int64
    return out


# ------------------------------------------------------------------------------------------------
# Q1_0 (1-bit) linear
# ------------------------------------------------------------------------------------------------
def q1_unpack_signs(bits) -> np.ndarray:
    """[out, nb, 16] packed bytes -> [out, nb, 128] in {-1,+1}; bit i of byte j (LSB first) is
    weight 8j+i, set bit = +1 (reference_bonsai.py:118-123)."""
    u = np.unpackbits(np.asarray(bits, np.uint8), axis=-1, bitorder="little").astype(np.int64)
    return u * 2 - 1


def q1_linear(x_int, bits, scale_fp, frac: int) -> np.ndarray:
    """out[t,o] = sum_b arshift((sum_i sign*x) * scale[o,b], frac), every step modulo 2**64
    (reference_bonsai.py:100-113,149-219; bonsai_q1_kernel.c:85-106)."""
    x = np.atleast_2d(np.asarray(x_int, np.int64))
    s = np.asarray(scale_fp, np.int64)
    out_f, nb = s.shape
    signs = q1_unpack_signs(bits)
    xg = x.reshape(x.shape[0], nb, Q1_GROUP)
    with np.errstate(over="ignore"):
        acc = np.einsum("tbi,obi->tob", xg, signs)
        return ((acc * s[None]) >> frac).sum(axis=2, dtype=np.int64)


# ------------------------------------------------------------------------------------------------
# seeded synthetic tensors (raw block bytes with the benchmark's value distributions)
# ------------------------------------------------------------------------------------------------
def synth_q4k(rng: np.random.Generator, out_f: int, n_blocks: int, dmag: float = 0.01) -> bytes:
    """Random Q4_K tensor: d, dmin = float16(|N(0,1)|*dmag); scales and nibbles uniform bytes.
    Draw order: d, dmin, scales, qs."""
    n = out_f * n_blocks
    blk = np.empty((n, 144), np.uint8)
    blk[:, 0:2] = np.abs(rng.standard_normal(n) * dmag).astype(np.float16).view(np.uint8).reshape(n, 2)
    blk[:, 2:4] = np.abs(rng.standard_normal(n) * dmag).astype(np.float16).view(np.uint8).reshape(n, 2)
    blk[:, 4:16] = rng.integers(0, 256, size=(n, 12), dtype=np.uint8)
    blk[:, 16:144] = rng.integers(0, 256, size=(n, 128), dtype=np.uint8)
    return blk.tobytes()


def synth_q6k(rng: np.random.Generator, out_f: int, n_blocks: int, dmag: float = 0.01) -> bytes:
    """Random Q6_K tensor: ql, qh uniform bytes, int8 scales uniform in [-128,127],
    d = float16(|N(0,1)|*dmag).  Draw order: ql, qh, scales, d."""
    n = out_f * n_blocks
    blk = np.empty((n, 210), np.uint8)
    blk[:, 0:128] = rng.integers(0, 256, size=(n, 128), dtype=np.uint8)
    blk[:, 128:192] = rng.integers(0, 256, size=(n, 64), dtype=np.uint8)
    blk[:, 192:208] = rng.integers(-128, 128, size=(n, 16), dtype=np.int8).view(np.uint8)
    blk[:, 208:210] = np.abs(rng.standard_normal(n) * dmag).astype(np.float16).view(np.uint8).reshape(n, 2)
    return blk.tobytes()


def synth_q1(rng: np.random.Generator, out_f: int, n_blocks: int, frac: int = 16, smag: float = 0.02):
    """Random Q1_0 tensor: packed sign bytes and int64 scales rint(float16(|N(0,1)|*smag)*2**frac)."""
    bits = rng.integers(0, 256, size=(out_f, n_blocks, 16), dtype=np.uint8)
    sc16 = np.abs(rng.standard_normal((out_f, n_blocks)) * smag).astype(np.float16)
    scale = np.rint(sc16.astype(np.float64) * (1 << frac)).astype(np.int64)
    return bits, scale


def synth_moe(seed: int, d: int, eff: int, n_experts: int, T: int, fa: int = 16):
    """One MoE block's raw tensors and input: Q4_K router [E,d], per expert Q4_K gate/up [eff,d] and
    Q6_K down [d,eff], hidden state to_fixed(N(0,1) [T,d]).  Draw order: router, then per expert
    gate, up, down, then the hidden state."""
    rng = np.random.default_rng(seed)
    router = synth_q4k(rng, n_experts, d // 256)
    gate, up, down = [], [], []
    for _ in range(n_experts):
        gate.append(synth_q4k(rng, eff, d // 256))
        up.append(synth_q4k(rng, eff, d // 256))
        down.append(synth_q6k(rng, d, eff // 256))
    h = to_fixed(rng.standard_normal((T, d)), fa)
    return router, gate, up, down, h


# Cases the committed golden vectors were generated for: (qtype, out_f, n_blocks, T, log2 |x| bound)
GOLDEN_LINEAR_CASES = [(0, 8, 1, 1, 18), (0, 16, 2, 3, 18), (1, 5, 3, 4, 18), (1, 64, 2, 2, 30), (0, 7, 2, 2, 40),
                       (1, 9, 1, 1, 50)]
# name -> (seed, d_model, expert_ffn, n_experts, top_k, tokens); "config1" is the single-block benchmark shape
GOLDEN_MOE_CASES = {"small": (400, 256, 256, 8, 3, 4), "config1": (0, 2048, 768, 128, 8, 16)}


# The small decoder the committed decode-step fixture (tests/golden/nmc_decode.npz) was recorded on: two blocks, the first
# attends to every key without rotation, the second through a sliding window with interleaved RoPE (cohere2.py:72-84).
NMC_DECODE_CASE = {"seed": 900, "d": 256, "H": 4, "Hkv": 2, "hd": 64, "eff": 256, "E": 8, "k": 2, "vocab": 96, "window": 4,
                   "rope_base": 50000.0, "rows": 16, "prompt": (3, 90, 41, 7, 66, 12), "steps": 3, "layers": 2}


def synth_decoder(seed: int, case: dict, fa: int = 16) -> dict:
    """Raw tensors of a small decoder of the north-mini-code shape.  Draw order per block: norm gain
    (to_fixed(|N(0,1)| + 0.5), cohere2.py:511), Wq, Wk, Wv, Wo (Q4_K), router, then per expert gate, up (Q4_K), down
    (Q6_K); after the blocks the output-norm gain and the tied embedding / head matrix (Q6_K).  Returns
    {"layers": [{gain, wq, wk, wv, wo, moe: (router, gates, ups, downs)}], "out_gain", "embd"}."""
    rng = np.random.default_rng(seed)
    d, H, Hkv, hd, eff, E = (case[n] for n in ("d", "H", "Hkv", "hd", "eff", "E"))
    nb = d // 256
    layers = []
    for _ in range(case["layers"]):
        L = {"gain": to_fixed(np.abs(rng.standard_normal(d)) + 0.5, fa)}
        L["wq"] = synth_q4k(rng, H * hd, nb); L["wk"] = synth_q4k(rng, Hkv * hd, nb); L["wv"] = synth_q4k(rng, Hkv * hd, nb)
        L["wo"] = synth_q4k(rng, d, H * hd // 256)
        router = synth_q4k(rng, E, nb)
        gate, up, down = [], [], []
        for _e in range(E):
            gate.append(synth_q4k(rng, eff, nb)); up.append(synth_q4k(rng, eff, nb)); down.append(synth_q6k(rng, d, eff // 256))
        L["moe"] = (router, gate, up, down)
        layers.append(L)
    out_gain = to_fixed(np.abs(rng.standard_normal(d)) + 0.5, fa)
    embd = synth_q6k(rng, case["vocab"], nb)
    return {"layers": layers, "out_gain": out_gain, "embd": embd}


# The synthetic checkpoint and request the committed generation fixture (tests/golden/engine_generate.npz) was recorded on:
# two MoE blocks (the first full attention without rotation, the second a sliding window of 8 with RoPE), a prompt longer
# than the window, eight greedy tokens.
ENGINE_CASE = {"model": dict(n_layers=2, d_model=256, n_heads=4, n_kv=2, head_dim=64, e_ffn=256, n_experts=8, top_k=2, vocab=96,
                             window=8, context=64, rope_base=50000.0, seed=5),
               "prompt": (3, 50, 7, 11, 90, 2, 33, 8, 41, 5), "n_new": 8}
