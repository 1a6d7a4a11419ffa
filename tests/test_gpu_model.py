"""GPU parity of whole decode steps (embedding -> blocks with attention + MoE -> tied head -> greedy pick)
against the CPU checker, on a small decoder; eager and as one replayed CUDA graph."""
import numpy as np
import pytest

from oracle import model_oracle
from oracle import qk_oracle as o

pytestmark = pytest.mark.gpu


def _host_view(model):
    from integer_inference_engine_b200 import device
    nb = model.d // 256
    layers = []
    for li in range(model.n_layers):
        a, hs = model.attn[li], model.moe.handles[li]
        E = model.moe.n_experts
        qr, kr = model.H * model.hd, model.Hkv * model.hd
        fused = device.export_weight(a["wqkv"], qr + 2 * kr, nb, o.Q4_K)          # rows of Wq, Wk, Wv stacked
        cut = lambda r0, r1: bytes(fused[r0 * nb * 144:r1 * nb * 144])
        layers.append({
            "gain": hs["gain"].cpu().numpy(), "wq": cut(0, qr), "wk": cut(qr, qr + kr), "wv": cut(qr + kr, qr + 2 * kr),
            "wo": device.export_weight(a["wo"], model.d, model.H * model.hd // 256, o.Q4_K),
            "k": a["k"].cpu().numpy().astype(np.int64), "v": a["v"].cpu().numpy().astype(np.int64), "full": model.layer_is_full(li),
            "moe": (device.export_weight(hs["router"], E, nb, o.Q4_K),
                    [device.export_weight(h, model.moe.e_ffn, nb, o.Q4_K) for h in hs["gate"]],
                    [device.export_weight(h, model.moe.e_ffn, nb, o.Q4_K) for h in hs["up"]],
                    [device.export_weight(h, model.d, model.moe.e_ffn // 256, o.Q6_K) for h in hs["down"]])})
    cfg = dict(d=model.d, H=model.H, Hkv=model.Hkv, hd=model.hd, eff=model.moe.e_ffn, E=model.moe.n_experts, k=model.top_k,
               vocab=model.vocab, window=model.window, fa=model.fa, fw=model.fw)
    embd = device.export_weight(model.embd, model.vocab, nb, o.Q6_K)
    return layers, embd, model.out_gain.cpu().numpy(), cfg


@pytest.mark.parametrize("overlap", [False, True], ids=["halves-in-sequence", "halves-side-by-side"])
def test_decode_steps_match_the_checker_eager_and_replayed(overlap):
    import torch

    from integer_inference_engine_b200 import device, qk_cuda as qk
    from integer_inference_engine_b200.model import SyntheticDecoder
    qk.free_all()
    device.set_block_overlap(overlap)
    model = SyntheticDecoder(n_layers=5, d_model=512, n_heads=8, n_kv=2, head_dim=64, e_ffn=256, n_experts=8, top_k=2,
                             vocab=1000, context=40, max_new=12, window=16, seed=3)
    layers, embd, out_gain, cfg = _host_view(model)
    cos, sin = model.cos.cpu().numpy(), model.sin.cpu().numpy()
    tok, pos = 123, model.context
    model.token.fill_(tok)
    want = []
    t = tok
    for i in range(6):                                      # the checker's own greedy chain
        t, _, _ = model_oracle.decode_token(t, pos + i, layers, embd, out_gain, cfg, cos, sin)
        want.append(t)
    got = []
    for i in range(2):                                      # eager
        model.step(pos + i)
        got.append(int(model.token.item()))
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        snapshot = (model.token.clone(), model.pos.clone())
        with torch.cuda.graph(g, stream=side):
            model.step(pos + 11)                            # the captured launches use the upper bound of the position
        model.token.copy_(snapshot[0]); model.pos.copy_(snapshot[1])
    torch.cuda.synchronize()
    for i in range(4):                                      # replayed: position and token advance on the device
        g.replay()
        got.append(int(model.token.item()))
    device.set_block_overlap(False)
    assert device.read_flags() == 0
    assert got == want
    for li in (0, 1, 4):                                    # the caches hold what the checker appended
        assert np.array_equal(model.attn[li]["k"][:, pos:pos + 6].cpu().numpy(), layers[li]["k"][:, pos:pos + 6].astype(np.int32))
