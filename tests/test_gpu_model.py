"""GPU parity of whole decode steps (embedding -> blocks with attention + MoE -> tied head -> greedy pick)
against the CPU checker, on a small decoder; eager and as one replayed CUDA graph."""
import numpy as np
import pytest

from oracle import model_oracle
from oracle import qk_oracle as o

pytestmark = pytest.mark.gpu


def _host_view(model):
    from integer_inference_engine_b200.model import host_view
    return host_view(model)


FORMS = pytest.mark.parametrize(("one_launch", "fused_block"), [(True, True), (False, True), (False, False)],
                                ids=["all-blocks-in-one-launch", "five-launches-per-block", "two-entries-per-block"])


@FORMS
def test_decode_steps_match_the_checker_eager_and_replayed(one_launch, fused_block):
    import torch

    from integer_inference_engine_b200 import device, qk_cuda as qk
    from integer_inference_engine_b200.model import SyntheticDecoder
    qk.free_all()
    model = SyntheticDecoder(n_layers=5, d_model=512, n_heads=8, n_kv=2, head_dim=64, e_ffn=256, n_experts=8, top_k=2,
                             vocab=1000, context=40, max_new=12, window=16, seed=3, one_launch=one_launch)
    assert (model.kernel is not None) == one_launch
    model.fused_block = fused_block
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
    model.capture(pos + 5)                                  # the captured launches use an upper bound of the position
    for i in range(4):                                      # replayed: position and token advance on the device
        model.replay()
        got.append(int(model.token.item()))
    with pytest.raises(qk.CudaContextError):                # position pos + 6 is past the bound the graph was captured for:
        model.replay()                                      # refused on the host, nothing is launched
    assert int(model.pos.item()) == pos + 6
    assert device.read_flags() == 0
    assert got == want
    assert model.fused_block == fused_block                 # the five-launch form was not silently dropped
    for li in (0, 1, 4):                                    # the caches hold what the checker appended
        assert np.array_equal(model.attn[li]["k"][:, pos:pos + 6].cpu().numpy(), layers[li]["k"][:, pos:pos + 6].astype(np.int32))


def test_replay_is_refused_after_the_workspaces_changed():
    """A captured step holds the library's scratch addresses: once a larger call has regrown them, or they were released,
    replay() raises instead of launching on freed memory."""
    import torch

    from integer_inference_engine_b200 import device, qk_cuda as qk
    from integer_inference_engine_b200.model import SyntheticDecoder
    qk.free_all()
    model = SyntheticDecoder(n_layers=1, d_model=256, n_heads=4, n_kv=2, head_dim=64, e_ffn=256, n_experts=4, top_k=2,
                             vocab=128, context=8, max_new=8, window=16, seed=4)
    model.token.fill_(5)
    model.capture(12)
    model.replay()
    torch.cuda.synchronize()
    gen = device.workspace_generation()
    big = torch.zeros((64, 256), dtype=torch.int64, device="cuda")
    model.moe_layers[0].forward(big, model.fa, model.fw)    # 64 rows: the digit-plane scratch of one row must grow
    torch.cuda.synchronize()
    assert device.workspace_generation() != gen
    with pytest.raises(qk.CudaContextError):
        model.replay()
    model.capture(12)                                       # capturing again makes the step usable
    model.replay()
    torch.cuda.synchronize()
    assert device.read_flags() == 0
    qk.free_all()


@FORMS
def test_reference_recorded_decode_steps(golden_dir, one_launch, fused_block):
    """Three decode steps recorded from the reference's own block_cached / tied_head_int (tests/golden/nmc_decode.npz): the
    device decoder built from the same raw tensors and prompt caches yields the same picks, residual rows and cache rows."""
    import torch

    from integer_inference_engine_b200 import device, qk_cuda as qk
    from integer_inference_engine_b200.model import Decoder
    qk.free_all()
    g = np.load(golden_dir / "nmc_decode.npz")
    case = o.NMC_DECODE_CASE
    m = o.synth_decoder(case["seed"], case)
    n_prompt = len(case["prompt"])
    dec = Decoder.from_raw(m["layers"], m["embd"], m["out_gain"], d_model=case["d"], n_heads=case["H"], n_kv=case["Hkv"],
                           head_dim=case["hd"], e_ffn=case["eff"], top_k=case["k"], vocab=case["vocab"], window=case["window"],
                           rows=case["rows"], rope_base=case["rope_base"], caches=[(g[f"k{li}"], g[f"v{li}"]) for li in range(2)],
                           position=n_prompt, one_launch=one_launch)
    assert (dec.kernel is not None) == one_launch
    dec.fused_block = fused_block
    assert np.array_equal(dec.cos.cpu().numpy(), g["cos"]) and np.array_equal(dec.sin.cpu().numpy(), g["sin"])
    dec.token.fill_(int(g["picks"][0]))
    for step in range(case["steps"]):
        dec.step(n_prompt + step)
        torch.cuda.synchronize()
        assert np.array_equal(dec.x.cpu().numpy()[0], g["x"][step][-1]), step
        assert np.array_equal(dec.logits.cpu().numpy()[0], g["logits"][step]), step
        assert int(dec.token.item()) == int(g["picks"][step + 1])
    assert device.read_flags() == 0 and dec.fused_block == fused_block
    n = n_prompt + case["steps"]
    for li in range(2):
        assert np.array_equal(dec.attn[li]["k"][:, :n].cpu().numpy(), g[f"k{li}_after"].astype(np.int32))
        assert np.array_equal(dec.attn[li]["v"][:, :n].cpu().numpy(), g[f"v{li}_after"].astype(np.int32))
    qk.free_all()
