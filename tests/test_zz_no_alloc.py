"""GPU test of the allocation-free product entry, collected last.

``iie_apply_dev_static`` serves callers that cannot let the library allocate device memory at call
time (their own memory pool already holds the whole device, or they sit in a loop that must not
absorb the synchronisation of an allocation): its activation scratch is a fixed array inside the
library.  The test calls it through the C-ABI twice in a row, with different inputs, and requires
byte-identical results to the ordinary entry ``iie_apply_dev``; the second call would expose stale
scratch from the first.  It also checks that a request beyond the fixed size is refused.
"""
import numpy as np
import pytest

from oracle import qk_oracle as o

pytestmark = pytest.mark.gpu

FW = 24


def test_static_scratch_entry_matches_the_allocating_entry_twice_in_a_row():
    import torch

    from integer_inference_engine_b200 import device, qk_cuda
    assert qk_cuda.available(), "CUDA library or GPU missing"
    lib = qk_cuda._lib()
    rng = np.random.default_rng(2024)
    cases = [(o.Q4_K, 40, 8, 3), (o.Q6_K, 24, 3, 5)]
    for qt, out_f, nb, T in cases:
        raw = (o.synth_q4k if qt == o.Q4_K else o.synth_q6k)(rng, out_f, nb)
        h = qk_cuda.register_weight(raw, out_f, nb, qt)
        for call in range(2):                                   # two calls in a row share the scratch array
            x = torch.from_numpy(rng.integers(-(1 << (18 + 4 * call)), 1 << (18 + 4 * call), size=(T, nb * 256),
                                              dtype=np.int64)).cuda()
            want = device.apply(h, x, out_f, FW)
            got = torch.empty_like(want)
            with qk_cuda._CUDA_LOCK:
                rc = lib.iie_apply_dev_static(h, x.data_ptr(), T, FW, got.data_ptr(),
                                              torch.cuda.current_stream().cuda_stream)
            assert rc == 0
            torch.cuda.synchronize()
            assert device.read_flags() == 0
            assert torch.equal(got, want), (qt, call)
    # 4 MiB of limb planes: T * 8 * in_features bytes; one row more than fits is refused with rc 4
    raw = o.synth_q4k(rng, 8, 8)
    h = qk_cuda.register_weight(raw, 8, 8, o.Q4_K)
    too_many = (4 << 20) // (8 * 2048) + 1
    x = torch.zeros((too_many, 2048), dtype=torch.int64, device="cuda")
    out = torch.zeros((too_many, 8), dtype=torch.int64, device="cuda")
    with qk_cuda._CUDA_LOCK:
        assert lib.iie_apply_dev_static(h, x.data_ptr(), too_many, FW, out.data_ptr(), 0) == 4
        assert lib.iie_apply_dev_static(h, x.data_ptr(), too_many - 1, FW, out.data_ptr(), 0) == 0
    torch.cuda.synchronize()
    qk_cuda.free_all()
