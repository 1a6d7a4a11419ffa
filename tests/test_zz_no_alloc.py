"""GPU test of the allocation-free product entry, collected last.

``iie_apply_dev_static`` serves callers that cannot let the library allocate device memory at call
time (their own memory pool already holds the whole device, or they sit in a loop that must not
absorb the synchronisation of an allocation): its activation scratch is a fixed array inside the
library.  The test calls it through the C-ABI twice in a row, with different inputs, and requires
byte-identical results to the ordinary entry ``iie_apply_dev`` and to the CPU oracle; the second call
would expose stale scratch from the first.  It also checks that the call allocates nothing (the
library's workspace counter and the free device memory stay as they were) and that a request beyond
the fixed size is refused.
"""
import numpy as np
import pytest

from oracle import qk_oracle as o

pytestmark = pytest.mark.gpu

FW = 24


def _free_device_bytes():
    import torch
    return torch.cuda.mem_get_info()[0]


def test_static_scratch_entry_matches_the_allocating_entry_twice_in_a_row():
    import torch

    from integer_inference_engine_b200 import device, qk_cuda
    from oracle import native as onat
    assert qk_cuda.available(), "CUDA library or GPU missing"
    lib = qk_cuda._lib()
    rng = np.random.default_rng(2024)
    # (qtype, rows of the matrix, 256-column blocks, activation rows, weight scale bits): one row and several rows inside
    # the fast envelope, and fw = 40 outside it, where the entry runs the exact 128-bit kernel (no scratch at all)
    cases = [(o.Q4_K, 40, 8, 3, FW), (o.Q6_K, 24, 3, 5, FW), (o.Q4_K, 264, 2, 1, FW), (o.Q6_K, 16, 2, 2, 40)]
    for qt, out_f, nb, T, fw in cases:
        raw = (o.synth_q4k if qt == o.Q4_K else o.synth_q6k)(rng, out_f, nb)
        h = qk_cuda.register_weight(raw, out_f, nb, qt)
        # the first call on a device resolves the scratch address and the driver may load the kernels' code then;
        # that set-up is not part of what is measured below
        warm_x = torch.zeros((T, nb * 256), dtype=torch.int64, device="cuda")
        warm_out = torch.zeros((T, out_f), dtype=torch.int64, device="cuda")
        with qk_cuda._CUDA_LOCK:
            assert lib.iie_apply_dev_static(h, warm_x.data_ptr(), T, fw, warm_out.data_ptr(),
                                            torch.cuda.current_stream().cuda_stream) == 0
        torch.cuda.synchronize()
        for call in range(2):                                   # two calls in a row share the scratch array
            xh = rng.integers(-(1 << (18 + 4 * call)), 1 << (18 + 4 * call), size=(T, nb * 256), dtype=np.int64)
            x = torch.from_numpy(xh).cuda()
            want = device.apply(h, x, out_f, fw)
            got = torch.empty_like(want)
            torch.cuda.synchronize()
            allocs, free_before = qk_cuda.moe_workspace_allocations(), _free_device_bytes()
            with qk_cuda._CUDA_LOCK:
                rc = lib.iie_apply_dev_static(h, x.data_ptr(), T, fw, got.data_ptr(),
                                              torch.cuda.current_stream().cuda_stream)
            assert rc == 0
            torch.cuda.synchronize()
            # nothing was allocated: neither a library workspace nor any other device memory
            assert qk_cuda.moe_workspace_allocations() == allocs and _free_device_bytes() == free_before
            assert device.read_flags() == 0
            assert torch.equal(got, want), (qt, call)
            assert np.array_equal(got.cpu().numpy(), onat.qk_linear(raw, xh, out_f, nb, fw, qt)), (qt, call, "oracle")
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
