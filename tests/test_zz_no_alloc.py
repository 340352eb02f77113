"""attn_sm100_forward_static: the forward entry point that allocates nothing.

It serves callers that cannot hand the library a scratch buffer and must keep it out of the CUDA
allocator (a process whose own pool owns the device memory, a serving loop that cannot afford the
stall of a cudaMalloc).  Its scratch is a fixed 16 MiB device array inside the library, shared by
all calls and never cleared, so the test calls it twice in a row with different inputs and checks
each result against the ordinary entry point and against the CPU oracle, reads the entry point's own
status word after each call, and checks that a problem beyond the array's capacity is refused with
its own error code.

This file sorts last on purpose: a run that stops at the first failure has then already run every
other test.  It also passes when run alone in a fresh process (the first call performs the
per-device set-up itself).
"""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ERR_STATIC_CAPACITY = -7


def _static_forward(pkg, torch, xt, H):
    B, T, C3 = xt.shape
    D = C3 // 3 // H
    out = torch.empty((B, T, C3 // 3), device="cuda", dtype=torch.float32)
    lse = torch.empty((B, H, T), device="cuda", dtype=torch.float32)
    rc = pkg.lib().attn_sm100_forward_static(xt.data_ptr(), out.data_ptr(), lse.data_ptr(), B, T, H, D,
                                             torch.cuda.current_stream().cuda_stream)
    return rc, out, lse


def test_static_forward_matches_regular_forward_twice(pkg, oracle):
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    torch.cuda.set_device(0)
    rng = np.random.default_rng(77)
    # two calls in a row, different shapes and data: the shared array keeps the first call's bytes
    for B, T, H in [(2, 300, 3), (1, 130, 2)]:
        x = rng.standard_normal((B, T, 3 * H * 64), dtype=np.float32)
        xt = torch.from_numpy(x).cuda()
        rc, out, lse = _static_forward(pkg, torch, xt, H)
        assert rc == 0, pkg.lib().attn_sm100_strerror(rc)
        # this path has its own status word: a bounded wait that ran out inside its kernel shows here
        assert pkg.static_status() == 0
        ref_out, ctx = pkg.forward(xt, H)
        assert pkg.device_status() == 0
        # same kernels on the same split: the tolerance of the other tests is 2e-3, here the bits agree
        assert float((out - ref_out).abs().max()) <= 2e-3
        assert torch.equal(out, ref_out)
        assert float((lse - ctx.lse).abs().max()) <= 1e-4
        # ... and against the CPU oracle, within the tolerance of the forward path
        want = oracle.forward(x, H)
        assert float(np.abs(out.cpu().numpy() - want).max()) <= 2e-3


def test_static_forward_rejects_what_does_not_fit(pkg):
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    L = pkg.lib()
    one = ctypes.c_void_p(256)
    # 8 x 1024 x 2304 = 18.9 M elements > 4,194,304: refused before anything is launched
    assert L.attn_sm100_forward_static(one, one, one, 8, 1024, 12, 64, None) == ERR_STATIC_CAPACITY
    assert b"4,194,304" in L.attn_sm100_strerror(ERR_STATIC_CAPACITY)
    assert L.attn_sm100_forward_static(one, one, one, 1, 16, 2, 32, None) == -3  # only D = 64 has this variant
    assert L.attn_sm100_forward_static(None, one, one, 1, 16, 2, 64, None) == -1
