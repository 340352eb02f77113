"""Failure detection on the device without a fault: a bounded wait that runs out.

Every tcgen05 kernel of the library waits on its barriers through one helper with a time limit;
when the limit passes the kernel records which wait gave up and returns normally.  The reference
has no counterpart (it checks cudaGetLastError after each launch, kernels/src/cuda/Attention.cu:119);
this test drives the helper through attn_sm100_selftest_wait_limit, whose kernel waits on a barrier
nothing completes, and checks that the status is reported, can be cleared, and that the context
keeps working afterwards.
"""
import time

import numpy as np
import pytest

torch = pytest.importorskip("torch")

pytestmark = pytest.mark.gpu


def test_wait_limit_reports_status_and_context_survives(pkg, oracle):
    pkg.init()
    assert pkg.device_status() == 0
    L = pkg.lib()
    stream = torch.cuda.current_stream().cuda_stream

    t0 = time.perf_counter()
    assert L.attn_sm100_selftest_wait_limit(2000, stream) == 0  # 2 ms
    code = pkg.device_status(clear=False)
    elapsed = time.perf_counter() - t0
    assert code == 1900, code
    assert elapsed < 1.0, f"the wait took {elapsed:.3f} s for a 2 ms limit"
    # the word is sticky until cleared ...
    assert pkg.device_status(clear=True) == 1900
    # ... and clean afterwards
    assert pkg.device_status() == 0

    # the context is still usable: a forward pass right after matches the oracle
    B, T, H, D = 1, 160, 2, 64
    g = torch.Generator(device="cpu").manual_seed(5)
    x = torch.randn(B, T, 3 * H * D, generator=g)
    out, _ = pkg.forward(x.cuda(), H)
    ref = oracle.forward(x.numpy(), H)
    assert np.abs(out.cpu().numpy() - ref).max() < 2e-3
    assert pkg.device_status() == 0


def test_wait_limit_argument_range(pkg):
    L = pkg.lib()
    assert L.attn_sm100_selftest_wait_limit(0, None) == -2
    assert L.attn_sm100_selftest_wait_limit(100001, None) == -2
