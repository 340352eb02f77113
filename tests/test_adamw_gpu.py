"""Parity of the AdamW step (include/adamw_sm100.h) against the numpy restatement of the reference's update in
oracle/ops_oracle.py, pinned to the reference's own CPU kernel by tests/test_ops_oracle.py
(kernels/src/cuda/AdamW.cu:13-57, same formula as kernels/src/cpu/AdamW.c): decoupled weight decay, moments
by lerp(a, b, w) = fma(w, b, fma(-w, a, a)), bias corrections as multiplications.  The restatement runs in
float64 with a rounding to float32 after every operation the kernel rounds at, so the results agree to one
or two float32 roundings (fused multiply-adds and the division are the only places they can differ).
"""
import ctypes

import numpy as np
import pytest

torch = pytest.importorskip("torch")
from oracle import ops_oracle as ops  # noqa: E402

pytestmark = pytest.mark.gpu

f32 = np.float32


def test_adamw_steps_match_reference_formula(pkg):
    L = pkg.lib()
    rng = np.random.default_rng(3)
    lengths = [768 * 50, 768, 5, 4099, 2304 * 768, 1]
    n = len(lengths)
    host = {k: [rng.standard_normal(l).astype(f32) * s for l in lengths]
            for k, s in (("p", 0.05), ("g", 0.01), ("m", 0.001), ("v", 0.0))}
    host["v"] = [np.abs(rng.standard_normal(l)).astype(f32) * 1e-4 for l in lengths]
    dev = {k: [torch.from_numpy(a.copy()).cuda() for a in host[k]] for k in host}
    # an unaligned tensor takes the scalar path: view into a bigger buffer at +4 bytes
    big = {k: torch.zeros(lengths[3] + 1, device="cuda") for k in host}
    for k in host:
        big[k][1:].copy_(dev[k][3])
        dev[k][3] = big[k][1:]

    def table(k):
        return (ctypes.c_void_p * n)(*[t.data_ptr() for t in dev[k]])

    lens = (ctypes.c_int * n)(*lengths)
    lr, b1, b2, wd, eps = 3e-4, 0.9, 0.999, 0.01, 1e-8
    stream = torch.cuda.current_stream().cuda_stream
    ref = {k: [a.copy() for a in host[k]] for k in host}
    for step in (1, 2, 3):
        assert L.adamw_sm100_step(table("p"), table("g"), table("m"), table("v"), lens, n, lr, b1, b2, wd, eps, step, stream) == 0
        for i in range(n):
            ref["p"][i], ref["m"][i], ref["v"][i] = ops.adamw_step(ref["p"][i], ref["g"][i], ref["m"][i], ref["v"][i],
                                                             lr, b1, b2, wd, eps, step)
        for i in range(n):
            for k in ("p", "m", "v"):
                got = dev[k][i].cpu().numpy().astype(np.float64)
                want = ref[k][i]
                # a few roundings at the magnitude of the operands: the parameter update subtracts a term of
                # size ~lr, so results near zero carry the rounding of that term, not of themselves
                floor = lr if k == "p" else 0.0
                tol = 4 * np.spacing(np.maximum(np.abs(want), floor).astype(f32)).astype(np.float64) + 1e-12
                assert np.all(np.abs(got - want) <= tol), (step, i, k, np.abs(got - want).max())
            # carry the device values forward so that rounding differences do not accumulate in the check
            ref["p"][i], ref["m"][i], ref["v"][i] = (dev[k][i].cpu().numpy().astype(np.float64) for k in ("p", "m", "v"))
            assert torch.equal(dev["g"][i].cpu(), torch.from_numpy(host["g"][i]))  # gradients untouched
    torch.cuda.synchronize()


def test_adamw_argument_errors(pkg):
    L = pkg.lib()
    assert L.adamw_sm100_step(None, None, None, None, None, 1, 1e-3, 0.9, 0.999, 0.0, 1e-8, 1, None) == -1
    t = torch.zeros(4, device="cuda")
    tab = (ctypes.c_void_p * 1)(t.data_ptr())
    lens = (ctypes.c_int * 1)(4)
    assert L.adamw_sm100_step(tab, tab, tab, tab, lens, 0, 1e-3, 0.9, 0.999, 0.0, 1e-8, 1, None) == -2
    assert L.adamw_sm100_step(tab, tab, tab, tab, lens, 1, 1e-3, 0.9, 0.999, 0.0, 1e-8, 0, None) == -2
