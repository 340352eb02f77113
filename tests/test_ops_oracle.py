"""Pins of the numpy restatements in oracle/ops_oracle.py (Linear, LayerNorm, cross-entropy, AdamW, GELU):
against fixtures the reference's own CPU kernels produced (tests/golden/ops_cases.npz, made by
tests/golden/make_golden.py) and, when oracle/_ref/libref_ops.so exists, against those kernels run live on
fresh seeded inputs.  The GPU parity tests of those kernels check the CUDA code against the same
restatements, so this file is what ties them to the reference.

Tolerances: the reference kernels are float32 (OpenBLAS SGEMM, expf/tanhf, float32 accumulation over up to
~100 terms); the restatements are float64.  5e-6 relative to the largest magnitude covers that everywhere;
the AdamW restatement rounds like the kernel and is held to 2 float32 ulps.
"""
import os

import numpy as np
import pytest

from oracle import ops_oracle as ops

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "ops_cases.npz")


def close(got, want, rel=5e-6):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    assert got.shape == want.shape
    lim = rel * max(1.0, np.abs(want).max())
    assert np.abs(got - want).max() <= lim, (np.abs(got - want).max(), lim)


def check_all(d, ref_out):
    """d: inputs; ref_out: the reference kernels' results for them (fixture or live)."""
    close(ops.linear_forward(d["lin_x"], d["lin_w"], d["lin_b"]), ref_out["lin_y"])
    dx, dw, db = ops.linear_backward(d["lin_dy"], d["lin_x"], d["lin_w"], d["lin_dw0"], d["lin_db0"])
    close(dx, ref_out["lin_dx"]), close(dw, ref_out["lin_dw"]), close(db, ref_out["lin_db"])

    y, mean, rstd = ops.layernorm_forward(d["ln_x"], d["ln_w"], d["ln_b"], 1e-5)
    close(y, ref_out["ln_y"]), close(mean, ref_out["ln_mean"]), close(rstd, ref_out["ln_rstd"])
    dw, db, dx = ops.layernorm_backward(d["ln_dy"], d["ln_x"], ref_out["ln_mean"], ref_out["ln_rstd"], d["ln_w"])
    close(d["ln_dw0"] + dw, ref_out["ln_dw"], 2e-5), close(d["ln_db0"] + db, ref_out["ln_db"], 2e-5)
    close(d["ln_dx0"] + dx, ref_out["ln_dx"], 2e-5)

    logsm, loss = ops.xent_forward(d["ce_logits"], d["ce_targets"])
    close(logsm, ref_out["ce_logsm"]), close(loss, ref_out["ce_loss"])
    close(ops.xent_backward(d["ce_g"], d["ce_targets"], ref_out["ce_logsm"]), ref_out["ce_dout_zero"])
    close(ops.xent_backward(d["ce_g"], d["ce_targets"], ref_out["ce_logsm"], d["ce_d0"]), ref_out["ce_dout_d0"])

    p, m, v = d["ad_p"], d["ad_m"], d["ad_v"]
    for step in (1, 2, 3):
        p, m, v = ops.adamw_step(p, d["ad_g"], m, v, 3e-4, 0.9, 0.999, 0.01, 1e-8, step)
    for got, want, floor in ((p, ref_out["ad_p3"], 3e-4), (m, ref_out["ad_m3"], 0.0), (v, ref_out["ad_v3"], 0.0)):
        want = np.asarray(want, np.float64)
        tol = 4 * np.spacing(np.maximum(np.abs(want), floor).astype(np.float32)).astype(np.float64) + 1e-12
        assert np.all(np.abs(got - want) <= tol), np.abs(got - want).max()

    close(ops.gelu_forward(d["ge_x"]), ref_out["ge_y"])
    close(ops.gelu_backward(d["ge_g"], d["ge_x"]), ref_out["ge_dx"])


def test_restatements_match_reference_fixtures():
    z = dict(np.load(GOLDEN))
    check_all(z, z)


def test_restatements_match_reference_kernels_live():
    from oracle import oracle

    if not oracle.have_reference_ops():
        pytest.skip("oracle/_ref/libref_ops.so not built (reference tree absent)")
    ref = oracle.reference_ops()
    rng = np.random.default_rng(8)
    M, N, K, rows, C, V = 64, 96, 32, 50, 64, 257
    d = {
        "lin_x": rng.standard_normal((M, K), dtype=np.float32), "lin_w": (rng.standard_normal((N, K), dtype=np.float32) * 0.1).astype(np.float32),
        "lin_b": rng.standard_normal(N, dtype=np.float32), "lin_dy": rng.standard_normal((M, N), dtype=np.float32),
        "lin_dw0": rng.standard_normal((N, K), dtype=np.float32), "lin_db0": rng.standard_normal(N, dtype=np.float32),
        "ln_x": (rng.standard_normal((rows, C)) * 1.7 + 0.3).astype(np.float32), "ln_w": (1.0 + 0.1 * rng.standard_normal(C)).astype(np.float32),
        "ln_b": (0.1 * rng.standard_normal(C)).astype(np.float32), "ln_dy": rng.standard_normal((rows, C)).astype(np.float32),
        "ln_dw0": rng.standard_normal(C).astype(np.float32), "ln_db0": rng.standard_normal(C).astype(np.float32),
        "ln_dx0": rng.standard_normal((rows, C)).astype(np.float32),
        "ce_logits": (rng.standard_normal((rows, V)) * 3.0).astype(np.float32), "ce_targets": rng.integers(0, V, size=rows).astype(np.float32),
        "ce_g": rng.standard_normal(rows).astype(np.float32), "ce_d0": (rng.standard_normal((rows, V)) * 0.01).astype(np.float32),
        "ad_p": (rng.standard_normal(500) * 0.05).astype(np.float32), "ad_g": (rng.standard_normal(500) * 0.01).astype(np.float32),
        "ad_m": (rng.standard_normal(500) * 0.001).astype(np.float32), "ad_v": (np.abs(rng.standard_normal(500)) * 1e-4).astype(np.float32),
        "ge_x": (rng.standard_normal(300) * 2.5).astype(np.float32), "ge_g": rng.standard_normal(300).astype(np.float32),
    }
    out = {}
    out["lin_y"] = ref.linear_forward(d["lin_x"], d["lin_w"], d["lin_b"])
    out["lin_dx"], out["lin_dw"], out["lin_db"] = ref.linear_backward(d["lin_dy"], d["lin_x"], d["lin_w"], d["lin_dw0"], d["lin_db0"])
    out["ln_y"], out["ln_mean"], out["ln_rstd"] = ref.layernorm_forward(d["ln_x"], d["ln_w"], d["ln_b"], 1e-5)
    out["ln_dw"], out["ln_db"], out["ln_dx"] = ref.layernorm_backward(d["ln_dy"], d["ln_x"], out["ln_mean"], out["ln_rstd"], d["ln_w"],
                                                                    d["ln_dw0"], d["ln_db0"], d["ln_dx0"])
    out["ce_logsm"], out["ce_loss"] = ref.xent_forward(d["ce_logits"], d["ce_targets"])
    out["ce_dout_zero"] = ref.xent_backward(d["ce_g"], d["ce_targets"], out["ce_logsm"], np.zeros_like(d["ce_d0"]))
    out["ce_dout_d0"] = ref.xent_backward(d["ce_g"], d["ce_targets"], out["ce_logsm"], d["ce_d0"])
    p, m, v = d["ad_p"], d["ad_m"], d["ad_v"]
    for step in (1, 2, 3):
        p, m, v = ref.adamw_step(p, d["ad_g"], m, v, 3e-4, 0.9, 0.999, 0.01, 1e-8, step)
    out["ad_p3"], out["ad_m3"], out["ad_v3"] = p, m, v
    out["ge_y"], out["ge_dx"] = ref.gelu_forward(d["ge_x"]), ref.gelu_backward(d["ge_g"], d["ge_x"])
    check_all(d, out)
