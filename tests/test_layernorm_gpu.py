"""Parity of the LayerNorm kernels (include/layernorm_sm100.h) against the float64 numpy restatement of
the reference's CPU LayerNorm (kernels/src/cpu/LayerNorm.c:5-59 forward, :61-123 backward) in
oracle/ops_oracle.py, which tests/test_ops_oracle.py pins to the reference's own kernel: mean and
E[x^2] in one pass, rstd = 1/sqrt(var + eps); dW += sum dy*xhat, db += sum dy, dx += a*dy*w + b*x + c.

Tolerance: everything is fp32 with fp32 accumulation over C (rows) or over the rows (dW, db), so the
results must agree with float64 to a few fp32 ulps of the summed magnitudes: 2e-5 relative to the
largest value for y and dx, 1e-4 for the column sums over thousands of rows (atomics, any order).
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
from oracle import ops_oracle as ops  # noqa: E402

pytestmark = pytest.mark.gpu

SHAPES = [(8 * 128, 768), (1000, 768), (333, 1024), (64, 1600), (17, 64), (256, 2048), (5, 4)]


@pytest.mark.parametrize("rows,C", SHAPES)
@pytest.mark.parametrize("with_bias", [True, False])
def test_layernorm_forward_and_backward_vs_cpu(pkg, rows, C, with_bias):
    rng = np.random.default_rng(rows * 7 + C)
    x = (rng.standard_normal((rows, C)) * 1.7 + 0.3).astype(np.float32)
    w = (1.0 + 0.1 * rng.standard_normal(C)).astype(np.float32)
    b = (0.1 * rng.standard_normal(C)).astype(np.float32) if with_bias else None
    dy = rng.standard_normal((rows, C)).astype(np.float32)
    eps = 1e-5
    xt, wt, dyt = (torch.from_numpy(a).cuda() for a in (x, w, dy))
    bt = torch.from_numpy(b).cuda() if with_bias else None

    y, mean, rstd = pkg.layernorm_forward(xt, wt, bt, eps)
    y_ref, m_ref, r_ref = ops.layernorm_forward(x, w, b, eps)
    assert np.abs(y.cpu().numpy() - y_ref).max() <= 2e-5 * max(1.0, np.abs(y_ref).max())
    assert np.abs(mean.cpu().numpy() - m_ref).max() <= 1e-5
    assert np.abs(rstd.cpu().numpy() / r_ref - 1.0).max() <= 1e-5

    # backward accumulates on top of what the buffers hold
    dw0 = rng.standard_normal(C).astype(np.float32)
    db0 = rng.standard_normal(C).astype(np.float32)
    dx0 = rng.standard_normal((rows, C)).astype(np.float32)
    dw, db, dx = (torch.from_numpy(a.copy()).cuda() for a in (dw0, db0, dx0))
    pkg.layernorm_backward(dyt, xt, mean, rstd, wt, dw, db if with_bias else None, dx)
    dw_ref, db_ref, dx_ref = ops.layernorm_backward(dy, x, mean.cpu().numpy(), rstd.cpu().numpy(), w)
    scale_cols = max(1.0, np.abs(dw_ref).max(), np.abs(db_ref).max())
    assert np.abs(dw.cpu().numpy() - (dw0 + dw_ref)).max() <= 1e-4 * scale_cols
    if with_bias:
        assert np.abs(db.cpu().numpy() - (db0 + db_ref)).max() <= 1e-4 * scale_cols
    else:
        assert np.array_equal(db.cpu().numpy(), db0)  # untouched
    assert np.abs(dx.cpu().numpy() - (dx0 + dx_ref)).max() <= 2e-5 * max(1.0, np.abs(dx_ref).max())


def test_layernorm_argument_errors(pkg):
    L = pkg.lib()
    t = torch.zeros(64, device="cuda")
    p = t.data_ptr()
    assert L.layernorm_sm100_forward(None, p, None, 1e-5, p, p, p, 1, 4, None) == -1
    assert L.layernorm_sm100_forward(p, p, None, 1e-5, p, p, p, 0, 4, None) == -2
    assert L.layernorm_sm100_forward(p, p, None, 1e-5, p, p, p, 1, 6, None) == -3
    assert L.layernorm_sm100_forward(p, p, None, 1e-5, p, p, p, 1, 4096, None) == -3
    assert L.layernorm_sm100_backward(p, p, p, p, p, None, None, p, 1, 4, None) == -1
