"""Float64 numpy restatements of the reference's CPU kernels either side of the attention layer.
TEST INFRASTRUCTURE ONLY: the GPU parity tests and the CPU pinning tests import this one copy.

Each function follows one kernel of gpt.c, with its buffer semantics (what is overwritten, what is
accumulated on top of the caller's contents):

  linear_forward / linear_backward        kernels/src/cpu/Linear.c:4-31, :33-88
  layernorm_forward / layernorm_backward  kernels/src/cpu/LayerNorm.c:5-59, :61-123
  xent_forward / xent_backward            kernels/src/cpu/CrossEntropyLoss.c:7-51, :53-97
  adamw_step                              kernels/src/cpu/AdamW.c:5-50
  gelu_forward / gelu_backward            kernels/src/cpu/GeLU.c:7-18, :20-42

`tests/test_ops_oracle.py` holds them to the reference's own kernels compiled out of tree
(oracle/_ref/libref_ops.so, live when the reference tree was present at build time) and to fixtures
those kernels produced (tests/golden/ops_*.npz, made by tests/golden/make_golden.py).
"""
from __future__ import annotations

import numpy as np

f32 = np.float32
f64 = np.float64


def linear_forward(x, w, b=None):
    """y[M, N] = x[M, K] . w[N, K]^T (+ b): one SGEMM and a bias loop (Linear.c:15-30)."""
    y = x.astype(f64) @ w.astype(f64).T
    return y + b.astype(f64) if b is not None else y


def linear_backward(dy, x, w, dw0=None, db0=None):
    """dx = dy . w (overwritten, beta = 0), dW += dy^T . x, db += column sums of dy (Linear.c:54-87)."""
    dy64 = dy.astype(f64)
    dx = dy64 @ w.astype(f64)
    dw = dy64.T @ x.astype(f64) + (0.0 if dw0 is None else dw0.astype(f64))
    db = dy64.sum(axis=0) + (0.0 if db0 is None else db0.astype(f64))
    return dx, dw, db


def layernorm_forward(x, w, b, eps):
    """mean and E[x^2] in one pass, rstd = 1/sqrt(var + eps), y = (x - mean) * rstd * w (+ b)
    (LayerNorm.c:30-57).  Returns y, mean [rows], rstd [rows]."""
    x = x.astype(f64)
    m = x.mean(axis=1, keepdims=True)
    var = (x * x).mean(axis=1, keepdims=True) - m * m
    r = 1.0 / np.sqrt(var + eps)
    y = (x - m) * r * w
    if b is not None:
        y = y + b
    return y, m[:, 0], r[:, 0]


def layernorm_backward(dy, x, mean, rstd, w):
    """The increments the kernel ADDS to dW, db and dx (LayerNorm.c:92-121):
    dW += sum dy * (a x - a mu), db += sum dy, dx += a dy w + b x + c with
    b = (dbs mu - ds) a^3 / C, c = -b mu - dbs a / C."""
    dy, x, w = dy.astype(f64), x.astype(f64), w.astype(f64)
    a = rstd[:, None].astype(f64)
    mu = mean[:, None].astype(f64)
    C = x.shape[1]
    dw = (dy * (a * x - a * mu)).sum(axis=0)
    db = dy.sum(axis=0)
    ds = (dy * x * w).sum(axis=1, keepdims=True)
    dbs = (dy * w).sum(axis=1, keepdims=True)
    bb = (dbs * mu - ds) * a ** 3 / C
    cc = -bb * mu - dbs * a / C
    dx = a * dy * w + bb * x + cc
    return dw, db, dx


def xent_forward(logits, targets):
    """log-softmax [rows, C] (kept for backward) and the mean negative log-likelihood
    (CrossEntropyLoss.c:24-50).  targets are class indices stored as floats."""
    x = logits.astype(f64)
    m = x.max(axis=1, keepdims=True)
    logsm = x - m - np.log(np.exp(x - m).sum(axis=1, keepdims=True))
    idx = targets.astype(np.int64)
    loss = -logsm[np.arange(x.shape[0]), idx].mean()
    return logsm, loss


def xent_backward(g, targets, logsm, dout0=None):
    """The kernel works on what `dout` already holds (the layer passes zeros): the target entry of every
    row is SET to -g / rows, then every row becomes cur - exp(logsm) * sum(cur) (CrossEntropyLoss.c:72-96)."""
    rows, C = logsm.shape
    cur = np.zeros((rows, C), f64) if dout0 is None else dout0.astype(f64).copy()
    idx = targets.astype(np.int64)
    cur[np.arange(rows), idx] = -g.astype(f64) / rows
    return cur - np.exp(logsm.astype(f64)) * cur.sum(axis=1, keepdims=True)


def adamw_step(p, g, m, v, lr, b1, b2, wd, eps, step):
    """One AdamW step in float64 with a rounding to float32 wherever the float32 kernel rounds
    (AdamW.c:36-47: decoupled weight decay, moments by lerp(a, b, w) = fma(w, b, fma(-w, a, a)), bias
    corrections 1 - beta^step).  Hyper-parameters are taken as float32, as the kernel receives them.
    The kernel divides by the corrections; multiplying by their float32 reciprocals, as the CUDA build
    does, differs by one rounding."""
    p, g, m, v = (a.astype(f64) for a in (p, g, m, v))
    lr, b1, b2, wd, eps = (f64(f32(a)) for a in (lr, b1, b2, wd, eps))
    r = lambda a: a.astype(f32).astype(f64)  # noqa: E731
    p = r(p - r(r(f32(lr) * f32(wd)) * p))
    m = r(b1 * m + r(-b1 * g + g))
    gg = r(g * g)
    v = r(b2 * v + r(-b2 * gg + gg))
    c1 = f64(f32(1.0) / (f32(1.0) - f32(np.power(f32(b1), f32(step)))))
    c2 = f64(f32(1.0) / (f32(1.0) - f32(np.power(f32(b2), f32(step)))))
    mh, vh = r(m * c1), r(v * c2)
    p = r(p - r(r(lr * mh) / r(r(np.sqrt(vh)) + eps)))
    return p, m, v


def gelu_forward(x):
    """0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))) (GeLU.c:10-17)."""
    x = x.astype(f64)
    kb = np.sqrt(2.0 / np.pi)
    return 0.5 * x * (1.0 + np.tanh(kb * (x + 0.044715 * x ** 3)))


def gelu_backward(g, x):
    """g * d/dx of the above (GeLU.c:26-41)."""
    x, g = x.astype(f64), g.astype(f64)
    kb = np.sqrt(2.0 / np.pi)
    t = np.tanh(kb * (x + 0.044715 * x ** 3))
    return g * (0.5 * (1.0 + t) + 0.5 * x * (1.0 - t * t) * kb * (1.0 + 3.0 * 0.044715 * x ** 2))
