"""ctypes front end of the CPU checkers.  TEST INFRASTRUCTURE ONLY.

``forward`` / ``backward`` call the plain-C restatement (``oracle/attention_oracle.c``);
``reference_run`` calls the reference's own CPU kernel compiled out of tree
(``oracle/_ref/libref_attention.so``) when that library exists.  Only the test-suite, the smoke
check and the CPU-baseline legs of the benchmark may import this module; the product path never
does.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "liboracle.so")
REF_SO = os.path.join(HERE, "_ref", "libref_attention.so")

_f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_oracle = None
_ref = None


def _load_oracle():
    global _oracle
    if _oracle is None:
        if not os.path.exists(ORACLE_SO):
            from . import build as _b  # type: ignore

            _b.build_oracle()
        lib = ctypes.CDLL(ORACLE_SO)
        lib.oracle_attention_forward.restype = ctypes.c_int
        lib.oracle_attention_forward.argtypes = [_f32p, _f32p, ctypes.c_void_p] + [ctypes.c_int] * 4
        lib.oracle_attention_backward.restype = ctypes.c_int
        lib.oracle_attention_backward.argtypes = [_f32p, _f32p, _f32p] + [ctypes.c_int] * 4
        lib.oracle_num_threads.restype = ctypes.c_int
        _oracle = lib
    return _oracle


def have_reference() -> bool:
    return os.path.exists(REF_SO)


def _load_ref():
    global _ref
    if _ref is None:
        lib = ctypes.CDLL(REF_SO)
        lib.ref_attention_run.restype = ctypes.c_int
        lib.ref_attention_run.argtypes = [_f32p, ctypes.c_void_p, _f32p, ctypes.c_void_p] + [ctypes.c_int] * 4 + [
            ctypes.POINTER(ctypes.c_double)]
        lib.ref_set_num_threads.argtypes = [ctypes.c_int]
        lib.ref_get_num_threads.restype = ctypes.c_int
        lib.ref_blas_config.restype = ctypes.c_char_p
        _ref = lib
    return _ref


def num_threads() -> int:
    return _load_oracle().oracle_num_threads()


def _dims(x: np.ndarray, n_heads: int):
    B, T, C3 = x.shape
    assert C3 % (3 * n_heads) == 0
    return B, T, n_heads, C3 // 3 // n_heads


def forward(x: np.ndarray, n_heads: int, want_lse: bool = False):
    """x [B,T,3C] float32 -> out [B,T,C] (and lse [B,H,T])."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    B, T, H, D = _dims(x, n_heads)
    out = np.empty((B, T, H * D), dtype=np.float32)
    lse = np.empty((B, H, T), dtype=np.float32) if want_lse else None
    rc = _load_oracle().oracle_attention_forward(x, out, lse.ctypes.data if want_lse else None, B, T, H, D)
    if rc != 0:
        raise RuntimeError(f"oracle_attention_forward returned {rc}")
    return (out, lse) if want_lse else out


def backward(x: np.ndarray, dout: np.ndarray, n_heads: int) -> np.ndarray:
    """x [B,T,3C], dout [B,T,C] -> dx [B,T,3C] = [dq | dk | dv]."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    dout = np.ascontiguousarray(dout, dtype=np.float32)
    B, T, H, D = _dims(x, n_heads)
    assert dout.shape == (B, T, H * D)
    dx = np.empty_like(x)
    rc = _load_oracle().oracle_attention_backward(x, dout, dx, B, T, H, D)
    if rc != 0:
        raise RuntimeError(f"oracle_attention_backward returned {rc}")
    return dx


def reference_run(x: np.ndarray, dout: np.ndarray | None, n_heads: int, threads: int | None = None):
    """Run the reference's own CPU kernel.  Returns (out, dx or None, (fwd_s, bwd_s))."""
    lib = _load_ref()
    if threads is not None:
        lib.ref_set_num_threads(int(threads))
    x = np.ascontiguousarray(x, dtype=np.float32)
    B, T, H, D = _dims(x, n_heads)
    out = np.empty((B, T, H * D), dtype=np.float32)
    dx = None
    dptr = None
    dxptr = None
    if dout is not None:
        dout = np.ascontiguousarray(dout, dtype=np.float32)
        dx = np.empty_like(x)
        dptr, dxptr = dout.ctypes.data, dx.ctypes.data
    secs = (ctypes.c_double * 2)(0.0, 0.0)
    rc = lib.ref_attention_run(x, dptr, out, dxptr, B, T, H, D, secs)
    if rc != 0:
        raise RuntimeError(f"ref_attention_run returned {rc}")
    return out, dx, (secs[0], secs[1])


def reference_info() -> dict:
    lib = _load_ref()
    return {"threads": lib.ref_get_num_threads(), "blas": lib.ref_blas_config().decode(errors="replace")}


# ---------------------------------------------------------------------------------------------
# the reference's own CPU kernels of Linear, LayerNorm, cross-entropy, AdamW and GELU
# (oracle/_ref/libref_ops.so, compiled out of tree by oracle/build.py with oracle/ref_ops_driver.c)
# ---------------------------------------------------------------------------------------------
REF_OPS_SO = os.path.join(HERE, "_ref", "libref_ops.so")
_ref_ops = None


def have_reference_ops() -> bool:
    return os.path.exists(REF_OPS_SO)


def _c(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


class ReferenceOps:
    """numpy in, numpy out; in/out buffers of the kernels are passed as copies and returned."""

    def __init__(self):
        lib = ctypes.CDLL(REF_OPS_SO)
        for name in ("ref_linear_forward", "ref_linear_backward", "ref_layernorm_forward", "ref_layernorm_backward",
                     "ref_xent_forward", "ref_xent_backward", "ref_adamw_step", "ref_gelu_forward", "ref_gelu_backward"):
            getattr(lib, name).restype = ctypes.c_int
        self.lib = lib

    @staticmethod
    def _ok(rc, what):
        if rc != 0:
            raise RuntimeError(f"{what} returned {rc}")

    def linear_forward(self, x, w, b=None):
        x, w = _c(x), _c(w)
        b = None if b is None else _c(b)
        M, K = x.shape
        N = w.shape[0]
        y = np.empty((M, N), np.float32)
        self._ok(self.lib.ref_linear_forward(_p(x), _p(w), _p(b), _p(y), M, N, K), "ref_linear_forward")
        return y

    def linear_backward(self, dy, x, w, dw0, db0=None):
        dy, x, w = _c(dy), _c(x), _c(w)
        M, N = dy.shape
        K = x.shape[1]
        dx = np.empty((M, K), np.float32)
        dw = _c(dw0).copy()
        db = None if db0 is None else _c(db0).copy()
        self._ok(self.lib.ref_linear_backward(_p(dy), _p(x), _p(w), _p(dx), _p(dw), _p(db), M, N, K), "ref_linear_backward")
        return dx, dw, db

    def layernorm_forward(self, x, w, b, eps):
        x, w = _c(x), _c(w)
        b = None if b is None else _c(b)
        rows, C = x.shape
        y, mean, rstd = np.empty((rows, C), np.float32), np.empty(rows, np.float32), np.empty(rows, np.float32)
        self._ok(self.lib.ref_layernorm_forward(_p(x), _p(w), _p(b), ctypes.c_float(eps), _p(y), _p(mean), _p(rstd), rows, C),
                 "ref_layernorm_forward")
        return y, mean, rstd

    def layernorm_backward(self, dy, x, mean, rstd, w, dw0, db0, dx0):
        dy, x, mean, rstd, w = _c(dy), _c(x), _c(mean), _c(rstd), _c(w)
        rows, C = x.shape
        dw, dx = _c(dw0).copy(), _c(dx0).copy()
        db = None if db0 is None else _c(db0).copy()
        self._ok(self.lib.ref_layernorm_backward(_p(dy), _p(x), _p(mean), _p(rstd), _p(w), _p(dw), _p(db), _p(dx), rows, C),
                 "ref_layernorm_backward")
        return dw, db, dx

    def xent_forward(self, logits, targets):
        logits, targets = _c(logits), _c(targets)
        rows, C = logits.shape
        logsm, loss = np.empty((rows, C), np.float32), np.zeros(1, np.float32)
        self._ok(self.lib.ref_xent_forward(_p(logits), _p(targets), _p(logsm), _p(loss), rows, C), "ref_xent_forward")
        return logsm, float(loss[0])

    def xent_backward(self, g, targets, logsm, dout0):
        g, targets, logsm = _c(g), _c(targets), _c(logsm)
        rows, C = logsm.shape
        dout = _c(dout0).copy()
        self._ok(self.lib.ref_xent_backward(_p(g), _p(targets), _p(logsm), _p(dout), rows, C), "ref_xent_backward")
        return dout

    def adamw_step(self, p, g, m, v, lr, b1, b2, wd, eps, step):
        p, m, v = _c(p).copy(), _c(m).copy(), _c(v).copy()
        g = _c(g)
        f = ctypes.c_float
        self._ok(self.lib.ref_adamw_step(_p(p), _p(g), _p(m), _p(v), p.size, f(lr), f(b1), f(b2), f(wd), f(eps), int(step)),
                 "ref_adamw_step")
        return p, m, v

    def gelu_forward(self, x):
        x = _c(x)
        y = np.empty_like(x)
        self._ok(self.lib.ref_gelu_forward(_p(x), _p(y), x.size), "ref_gelu_forward")
        return y

    def gelu_backward(self, g, x):
        g, x = _c(g), _c(x)
        dx = np.empty_like(x)
        self._ok(self.lib.ref_gelu_backward(_p(g), _p(x), _p(dx), x.size), "ref_gelu_backward")
        return dx


def reference_ops() -> ReferenceOps:
    global _ref_ops
    if _ref_ops is None:
        _ref_ops = ReferenceOps()
    return _ref_ops
