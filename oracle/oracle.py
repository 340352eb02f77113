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
