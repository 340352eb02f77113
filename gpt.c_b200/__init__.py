"""B200-native causal self-attention for gpt.c: ctypes access to ``libattn_sm100.so``.

The product is the C-ABI library declared in ``include/attn_sm100.h`` (hand-written sm_100a CUDA).
This package only loads it and offers a thin convenience layer that takes ``torch`` CUDA tensors
for device memory and streams; every call goes through the C ABI with raw pointers.  There is no
CPU or PyTorch fallback: if the library is missing or the device is not an sm_100 GPU the calls
raise.

The directory name contains a dot, so it cannot be imported with a plain ``import`` statement;
load it with ``importlib`` (see ``load_package`` in ``__graft_entry__.py``) under the module name
``gptc_b200``.
"""
from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "lib", "libattn_sm100.so")
HEADER_PATH = os.path.join(HERE, "..", "include", "attn_sm100.h")

FLAG_FORCE_GENERIC = 1
FLAG_PREPARE_ONLY = 2
FLAG_CORE_ONLY = 4

# name -> (restype, argtypes); must list every function include/attn_sm100.h declares
_c = ctypes
SIGNATURES = {
    "attn_sm100_version": (_c.c_int, []),
    "attn_sm100_init": (_c.c_int, []),
    "attn_sm100_saved_bytes": (_c.c_size_t, [_c.c_int] * 4),
    "attn_sm100_backward_scratch_bytes": (_c.c_size_t, [_c.c_int] * 4),
    "attn_sm100_forward": (_c.c_int, [_c.c_void_p] * 5 + [_c.c_int] * 5 + [_c.c_void_p]),
    "attn_sm100_backward": (_c.c_int, [_c.c_void_p] * 6 + [_c.c_int] * 5 + [_c.c_void_p]),
    "attn_sm100_forward_static": (_c.c_int, [_c.c_void_p] * 3 + [_c.c_int] * 4 + [_c.c_void_p]),
    "attn_sm100_static_status": (_c.c_int, [_c.POINTER(_c.c_int), _c.c_int]),
    "attn_sm100_selftest_wait_limit": (_c.c_int, [_c.c_uint, _c.c_void_p]),
    "attn_sm100_device_status": (_c.c_int, [_c.POINTER(_c.c_int), _c.c_int]),
    "attn_sm100_strerror": (_c.c_char_p, [_c.c_int]),
    "linear_sm100_forward": (_c.c_int, [_c.c_void_p] * 5 + [_c.c_int] * 3 + [_c.c_void_p]),
    "linear_sm100_backward_scratch_bytes": (_c.c_size_t, [_c.c_int] * 3),
    "linear_sm100_backward": (_c.c_int, [_c.c_void_p] * 7 + [_c.c_int] * 3 + [_c.c_void_p]),
    "layernorm_sm100_forward": (_c.c_int, [_c.c_void_p] * 3 + [_c.c_float] + [_c.c_void_p] * 3 + [_c.c_int] * 2 + [_c.c_void_p]),
    "layernorm_sm100_backward": (_c.c_int, [_c.c_void_p] * 8 + [_c.c_int] * 2 + [_c.c_void_p]),
    "tensor_sm100_fill": (_c.c_int, [_c.c_void_p, _c.c_size_t, _c.c_float, _c.c_void_p]),
    "tensor_sm100_arange": (_c.c_int, [_c.c_void_p, _c.c_size_t, _c.c_int, _c.c_int, _c.c_void_p]),
    "tensor_sm100_copy": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_size_t, _c.c_void_p]),
    "tensor_sm100_axpy": (_c.c_int, [_c.c_size_t, _c.c_float, _c.c_void_p, _c.c_void_p, _c.c_void_p]),
    "tensor_sm100_gelu_forward": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_size_t, _c.c_void_p]),
    "tensor_sm100_gelu_backward": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_size_t, _c.c_void_p]),
    "xent_sm100_forward": (_c.c_int, [_c.c_void_p] * 4 + [_c.c_int] * 2 + [_c.c_void_p]),
    "xent_sm100_backward": (_c.c_int, [_c.c_void_p] * 4 + [_c.c_int] * 2 + [_c.c_void_p]),
    "adamw_sm100_step": (_c.c_int, [_c.c_void_p] * 5 + [_c.c_int] + [_c.c_float] * 5 + [_c.c_int, _c.c_void_p]),
}

_lib = None


class AttnError(RuntimeError):
    def __init__(self, code: int, where: str):
        self.code = code
        msg = lib().attn_sm100_strerror(code).decode()
        super().__init__(f"{where} failed with status {code}: {msg}")


def lib() -> ctypes.CDLL:
    """Load libattn_sm100.so (once).  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FileNotFoundError(
                f"{LIB_PATH} is missing: build it with `python gpt.c_b200/build.py`; there is no fallback path")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def _check(code: int, where: str) -> None:
    if code != 0:
        raise AttnError(code, where)


def _ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def init() -> None:
    _check(lib().attn_sm100_init(), "attn_sm100_init")


def device_status(clear: bool = True) -> int:
    """Synchronise the current device and return its kernel status word (0 = fine)."""
    st = ctypes.c_int(0)
    rc = lib().attn_sm100_device_status(ctypes.byref(st), 1 if clear else 0)
    if rc not in (0, -6):
        raise AttnError(rc, "attn_sm100_device_status")
    return st.value


def static_status(clear: bool = True) -> int:
    """The same for the status word of attn_sm100_forward_static (a separate word inside the library)."""
    st = ctypes.c_int(0)
    rc = lib().attn_sm100_static_status(ctypes.byref(st), 1 if clear else 0)
    if rc not in (0, -6):
        raise AttnError(rc, "attn_sm100_static_status")
    return st.value


def saved_bytes(B: int, T: int, H: int, D: int) -> int:
    return lib().attn_sm100_saved_bytes(B, T, H, D)


def backward_scratch_bytes(B: int, T: int, H: int, D: int) -> int:
    return lib().attn_sm100_backward_scratch_bytes(B, T, H, D)


class Saved:
    """What forward leaves behind for backward (all device buffers, owned by torch)."""

    def __init__(self, saved, out, lse, shape, flags):
        self.saved, self.out, self.lse, self.shape, self.flags = saved, out, lse, shape, flags


def forward_into(qkv, out, out_copy, lse, saved, n_heads: int, flags: int = 0, stream=None) -> None:
    """Raw call: every buffer is supplied by the caller (torch CUDA tensors or None)."""
    import torch

    B, T, C3 = qkv.shape
    D = C3 // 3 // n_heads
    s = torch.cuda.current_stream() if stream is None else stream
    _check(lib().attn_sm100_forward(_ptr(qkv), _ptr(out), _ptr(out_copy), _ptr(lse), _ptr(saved), B, T, n_heads, D,
                                    flags, s.cuda_stream), "attn_sm100_forward")


def backward_into(saved, out, lse, dout, dqkv, scratch, n_heads: int, flags: int = 0, stream=None) -> None:
    import torch

    B, T, C = dout.shape
    D = C // n_heads
    s = torch.cuda.current_stream() if stream is None else stream
    _check(lib().attn_sm100_backward(_ptr(saved), _ptr(out), _ptr(lse), _ptr(dout), _ptr(dqkv), _ptr(scratch), B, T,
                                     n_heads, D, flags, s.cuda_stream), "attn_sm100_backward")


def forward(qkv, n_heads: int, flags: int = 0, keep_copy: bool = False):
    """qkv [B, T, 3C] fp32 CUDA tensor -> (out [B, T, C], Saved)."""
    import torch

    if not (qkv.is_cuda and qkv.dtype == torch.float32 and qkv.is_contiguous() and qkv.dim() == 3):
        raise ValueError("qkv must be a contiguous fp32 CUDA tensor of shape [B, T, 3C]")
    B, T, C3 = qkv.shape
    if C3 % (3 * n_heads) != 0:
        raise ValueError("last dimension must be 3 * n_heads * head_size")
    C = C3 // 3
    D = C // n_heads
    out = torch.empty((B, T, C), device=qkv.device, dtype=torch.float32)
    out_copy = torch.empty_like(out) if keep_copy else None
    lse = torch.empty((B, n_heads, T), device=qkv.device, dtype=torch.float32)
    saved = torch.empty(saved_bytes(B, T, n_heads, D), device=qkv.device, dtype=torch.uint8)
    forward_into(qkv, out, out_copy, lse, saved, n_heads, flags)
    return out, Saved(saved, out_copy if keep_copy else out, lse, (B, T, n_heads, D), flags)


def backward(ctx: Saved, dout):
    """dout [B, T, C] -> dqkv [B, T, 3C] = [dq | dk | dv]."""
    import torch

    B, T, H, D = ctx.shape
    if not (dout.is_cuda and dout.dtype == torch.float32 and dout.is_contiguous() and tuple(dout.shape) == (B, T, H * D)):
        raise ValueError("dout must be a contiguous fp32 CUDA tensor of shape [B, T, C]")
    dqkv = torch.empty((B, T, 3 * H * D), device=dout.device, dtype=torch.float32)
    scratch = torch.empty(backward_scratch_bytes(B, T, H, D), device=dout.device, dtype=torch.uint8)
    backward_into(ctx.saved, ctx.out, ctx.lse, dout, dqkv, scratch, H, ctx.flags)
    return dqkv


# ---------------------------------------------------------------------------------------------
# Linear either side of the attention layer (include/linear_sm100.h); mirrors the reference's
# linear_forward_cuda_kernel / linear_backward_cuda_kernel (kernels/src/cuda/Linear.cu:37-92).
# ---------------------------------------------------------------------------------------------
def linear_forward(x, w, bias=None, planes=None, stream=None):
    """y[..., N] = x[..., K] @ w[N, K].T + bias.  `planes`: optional uint8 CUDA tensor of
    saved_bytes(...) bytes that receives y as bf16 hi/lo planes for the attention kernels."""
    import torch

    K = x.shape[-1]
    N = w.shape[0]
    M = x.numel() // K
    y = torch.empty((*x.shape[:-1], N), device=x.device, dtype=torch.float32)
    s = torch.cuda.current_stream() if stream is None else stream
    _check(lib().linear_sm100_forward(_ptr(x), _ptr(w), _ptr(bias), _ptr(y), _ptr(planes), M, N, K, s.cuda_stream),
           "linear_sm100_forward")
    return y


def linear_backward(dy, x, w, dw, db=None, stream=None, want_dx=True):
    """Returns dx = dy @ w (None when want_dx is false); accumulates dy.T @ x into dw (skipped when dw is
    None) and the column sums of dy into db."""
    import torch

    K = x.shape[-1]
    N = w.shape[0]
    M = x.numel() // K
    dx = torch.empty_like(x) if want_dx else None
    s = torch.cuda.current_stream() if stream is None else stream
    nbytes = lib().linear_sm100_backward_scratch_bytes(M, N, K)
    scratch = torch.empty(nbytes, device=x.device, dtype=torch.uint8) if nbytes else None
    _check(lib().linear_sm100_backward(_ptr(dy), _ptr(x), _ptr(w), _ptr(dx), _ptr(dw), _ptr(db), _ptr(scratch), M, N, K,
                                       s.cuda_stream), "linear_sm100_backward")
    return dx


# ---------------------------------------------------------------------------------------------
# LayerNorm (include/layernorm_sm100.h); mirrors layer_norm_{forward,backward}_cuda_kernel
# (kernels/src/cuda/LayerNorm.cu:115-165).
# ---------------------------------------------------------------------------------------------
def layernorm_forward(x, w, b=None, eps: float = 1e-5, stream=None):
    """Returns (y, mean, rstd) for x [..., C]."""
    import torch

    C = x.shape[-1]
    rows = x.numel() // C
    y = torch.empty_like(x)
    mean = torch.empty(rows, device=x.device, dtype=torch.float32)
    rstd = torch.empty(rows, device=x.device, dtype=torch.float32)
    s = torch.cuda.current_stream() if stream is None else stream
    _check(lib().layernorm_sm100_forward(_ptr(x), _ptr(w), _ptr(b), eps, _ptr(mean), _ptr(rstd), _ptr(y), rows, C,
                                         s.cuda_stream), "layernorm_sm100_forward")
    return y, mean, rstd


def layernorm_backward(dy, x, mean, rstd, w, dw, db, dx, stream=None) -> None:
    """Accumulates into dw, db (may be None) and dx, like the reference."""
    import torch

    C = x.shape[-1]
    rows = x.numel() // C
    s = torch.cuda.current_stream() if stream is None else stream
    _check(lib().layernorm_sm100_backward(_ptr(dy), _ptr(x), _ptr(mean), _ptr(rstd), _ptr(w), _ptr(dw), _ptr(db), _ptr(dx),
                                          rows, C, s.cuda_stream), "layernorm_sm100_backward")
