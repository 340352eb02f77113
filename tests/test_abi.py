"""CPU tests of the C-ABI boundary: the library loads, exports every declared symbol, and rejects
bad arguments before touching the GPU."""
import ctypes
import os
import re

import pytest

INCLUDE = os.path.join(os.path.dirname(__file__), "..", "include")
HEADERS = ["attn_sm100.h", "linear_sm100.h", "layernorm_sm100.h", "tensor_sm100.h", "xent_sm100.h", "adamw_sm100.h"]


def declared_functions():
    names = set()
    for header in HEADERS:
        text = open(os.path.join(INCLUDE, header)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names |= set(re.findall(r"\b((?:attn|linear|layernorm|tensor|xent|adamw)_sm100_\w+)\s*\(", text))
    return sorted(names)


def test_header_declares_something():
    names = declared_functions()
    assert "attn_sm100_forward" in names and "attn_sm100_backward" in names


def test_library_exports_every_declared_symbol(pkg):
    handle = pkg.lib()
    for name in declared_functions():
        assert hasattr(handle, name), f"{name} declared under include/ but not exported"
    assert set(pkg.SIGNATURES) == set(declared_functions())


def test_version_and_strerror(pkg):
    L = pkg.lib()
    assert L.attn_sm100_version() >= 100
    assert L.attn_sm100_strerror(0) == b"success"
    for code in (-1, -2, -3, -4, -5, -6):
        assert len(L.attn_sm100_strerror(code)) > 8
    assert L.attn_sm100_strerror(-99) == b"unknown error"


def test_size_queries(pkg):
    # two bf16 planes of B*T*3C elements, each padded to 256 bytes
    assert pkg.saved_bytes(8, 1024, 12, 64) == 2 * 8 * 1024 * 3 * 768 * 2
    assert pkg.saved_bytes(1, 1, 1, 3) == 2 * 256
    # dO planes, delta, and 256 bytes for the backward kernel's item counter
    assert pkg.backward_scratch_bytes(8, 1024, 12, 64) == 2 * 8 * 1024 * 768 * 2 + 8 * 12 * 1024 * 4 + 256
    for bad in [(0, 1, 1, 1), (1, -1, 1, 1), (1, 1, 0, 1), (1, 1, 1, 0), (4096, 4096, 64, 64)]:
        assert pkg.saved_bytes(*bad) == 0
        assert pkg.backward_scratch_bytes(*bad) == 0


def test_argument_errors_are_reported_before_any_cuda_call(pkg):
    L = pkg.lib()
    one = ctypes.c_void_p(16)
    # NULL pointers
    assert L.attn_sm100_forward(None, one, None, one, one, 1, 1, 1, 64, 0, None) == -1
    assert L.attn_sm100_backward(one, one, one, None, one, one, 1, 1, 1, 64, 0, None) == -1
    # shapes
    assert L.attn_sm100_forward(one, one, None, one, one, 0, 1, 1, 64, 0, None) == -2
    assert L.attn_sm100_backward(one, one, one, one, one, one, 1, 1, 1, -3, 0, None) == -2
    # alignment
    odd = ctypes.c_void_p(20)
    assert L.attn_sm100_forward(odd, one, None, one, one, 1, 1, 1, 64, 0, None) == -4
    # shapes no kernel takes
    assert L.attn_sm100_forward(one, one, None, one, one, 1, 1, 1, 300, 0, None) == -3
    assert L.attn_sm100_forward(one, one, None, one, one, 1, 9000, 1, 32, 0, None) == -3
    assert L.attn_sm100_device_status(None, 0) == -1


def test_missing_library_raises(pkg, monkeypatch):
    monkeypatch.setattr(pkg, "_lib", None)
    monkeypatch.setattr(pkg, "LIB_PATH", "/nonexistent/libattn_sm100.so")
    with pytest.raises(FileNotFoundError):
        pkg.lib()


def test_no_cpu_fallback_without_gpu(pkg):
    """Without a CUDA device init must fail loudly instead of computing anything on the host."""
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    assert pkg.lib().attn_sm100_init() != 0
    with pytest.raises(pkg.AttnError):
        pkg.init()
