"""The Attention layer of gpt.c (include/attention.h API) driven through libgpt.so builds made from
the reference sources with this repository's overlay.  The builds live in oracle/_ref/ (made by
gpt.c_b200/overlay/build_libgpt.py where the reference tree is available); tests skip when absent.
"""
import os
import subprocess

import numpy as np
import pytest

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
OVERLAY = os.path.join(ROOT, "oracle", "_ref", "gptc_overlay", "layer_driver")
REFERENCE = os.path.join(ROOT, "oracle", "_ref", "gptc_reference", "layer_driver")


def run_driver(exe, device, x, g, H, tmp_path, repeat=1):
    B, T, C3 = x.shape
    C = C3 // 3
    paths = [str(tmp_path / n) for n in ("x.bin", "g.bin", "o.bin", "dx.bin")]
    x.tofile(paths[0])
    g.tofile(paths[1])
    res = subprocess.run([exe, device, str(B), str(T), str(C), str(H), *paths, str(repeat)], capture_output=True,
                         text=True, timeout=600)
    assert res.returncode == 0, res.stdout + res.stderr
    out = np.fromfile(paths[2], dtype=np.float32).reshape(B, T, C)
    dx = np.fromfile(paths[3], dtype=np.float32).reshape(B, T, C3)
    return out, dx, res.stdout


def seeded(seed, B, T, H, D):
    rng = np.random.default_rng(seed)
    return (rng.standard_normal((B, T, 3 * H * D), dtype=np.float32),
            rng.standard_normal((B, T, H * D), dtype=np.float32))


@pytest.mark.skipif(not os.path.exists(OVERLAY), reason="overlay build of libgpt.so not present")
def test_layer_cpu_device_keeps_reference_path(oracle, tmp_path):
    """On a CPU device the overlay layer runs the reference's own CPU kernel."""
    x, g = seeded(41, 2, 40, 2, 8)
    out, dx, _ = run_driver(OVERLAY, "cpu", x, g, 2, tmp_path)
    assert np.abs(out - oracle.forward(x, 2)).max() < 2e-5
    assert np.abs(dx - oracle.backward(x, g, 2)).max() < 2e-5


@pytest.mark.gpu
@pytest.mark.skipif(not os.path.exists(OVERLAY), reason="overlay build of libgpt.so not present")
@pytest.mark.parametrize("shape", [(2, 200, 3, 64), (8, 128, 12, 64), (4, 2, 2, 3), (1, 1024, 2, 64)])
def test_layer_cuda_device_matches_oracle(oracle, tmp_path, shape):
    """Attention()->to(CUDA)->forward->backward through the unchanged gpt.c tensor/runtime code."""
    B, T, H, D = shape
    x, g = seeded(42, B, T, H, D)
    out, dx, _ = run_driver(OVERLAY, "cuda", x, g, H, tmp_path)
    assert np.abs(out - oracle.forward(x, H)).max() < 2e-3
    assert np.abs(dx - oracle.backward(x, g, H)).max() < 5e-3


@pytest.mark.gpu
@pytest.mark.skipif(not (os.path.exists(OVERLAY) and os.path.exists(REFERENCE)), reason="libgpt.so builds not present")
def test_layer_forward_agrees_with_reference_cuda(tmp_path):
    """Forward of the reference's own CUDA attention (cuBLAS TF32) vs the overlay; the reference's
    CUDA backward reads an uninitialised buffer and is not compared."""
    x, g = seeded(43, 2, 256, 4, 64)
    o_new, _, _ = run_driver(OVERLAY, "cuda", x, g, 4, tmp_path)
    o_ref, _, _ = run_driver(REFERENCE, "cuda", x, g, 4, tmp_path)
    assert np.abs(o_new - o_ref).max() < 2e-2  # TF32 operands on the reference side
