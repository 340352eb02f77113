"""CPU tests: the plain-C oracle against the committed golden vectors and against the reference's
own compiled CPU kernel when that library is present."""
import glob
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
TOL = 2e-5  # fp32 restatement vs fp32 reference: differences are accumulation-order rounding only


def test_reference_own_test_case(oracle):
    """Inputs of the reference's tests/test_self_attention.py (D=3, H=2, T=2)."""
    z = np.load(os.path.join(GOLDEN, "ref_selfattn_case.npz"))
    H = int(z["n_heads"])
    out = oracle.forward(z["qkv"], H)
    dx = oracle.backward(z["qkv"], z["dout"], H)
    for key_o, key_d in (("out_model_py", "dqkv_model_py"), ("out_cpu_kernel", "dqkv_cpu_kernel")):
        assert np.abs(out - z[key_o]).max() < TOL
        assert np.abs(dx - z[key_d]).max() < TOL


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLDEN, "seeded_*.npz"))), ids=os.path.basename)
def test_seeded_golden(oracle, path):
    z = np.load(path)
    H = int(z["n_heads"])
    out = oracle.forward(z["x"], H)
    dx = oracle.backward(z["x"], z["dout"], H)
    assert np.abs(out - z["out"]).max() < TOL
    assert np.abs(dx - z["dx"]).max() < TOL


def test_config1_digest(oracle):
    """README CPU-training shape (B=8, T=128, H=12, D=64): digest of the reference kernel's output."""
    from tests.golden.make_golden import digest, seeded_inputs

    z = np.load(os.path.join(GOLDEN, "config1_digest.npz"))
    B, T, H, D = (int(v) for v in z["shape"])
    x, dout = seeded_inputs(int(z["seed"]), B, T, H, D)
    if abs(float(x.astype(np.float64).sum()) - float(z["x_sum"])) > 1e-6:
        pytest.skip("numpy generator stream differs from the one the fixture was made with")
    out = oracle.forward(x, H)
    dx = oracle.backward(x, dout, H)
    so, s1, _ = digest(out)
    sx, d1, _ = digest(dx)
    assert np.abs(so - z["out_samples"]).max() < TOL
    assert np.abs(sx - z["dx_samples"]).max() < TOL
    assert abs(s1 - float(z["out_sum"])) < 1e-2 and abs(d1 - float(z["dx_sum"])) < 1e-2


def test_lse_matches_definition(oracle):
    rng = np.random.default_rng(3)
    B, T, H, D = 1, 40, 2, 8
    x = rng.standard_normal((B, T, 3 * H * D), dtype=np.float32)
    _, lse = oracle.forward(x, H, want_lse=True)
    q = x[..., : H * D].reshape(B, T, H, D).transpose(0, 2, 1, 3).astype(np.float64)
    k = x[..., H * D: 2 * H * D].reshape(B, T, H, D).transpose(0, 2, 1, 3).astype(np.float64)
    s = q @ k.transpose(0, 1, 3, 2) / np.sqrt(D)
    s = np.where(np.tril(np.ones((T, T), bool)), s, -np.inf)
    ref = np.log(np.exp(s - s.max(-1, keepdims=True)).sum(-1)) + s.max(-1)
    assert np.abs(lse - ref).max() < 1e-5


def test_causality(oracle):
    """Changing a later token must not change earlier outputs; dx of a masked pair is zero."""
    rng = np.random.default_rng(4)
    B, T, H, D = 1, 17, 2, 4
    x = rng.standard_normal((B, T, 3 * H * D), dtype=np.float32)
    y0 = oracle.forward(x, H)
    x2 = x.copy()
    x2[:, 10:, :] += 1.0
    y1 = oracle.forward(x2, H)
    assert np.array_equal(y0[:, :10], y1[:, :10])


def test_against_reference_kernel_when_present(oracle):
    if not oracle.have_reference():
        pytest.skip("oracle/_ref/libref_attention.so not built (reference tree absent)")
    rng = np.random.default_rng(5)
    for B, T, H, D in [(2, 96, 4, 64), (1, 257, 2, 64), (3, 5, 1, 7)]:
        x = rng.standard_normal((B, T, 3 * H * D), dtype=np.float32)
        g = rng.standard_normal((B, T, H * D), dtype=np.float32)
        ro, rdx, _ = oracle.reference_run(x, g, H)
        assert np.abs(oracle.forward(x, H) - ro).max() < TOL
        assert np.abs(oracle.backward(x, g, H) - rdx).max() < TOL


def test_bad_arguments(oracle):
    x = np.zeros((1, 2, 12), np.float32)
    with pytest.raises(AssertionError):
        oracle.forward(x, 5)
