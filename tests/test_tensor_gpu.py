"""The element-wise tensor helpers (include/tensor_sm100.h) against numpy restatements of what the
reference's kernels compute (kernels/src/cuda/Tensor.cu:8-28 and cublasSaxpy): fill, arange and copy
are exact; axpy is one fused multiply-add per element, so it must be within one rounding of the
float64 value.  Sizes and offsets cover the vector body, the ragged tail and unaligned pointers.
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")

pytestmark = pytest.mark.gpu

SIZES = [0, 1, 3, 4, 1023, 4096, 1_000_003, 8 * 1024 * 768]


def stream():
    return torch.cuda.current_stream().cuda_stream


@pytest.mark.parametrize("n", SIZES)
@pytest.mark.parametrize("offset", [0, 1])
def test_fill_copy_arange_axpy(pkg, n, offset):
    L = pkg.lib()
    rng = np.random.default_rng(n + offset)
    guard = 8
    buf = torch.full((n + offset + guard,), -7.0, device="cuda")
    p = buf.data_ptr() + 4 * offset
    for value in (0.0, 1.0, -2.5):
        assert L.tensor_sm100_fill(p if n else None, n, value, stream()) == 0
        got = buf.cpu().numpy()
        assert np.all(got[:offset] == -7.0) and np.all(got[offset + n:] == -7.0), "wrote outside the range"
        assert np.all(got[offset:offset + n] == np.float32(value))
    assert L.tensor_sm100_arange(p if n else None, n, 3, 2, stream()) == 0
    got = buf.cpu().numpy()
    assert np.array_equal(got[offset:offset + n], (3 + 2 * np.arange(n)).astype(np.float32))
    assert np.all(got[offset + n:] == -7.0)

    src = torch.from_numpy(rng.standard_normal(n + offset).astype(np.float32)).cuda()
    ps = src.data_ptr() + 4 * offset
    assert L.tensor_sm100_copy(p if n else None, ps if n else None, n, stream()) == 0
    assert torch.equal(buf[offset:offset + n], src[offset:offset + n])
    assert torch.all(buf[offset + n:] == -7.0)

    y0 = buf[offset:offset + n].cpu().numpy().astype(np.float64)
    x = rng.standard_normal(n + offset).astype(np.float32)
    xt = torch.from_numpy(x).cuda()
    alpha = np.float32(0.37)
    assert L.tensor_sm100_axpy(n, float(alpha), xt.data_ptr() + 4 * offset if n else None, p if n else None, stream()) == 0
    got = buf[offset:offset + n].cpu().numpy()
    ref = np.float64(alpha) * x[offset:].astype(np.float64) + y0
    assert np.all(np.abs(got - ref) <= np.abs(ref) * 2.0 ** -23 + 1e-30)
    assert torch.all(buf[offset + n:] == -7.0)
    torch.cuda.synchronize()


@pytest.mark.parametrize("n,offset", [(1, 0), (1025, 1), (8 * 1024 * 3072 // 8, 0)])
def test_gelu_forward_backward(pkg, n, offset):
    """tanh-approximated GELU against its float64 evaluation (kernels/src/cuda/GeLU.cu:5-38)."""
    L = pkg.lib()
    rng = np.random.default_rng(n)
    x = (rng.standard_normal(n + offset) * 2.5).astype(np.float32)
    g = rng.standard_normal(n + offset).astype(np.float32)
    xt, gt = torch.from_numpy(x).cuda(), torch.from_numpy(g).cuda()
    y = torch.full((n + offset + 4,), -7.0, device="cuda")
    dx = torch.full((n + offset + 4,), -7.0, device="cuda")
    o = 4 * offset
    assert L.tensor_sm100_gelu_forward(xt.data_ptr() + o, y.data_ptr() + o, n, stream()) == 0
    assert L.tensor_sm100_gelu_backward(gt.data_ptr() + o, xt.data_ptr() + o, dx.data_ptr() + o, n, stream()) == 0
    from oracle import ops_oracle as ops  # the restatement tests/test_ops_oracle.py pins to kernels/src/cpu/GeLU.c

    y_ref = ops.gelu_forward(x[offset:])
    d_ref = ops.gelu_backward(g[offset:], x[offset:])
    assert np.abs(y[offset:offset + n].cpu().numpy() - y_ref).max() <= 2e-6 * max(1.0, np.abs(y_ref).max())
    assert np.abs(dx[offset:offset + n].cpu().numpy() - d_ref).max() <= 4e-6 * max(1.0, np.abs(d_ref).max())
    assert torch.all(y[offset + n:] == -7.0) and torch.all(dx[offset + n:] == -7.0)
    torch.cuda.synchronize()


def test_null_pointers(pkg):
    L = pkg.lib()
    assert L.tensor_sm100_fill(None, 4, 0.0, None) == -1
    assert L.tensor_sm100_copy(None, None, 4, None) == -1
    assert L.tensor_sm100_axpy(4, 1.0, None, None, None) == -1
