"""Parity of the cross-entropy kernels (include/xent_sm100.h) against the float64 numpy restatement of the
reference in oracle/ops_oracle.py, pinned to the reference's own CPU kernel by tests/test_ops_oracle.py
(kernels/src/cpu/CrossEntropyLoss.c; kernels/src/cuda/CrossEntropyLoss.cu:8-129 has the same arithmetic but
accumulates the loss into its output, which is what the CUDA kernels here do too):
log-softmax, mean negative log-likelihood accumulated into the loss, and the backward that works on what
dout already holds.  Tolerance: fp32 with fast exponentials, 2e-6 absolute on log-softmax values of order
10, 1e-6 relative on the loss, 1e-7 + 1e-5 relative on the gradient.
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
from oracle import ops_oracle as ops  # noqa: E402

pytestmark = pytest.mark.gpu


def stream():
    return torch.cuda.current_stream().cuda_stream


@pytest.mark.parametrize("rows,C", [(64, 50257), (1000, 1003), (7, 5), (2048, 512), (1, 1)])
def test_cross_entropy_forward_backward_vs_cpu(pkg, rows, C):
    L = pkg.lib()
    rng = np.random.default_rng(rows + C)
    logits = (rng.standard_normal((rows, C)) * 3.0).astype(np.float32)
    targets = rng.integers(0, C, size=rows).astype(np.float32)
    g = rng.standard_normal(rows).astype(np.float32)

    logsm_ref, loss_ref = ops.xent_forward(logits, targets)

    lt, tt, gt = (torch.from_numpy(a).cuda() for a in (logits, targets, g))
    logsm = torch.empty_like(lt)
    loss = torch.full((1,), 0.25, device="cuda")  # accumulates on top of what is there
    assert L.xent_sm100_forward(lt.data_ptr(), tt.data_ptr(), logsm.data_ptr(), loss.data_ptr(), rows, C, stream()) == 0
    assert np.abs(logsm.cpu().numpy() - logsm_ref).max() <= 2e-6 * max(1.0, np.abs(logsm_ref).max())
    assert abs(loss.item() - 0.25 - loss_ref) <= 1e-6 * max(1.0, abs(loss_ref)) + 2e-6

    # backward from a zero-filled dout (what the layer does) ...
    dout = torch.zeros_like(lt)
    assert L.xent_sm100_backward(gt.data_ptr(), tt.data_ptr(), logsm.data_ptr(), dout.data_ptr(), rows, C, stream()) == 0
    d_ref = ops.xent_backward(g, targets, logsm_ref)
    assert np.abs(dout.cpu().numpy() - d_ref).max() <= 1e-7 + 1e-5 * np.abs(d_ref).max()

    # ... and from a dout that already holds something: the reference's formula on its contents
    d0 = (rng.standard_normal((rows, C)) * 0.01).astype(np.float32)
    dout = torch.from_numpy(d0.copy()).cuda()
    assert L.xent_sm100_backward(gt.data_ptr(), tt.data_ptr(), logsm.data_ptr(), dout.data_ptr(), rows, C, stream()) == 0
    d_ref2 = ops.xent_backward(g, targets, logsm_ref, d0)
    assert np.abs(dout.cpu().numpy() - d_ref2).max() <= 1e-6 + 1e-5 * np.abs(d_ref2).max()
    torch.cuda.synchronize()


def test_cross_entropy_argument_errors(pkg):
    L = pkg.lib()
    assert L.xent_sm100_forward(None, None, None, None, 1, 1, None) == -1
    t = torch.zeros(8, device="cuda")
    p = t.data_ptr()
    assert L.xent_sm100_forward(p, p, p, p, 0, 4, None) == -2
    assert L.xent_sm100_backward(p, p, p, p, 4, 0, None) == -2
