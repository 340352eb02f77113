"""Parity of the tcgen05 Linear kernels (include/linear_sm100.h) against the float64 numpy restatement of the
reference's Linear (kernels/src/cpu/Linear.c:4-31 forward, :33-88 backward) in oracle/ops_oracle.py, pinned to
the reference's own CPU kernel by tests/test_ops_oracle.py: y = x W^T + b, dx = dy W, dW += dy^T x,
db += colsum(dy).

Tolerance: the kernels use TF32 inputs (the upper 19 bits of each fp32 operand: truncation, relative
error below 2^-10 per operand) with fp32 accumulation, the precision class of the reference's CUDA
path (cuBLAS TF32 tensor-op math).  Every product is therefore within 2^-9 of the exact one, which
gives the element-wise bound |err| <= 2^-9 * (|a| @ |b|) plus the fp32 accumulation error; the fused
bf16 planes must reproduce y itself to 2^-16 relative.
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
from oracle import ops_oracle as ops  # noqa: E402

pytestmark = pytest.mark.gpu

SHAPES = [
    # (M, N, K)                      what
    (8 * 128, 2304, 768),          # QKV projection, config 1
    (2 * 1024, 768, 768),          # c_proj
    (300, 2304, 768),              # ragged M (tail tile)
    (256, 96, 64),                 # N, K below one tile
    (1000, 3072, 768),             # MLP up-projection shape
    (260, 50257, 768),             # vocabulary projection: rows of y not 16-byte aligned, plain stores
    (130, 1001, 64),               # the same path with a ragged last tile in every direction
    (70, 95, 64),                  # 31 of 32 columns in the last block: the padded copy of dy reads its last word alone
    (70, 94, 32),                  # rows of dy start 0 or 2 floats past a 16-byte boundary
    (9, 16415, 32),                # long contraction for dx (513 steps): cut into pieces that add into a zeroed dx
    (260, 16392, 768),             # weight above 48 MB with 16-byte-aligned rows of y: row-fastest tile order, copy-engine stores
]


def within(got, ref, a, b):
    """a [M, L], b [L, N]: got must be within the TF32 truncation bound of ref = a @ b."""
    a64, b64 = np.abs(a.astype(np.float64)), np.abs(b.astype(np.float64))
    lim = 2.0 ** -9 * (a64 @ b64) + 2.0 ** -20 * a.shape[1] * a64.max() * b64.max()
    excess = np.abs(got.astype(np.float64) - ref) - lim
    assert excess.max() <= 0, f"max error {np.abs(got - ref).max():.3e}, exceeds the bound by {excess.max():.3e}"


def inputs(M, N, K, seed):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((M, K), dtype=np.float32)
    w = (rng.standard_normal((N, K), dtype=np.float32) * 0.05).astype(np.float32)
    b = rng.standard_normal(N, dtype=np.float32)
    dy = rng.standard_normal((M, N), dtype=np.float32)
    return x, w, b, dy


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_linear_forward_vs_cpu(pkg, M, N, K):
    x, w, b, _ = inputs(M, N, K, 11)
    ref = ops.linear_forward(x, w, b)
    y = pkg.linear_forward(torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda(), torch.from_numpy(b).cuda())
    assert pkg.device_status() == 0
    within(y.cpu().numpy(), ref, x, w.T)
    # without bias
    y0 = pkg.linear_forward(torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda(), None)
    within(y0.cpu().numpy(), ref - b, x, w.T)


def test_linear_forward_planes_feed_attention(pkg, oracle):
    """The fused bf16 planes equal the split of y, and attention run from them (core only) matches
    attention run from y itself."""
    B, T, H, D = 2, 256, 4, 64
    C = H * D
    x, w, b, _ = inputs(B * T, 3 * C, C, 5)
    xt, wt, bt = (torch.from_numpy(a).cuda() for a in (x, w, b))
    planes = torch.empty(pkg.saved_bytes(B, T, H, D), device="cuda", dtype=torch.uint8)
    y = pkg.linear_forward(xt.view(B, T, C), wt, bt, planes=planes)
    assert pkg.device_status() == 0
    n = B * T * 3 * C
    plane_bytes = pkg.saved_bytes(B, T, H, D) // 2
    hi = planes[: 2 * n].view(torch.bfloat16).float()
    lo = planes[plane_bytes: plane_bytes + 2 * n].view(torch.bfloat16).float()
    yy = y.reshape(-1)
    assert torch.equal(hi, yy.bfloat16().float())
    assert ((hi + lo) - yy).abs().max().item() <= 2.0 ** -16 * yy.abs().max().item()
    # attention from the planes (split pass skipped) == attention from y
    out_a = torch.empty(B, T, C, device="cuda")
    lse_a = torch.empty(B, H, T, device="cuda")
    pkg.forward_into(y, out_a, None, lse_a, planes, H, pkg.FLAG_CORE_ONLY)
    out_b, _ = pkg.forward(y, H)
    assert pkg.device_status() == 0
    assert torch.equal(out_a, out_b)
    ref = oracle.forward(y.cpu().numpy(), H)
    assert np.abs(out_a.cpu().numpy() - ref).max() < 2e-3


@pytest.mark.parametrize("M,N,K", [s for s in SHAPES if s[2] % 32 == 0])
def test_linear_backward_vs_cpu(pkg, M, N, K):
    x, w, b, dy = inputs(M, N, K, 23)
    rng = np.random.default_rng(99)
    dw0 = rng.standard_normal((N, K), dtype=np.float32)
    db0 = rng.standard_normal(N, dtype=np.float32)
    dx_ref, dw_ref, db_ref = ops.linear_backward(dy, x, w, dw0, db0)
    dw = torch.from_numpy(dw0.copy()).cuda()
    db = torch.from_numpy(db0.copy()).cuda()
    dx = pkg.linear_backward(torch.from_numpy(dy).cuda(), torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda(), dw, db)
    assert pkg.device_status() == 0
    within(dx.cpu().numpy(), dx_ref, dy, w)
    within(dw.cpu().numpy(), dw_ref, dy.T, x)
    assert np.abs(db.cpu().numpy() - db_ref).max() <= 1e-5 * np.sqrt(M) * 8


def test_linear_backward_parts_can_be_skipped(pkg):
    M, N, K = 512, 768, 768
    x, w, b, dy = inputs(M, N, K, 31)
    dyt, xt, wt = (torch.from_numpy(a).cuda() for a in (dy, x, w))
    dw_full = torch.zeros(N, K, device="cuda")
    dx_full = pkg.linear_backward(dyt, xt, wt, dw_full, None)
    # dx only
    dx_only = pkg.linear_backward(dyt, xt, wt, None, None)
    assert torch.equal(dx_only, dx_full)
    # dW only (accumulates on top of what is there)
    dw_only = torch.zeros(N, K, device="cuda")
    assert pkg.linear_backward(dyt, xt, wt, dw_only, None, want_dx=False) is None
    assert pkg.device_status() == 0
    within(dw_only.cpu().numpy(), dy.astype(np.float64).T @ x.astype(np.float64), dy.T, x)


def test_linear_argument_errors(pkg):
    L = pkg.lib()
    assert L.linear_sm100_forward(None, None, None, None, None, 1, 4, 4, None) == -1
    t = torch.zeros(64, device="cuda")
    p = t.data_ptr()
    assert L.linear_sm100_forward(p, p, None, p, None, 0, 4, 4, None) == -2
    assert L.linear_sm100_forward(p, p, None, p, None, 4, 4, 6, None) == -3
    assert L.linear_sm100_forward(p, p, None, p, p, 4, 12, 8, None) == -3  # planes need N % 8 == 0
    assert L.linear_sm100_backward(p, p, p, p, p, None, None, 4, 32, 48, None) == -3  # K % 32
    assert L.linear_sm100_backward(p, p, p, p, p, None, None, 4, 50, 32, None) == -1  # scratch needed, none given
    assert L.linear_sm100_backward_scratch_bytes(260, 50257, 768) == 260 * 50272 * 4
    assert L.linear_sm100_backward_scratch_bytes(260, 2304, 768) == 0
