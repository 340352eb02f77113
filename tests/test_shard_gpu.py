"""The batch split of one fixed workload over GPUs (no collective on the data path): every rank runs the
same kernels on a contiguous batch slice, so the gathered output, dk and dv must equal the single-GPU
result bit for bit; dq is accumulated with reductions whose order is not fixed, so it is held to 1e-4.

With two or more GPUs visible the slices run on different devices; with one they run one after the
other on the same device, which still checks that a slice computed alone equals the same entries of the
full batch.  The shapes are those of the reference's configuration list (GPT-2 124M block, GPT-2 XL heads).
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def torch_gpu(pkg):
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch


def run_on(pkg, torch, device, x, g, H):
    with torch.cuda.device(device):
        pkg.init()
        xt, gt = x.to(f"cuda:{device}"), g.to(f"cuda:{device}")
        out, ctx = pkg.forward(xt, H)
        dx = pkg.backward(ctx, gt)
        assert pkg.device_status() == 0
        return out.cpu(), ctx.lse.cpu(), dx.cpu()


@pytest.mark.parametrize("B,T,H,world", [(8, 1024, 12, 2), (8, 1024, 12, 8), (6, 1024, 25, 4), (5, 384, 25, 2)])
def test_gathered_slices_equal_single_gpu(pkg, torch_gpu, B, T, H, world):
    import __graft_entry__ as entry

    torch = torch_gpu
    shard = entry.load_submodule("shard")
    D, C = 64, H * 64
    gen = torch.Generator().manual_seed(1234)
    x = torch.randn((B, T, 3 * C), generator=gen)
    g = torch.randn((B, T, C), generator=gen)
    ndev = torch.cuda.device_count()
    out1, lse1, dx1 = run_on(pkg, torch, 0, x, g, H)
    outs, lses, dxs = [], [], []
    for rank, (lo, hi) in enumerate(shard.batch_slices(B, world)):
        if hi == lo:
            continue
        o, l, d = run_on(pkg, torch, rank % ndev, x[lo:hi].contiguous(), g[lo:hi].contiguous(), H)
        outs.append(o), lses.append(l), dxs.append(d)
    out, lse, dx = torch.cat(outs), torch.cat(lses), torch.cat(dxs)
    assert torch.equal(out, out1), "gathered output differs from the single-GPU output"
    assert torch.equal(lse, lse1)
    assert torch.equal(dx[:, :, C:], dx1[:, :, C:]), "gathered dk / dv differ from the single-GPU result"
    assert float((dx[:, :, :C] - dx1[:, :, :C]).abs().max()) <= 1e-4
