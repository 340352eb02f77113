"""Generate the golden fixtures of tests/golden/ from the reference itself.

Must be run in a container that has the reference tree (gpt.c) mounted; the fixtures it writes are
committed so the tests need neither the tree nor this script at run time.

    python tests/golden/make_golden.py [--reference DIR]

Fixtures
  ref_selfattn_case.npz   the reference's own hand-written test inputs (tests/test_self_attention.py:7-58
                          of gpt.c: X 4x2x6, qkv weight/bias; D=3, H=2, T=2) pushed through the reference's
                          PyTorch module (model.py:13-54, CausalSelfAttention) with c_proj set to identity,
                          so the module output IS the attention output; qkv and d(loss)/d(qkv) are taken
                          with hooks.  The same inputs are also run through the reference's compiled CPU
                          kernel (kernels/src/cpu/Attention.c) and both answers are stored.
  seeded_*.npz            seeded N(0,1) inputs of small shapes with the outputs of the reference's compiled
                          CPU kernel (forward and backward).
  config1_digest.npz      digest (strided samples and sums) of the reference CPU kernel's output on the
                          README CPU-training shape B=8, T=128, H=12, D=64 with seed 1234.
"""
from __future__ import annotations

import argparse
import ast
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.abspath(os.path.join(HERE, "..", ".."))
sys.path.insert(0, ROOT)

from oracle import build as oracle_build  # noqa: E402
from oracle import oracle  # noqa: E402


def seeded_inputs(seed: int, B: int, T: int, H: int, D: int):
    """The input convention every seeded test uses: x then dout from one numpy Generator."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((B, T, 3 * H * D), dtype=np.float32)
    dout = rng.standard_normal((B, T, H * D), dtype=np.float32)
    return x, dout


def literal_assignments(path: str, names: set[str]) -> dict:
    tree = ast.parse(open(path).read())
    found = {}
    for node in tree.body:
        if isinstance(node, ast.Assign) and len(node.targets) == 1 and isinstance(node.targets[0], ast.Name):
            name = node.targets[0].id
            if name in names and name not in found:
                try:
                    found[name] = ast.literal_eval(node.value)
                except ValueError:
                    pass
    return found


def make_ref_selfattn(ref_dir: str) -> None:
    import torch

    sys.path.insert(0, ref_dir)
    import model as ref_model  # the reference's PyTorch twin

    vals = literal_assignments(os.path.join(ref_dir, "tests", "test_self_attention.py"),
                               {"X", "qkv_weight", "qkv_bias"})
    X = torch.tensor(vals["X"], dtype=torch.float32)
    W = torch.tensor(vals["qkv_weight"], dtype=torch.float32)
    bvec = torch.tensor(vals["qkv_bias"], dtype=torch.float32)
    n_embd, n_head, block = X.shape[-1], 2, X.shape[1]

    cfg = ref_model.GPTConfig(block_size=block, vocab_size=8, n_layer=1, n_head=n_head, n_embd=n_embd)
    attn = ref_model.CausalSelfAttention(cfg)
    with torch.no_grad():
        attn.c_attn.weight.copy_(W)
        attn.c_attn.bias.copy_(bvec)
        attn.c_proj.weight.copy_(torch.eye(n_embd))
        attn.c_proj.bias.zero_()
    grabbed = {}

    def hook(_m, _inp, outp):
        outp.retain_grad()
        grabbed["qkv"] = outp

    attn.c_attn.register_forward_hook(hook)
    y = attn(X)
    y.backward(torch.ones_like(y))
    qkv = grabbed["qkv"].detach().numpy().astype(np.float32)
    dqkv = grabbed["qkv"].grad.numpy().astype(np.float32)
    out = y.detach().numpy().astype(np.float32)
    dout = np.ones_like(out)

    k_out, k_dx, _ = oracle.reference_run(qkv, dout, n_head)
    assert np.abs(k_out - out).max() < 1e-5 and np.abs(k_dx - dqkv).max() < 1e-5, "reference C and PyTorch disagree"
    np.savez(os.path.join(HERE, "ref_selfattn_case.npz"), qkv=qkv, dout=dout, n_heads=np.int32(n_head),
             out_model_py=out, dqkv_model_py=dqkv, out_cpu_kernel=k_out, dqkv_cpu_kernel=k_dx)
    print("ref_selfattn_case: qkv", qkv.shape, "max|C-py| out %.2e dx %.2e" % (
        np.abs(k_out - out).max(), np.abs(k_dx - dqkv).max()))


SEEDED = [  # name, seed, B, T, H, D
    ("seeded_t130_d64", 11, 1, 130, 2, 64),   # ragged tail crossing a 128 tile
    ("seeded_t256_d64", 12, 1, 256, 1, 64),   # two full tiles
    ("seeded_t33_d16", 13, 2, 33, 3, 16),     # general head size
    ("seeded_t1_d64", 14, 2, 1, 2, 64),       # single token
    ("seeded_t64_d100", 15, 1, 64, 2, 100),   # head size that is not a power of two
]


def make_seeded() -> None:
    for name, seed, B, T, H, D in SEEDED:
        x, dout = seeded_inputs(seed, B, T, H, D)
        out, dx, _ = oracle.reference_run(x, dout, H)
        np.savez(os.path.join(HERE, name + ".npz"), x=x, dout=dout, n_heads=np.int32(H), out=out, dx=dx,
                 seed=np.int32(seed))
        print(name, x.shape, "-> out", out.shape)


def digest(a: np.ndarray, stride: int = 97):
    flat = a.reshape(-1)
    return flat[::stride].copy(), np.float64(flat.astype(np.float64).sum()), np.float64((flat.astype(np.float64) ** 2).sum())


def make_config1_digest() -> None:
    B, T, H, D, seed = 8, 128, 12, 64, 1234
    x, dout = seeded_inputs(seed, B, T, H, D)
    out, dx, _ = oracle.reference_run(x, dout, H)
    so, s1, s2 = digest(out)
    sx, d1, d2 = digest(dx)
    np.savez(os.path.join(HERE, "config1_digest.npz"), shape=np.int32([B, T, H, D]), seed=np.int32(seed),
             x_sum=np.float64(x.astype(np.float64).sum()), out_samples=so, out_sum=s1, out_sumsq=s2,
             dx_samples=sx, dx_sum=d1, dx_sumsq=d2, stride=np.int32(97))
    print("config1_digest: out sum %.6f dx sum %.6f" % (s1, d1))


def ops_inputs():
    """Seeded inputs of the fixtures of the kernels either side of the attention layer (small shapes with
    ragged sizes; the tests recompute the restatements on the same inputs)."""
    rng = np.random.default_rng(20240415)
    M, N, K = 37, 50, 24
    rows, C = 29, 40
    d = {
        "lin_x": rng.standard_normal((M, K), dtype=np.float32), "lin_w": (rng.standard_normal((N, K), dtype=np.float32) * 0.1).astype(np.float32),
        "lin_b": rng.standard_normal(N, dtype=np.float32), "lin_dy": rng.standard_normal((M, N), dtype=np.float32),
        "lin_dw0": rng.standard_normal((N, K), dtype=np.float32), "lin_db0": rng.standard_normal(N, dtype=np.float32),
        "ln_x": (rng.standard_normal((rows, C)) * 1.7 + 0.3).astype(np.float32), "ln_w": (1.0 + 0.1 * rng.standard_normal(C)).astype(np.float32),
        "ln_b": (0.1 * rng.standard_normal(C)).astype(np.float32), "ln_dy": rng.standard_normal((rows, C)).astype(np.float32),
        "ln_dw0": rng.standard_normal(C).astype(np.float32), "ln_db0": rng.standard_normal(C).astype(np.float32),
        "ln_dx0": rng.standard_normal((rows, C)).astype(np.float32),
        "ce_logits": (rng.standard_normal((rows, 101)) * 3.0).astype(np.float32), "ce_targets": rng.integers(0, 101, size=rows).astype(np.float32),
        "ce_g": rng.standard_normal(rows).astype(np.float32), "ce_d0": (rng.standard_normal((rows, 101)) * 0.01).astype(np.float32),
        "ad_p": (rng.standard_normal(1003) * 0.05).astype(np.float32), "ad_g": (rng.standard_normal(1003) * 0.01).astype(np.float32),
        "ad_m": (rng.standard_normal(1003) * 0.001).astype(np.float32), "ad_v": (np.abs(rng.standard_normal(1003)) * 1e-4).astype(np.float32),
        "ge_x": (rng.standard_normal(777) * 2.5).astype(np.float32), "ge_g": rng.standard_normal(777).astype(np.float32),
    }
    return d


def make_ops() -> None:
    """One fixture per kernel either side of the layer, produced by the reference's own CPU kernels."""
    ref = oracle.reference_ops()
    d = ops_inputs()
    out = dict(d)
    out["lin_y"] = ref.linear_forward(d["lin_x"], d["lin_w"], d["lin_b"])
    out["lin_dx"], out["lin_dw"], out["lin_db"] = ref.linear_backward(d["lin_dy"], d["lin_x"], d["lin_w"], d["lin_dw0"], d["lin_db0"])
    out["ln_y"], out["ln_mean"], out["ln_rstd"] = ref.layernorm_forward(d["ln_x"], d["ln_w"], d["ln_b"], 1e-5)
    out["ln_dw"], out["ln_db"], out["ln_dx"] = ref.layernorm_backward(d["ln_dy"], d["ln_x"], out["ln_mean"], out["ln_rstd"], d["ln_w"],
                                                                    d["ln_dw0"], d["ln_db0"], d["ln_dx0"])
    out["ce_logsm"], loss = ref.xent_forward(d["ce_logits"], d["ce_targets"])
    out["ce_loss"] = np.float32(loss)
    out["ce_dout_zero"] = ref.xent_backward(d["ce_g"], d["ce_targets"], out["ce_logsm"], np.zeros_like(d["ce_d0"]))
    out["ce_dout_d0"] = ref.xent_backward(d["ce_g"], d["ce_targets"], out["ce_logsm"], d["ce_d0"])
    p, m, v = d["ad_p"], d["ad_m"], d["ad_v"]
    for step in (1, 2, 3):
        p, m, v = ref.adamw_step(p, d["ad_g"], m, v, 3e-4, 0.9, 0.999, 0.01, 1e-8, step)
    out["ad_p3"], out["ad_m3"], out["ad_v3"] = p, m, v
    out["ge_y"] = ref.gelu_forward(d["ge_x"])
    out["ge_dx"] = ref.gelu_backward(d["ge_g"], d["ge_x"])
    np.savez(os.path.join(HERE, "ops_cases.npz"), **out)
    print("ops_cases: %d arrays" % len(out))


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=oracle_build.REF_DIR,
                    help="gpt.c source tree (default: GPTC_REFERENCE_DIR, else ../reference beside the repository)")
    args = ap.parse_args()
    oracle_build.build_all()
    if not oracle.have_reference():
        sys.exit("the reference CPU kernel could not be built; fixtures need it")
    make_ref_selfattn(args.reference)
    make_seeded()
    make_config1_digest()
    if oracle.have_reference_ops():
        make_ops()
