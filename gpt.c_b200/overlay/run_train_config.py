"""GPT-2 124M training step through the unchanged train_gpt of gpt.c, with the reference's own CUDA
attention and with this repository's attention (the overlay build), on synthetic inputs.

    python gpt.c_b200/overlay/run_train_config.py [--steps 12] [--layers 12] [--out result.json] [--prepare DIR]

Needs this repository's build of gpt.c (build_libgpt.py, under overlay/_build/), the unmodified build
beside the CPU checkers (oracle/build.py) and a CUDA device.  A synthetic
checkpoint in the reference's format (train_gpt.c:201-287: 256-int header with magic 20240415,
block size, vocab, layers, heads, width, shape-header length, steps; then (ndims, dims...) per
tensor; then fp32 data in parameters() order) and a raw int32 token file (src/dataloader.c:44-80)
are written to a temporary directory: weights N(0, 0.02) with the residual projections scaled by
1/sqrt(2*layers), LayerNorm weight 1 / bias 0, biases 0, token ids uniform in [0, 50257).  These
stand in for the text datasets the reference's README trains on (they need a download).
Prints one JSON object with tokens/s (median of steps 3..N) and the loss curves of both builds.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import statistics
import subprocess
import sys
import tempfile

import numpy as np

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), "..", ".."))
BUILDS = {"reference_cuda_attention": os.path.join(ROOT, "oracle", "_ref", "gptc_reference"),
          "sm100_attention": os.path.join(ROOT, "gpt.c_b200", "overlay", "_build", "gptc_overlay")}


def write_checkpoint(path: str, n_layers: int, n_heads: int, n_embd: int, vocab: int, block: int, seed: int) -> None:
    rng = np.random.default_rng(seed)
    C = n_embd
    resid = 1.0 / np.sqrt(2.0 * n_layers)
    tensors = []  # (shape, kind, scale)
    tensors.append(((vocab, C), "w", 1.0))
    tensors.append(((block, C), "w", 1.0))
    for _ in range(n_layers):
        tensors += [((C,), "one", 0), ((C,), "zero", 0), ((3 * C, C), "w", 1.0), ((3 * C,), "zero", 0),
                    ((C, C), "w", resid), ((C,), "zero", 0), ((C,), "one", 0), ((C,), "zero", 0),
                    ((4 * C, C), "w", 1.0), ((4 * C,), "zero", 0), ((C, 4 * C), "w", resid), ((C,), "zero", 0)]
    tensors += [((C,), "one", 0), ((C,), "zero", 0)]
    shape_header = []
    for shape, _, _ in tensors:
        shape_header += [len(shape), *shape]
    header = np.zeros(256, dtype=np.int32)
    header[:8] = [20240415, block, vocab, n_layers, n_heads, n_embd, len(shape_header), 0]
    with open(path, "wb") as f:
        f.write(header.tobytes())
        f.write(np.asarray(shape_header, dtype=np.int32).tobytes())
        for shape, kind, scale in tensors:
            n = int(np.prod(shape))
            if kind == "w":
                f.write((rng.standard_normal(n, dtype=np.float32) * np.float32(0.02 * scale)).tobytes())
            elif kind == "one":
                f.write(np.ones(n, dtype=np.float32).tobytes())
            else:
                f.write(np.zeros(n, dtype=np.float32).tobytes())


def write_tokens(path: str, steps: int, batch: int, block: int, vocab: int, seed: int) -> None:
    rng = np.random.default_rng(seed)
    rng.integers(0, vocab, size=steps * (batch * block + 1), dtype=np.int32).tofile(path)


def run_build(build_dir: str, ckpt: str, tokens: str, batch: int, block: int, log_dir: str):
    cmd = [os.path.join(build_dir, "train_gpt"), f"--train-data={tokens}", "--max-epochs=1", f"--batch-size={batch}",
           f"--block-size={block}", f"--load-checkpoint={ckpt}", "--device=cuda", "--lr=3e-4", f"--log-dir={log_dir}"]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=3000)
    steps = re.findall(r"step: (\d+) \| train loss: ([-\d.naninf]+) lr: \S+ \| took ([\d.]+) ms", res.stdout)
    return res.returncode, [(int(s), float(l), float(ms)) for s, l, ms in steps], res.stdout[-1500:] + res.stderr[-1500:]


def run(steps: int = 12, layers: int = 12, heads: int = 12, embd: int = 768, batch: int = 8, block: int = 1024) -> dict:
    """Runs both builds on the same synthetic checkpoint and token file; returns the result dictionary."""
    missing = [k for k, d in BUILDS.items() if not os.path.exists(os.path.join(d, "train_gpt"))]
    if missing:
        raise RuntimeError(f"missing builds {missing}: run gpt.c_b200/overlay/build_libgpt.py and oracle/build.py "
                           "where the gpt.c tree is available")
    result = {"config": {"layers": layers, "heads": heads, "embd": embd, "batch": batch, "block": block,
                         "vocab": 50257, "steps": steps, "data": "synthetic uniform token ids, N(0,0.02) weights"}}
    with tempfile.TemporaryDirectory() as tmp:
        ckpt, tok = os.path.join(tmp, "ckpt.bin"), os.path.join(tmp, "tokens.bin")
        write_checkpoint(ckpt, layers, heads, embd, 50257, block, seed=1234)
        write_tokens(tok, steps, batch, block, 50257, seed=4321)
        for name, d in BUILDS.items():
            rc, log, tail = run_build(d, ckpt, tok, batch, block, os.path.join(tmp, "logs_" + name))
            entry = {"returncode": rc, "losses": [l for _, l, _ in log], "step_ms": [ms for _, _, ms in log]}
            timed = [ms for s, _, ms in log if s >= 3]
            if timed:
                entry["median_step_ms"] = statistics.median(timed)
                entry["tokens_per_s"] = batch * block / (entry["median_step_ms"] * 1e-3)
            if rc != 0 or not log:
                entry["output_tail"] = tail
            result[name] = entry
    ref, new = result["reference_cuda_attention"], result["sm100_attention"]
    if ref.get("losses") and new.get("losses"):
        n = min(len(ref["losses"]), len(new["losses"]))
        result["max_loss_difference"] = max(abs(x - y) for x, y in zip(ref["losses"][:n], new["losses"][:n]))
    if "tokens_per_s" in ref and "tokens_per_s" in new:
        result["speedup_tokens_per_s"] = new["tokens_per_s"] / ref["tokens_per_s"]
    return result


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=12)
    ap.add_argument("--layers", type=int, default=12)
    ap.add_argument("--heads", type=int, default=12)
    ap.add_argument("--embd", type=int, default=768)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--block", type=int, default=1024)
    ap.add_argument("--out", default=None)
    ap.add_argument("--prepare", default=None, metavar="DIR",
                    help="only write ckpt.bin and tokens.bin into DIR and print the train_gpt command lines "
                         "(e.g. to run one of them under a profiler)")
    a = ap.parse_args()
    if a.prepare:
        os.makedirs(a.prepare, exist_ok=True)
        ckpt, tok = os.path.join(a.prepare, "ckpt.bin"), os.path.join(a.prepare, "tokens.bin")
        write_checkpoint(ckpt, a.layers, a.heads, a.embd, 50257, a.block, seed=1234)
        write_tokens(tok, a.steps, a.batch, a.block, 50257, seed=4321)
        for name, d in BUILDS.items():
            print(name + ":", os.path.join(d, "train_gpt"), f"--train-data={tok}", "--max-epochs=1", f"--batch-size={a.batch}",
                  f"--block-size={a.block}", f"--load-checkpoint={ckpt}", "--device=cuda", "--lr=3e-4",
                  f"--log-dir={os.path.join(a.prepare, 'logs_' + name)}")
        sys.exit(0)
    try:
        result = run(a.steps, a.layers, a.heads, a.embd, a.batch, a.block)
    except RuntimeError as e:
        sys.exit(str(e))
    text = json.dumps(result)
    print(text)
    if a.out:
        with open(a.out, "w") as f:
            f.write(text + "\n")
