"""Build gpt.c with this repository's attention in place of its own (and, beside it, unmodified).

The reference tree is read where it lies (never copied, its Makefile is not run).  Two builds are
written under ``oracle/_ref/`` (git-ignored, reference-derived):

  oracle/_ref/gptc_overlay/    libgpt.so = reference sources, with src/attention.c,
                               kernels/src/core/Attention.c and kernels/src/cuda/{Attention,Linear,
                               LayerNorm,Tensor,GeLU,CrossEntropyLoss,AdamW,Alloc}.cu taken from gpt.c_b200/overlay/, linked
                               against libattn_sm100.so;
                               plus train_gpt, infer_gpt and layer_driver
  oracle/_ref/gptc_reference/  the same executables from the unmodified reference (its cuBLAS + SIMT
                               attention compiled for sm_100a): the GPU baseline

    python gpt.c_b200/overlay/build_libgpt.py [--reference DIR] [--only overlay|reference]
"""
from __future__ import annotations

import argparse
import glob
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.abspath(os.path.join(HERE, "..", ".."))
sys.path.insert(0, ROOT)
from oracle.build import find_openblas  # noqa: E402

ATTN_LIB_DIR = os.path.join(ROOT, "gpt.c_b200", "lib")
REPLACED = {"src/attention.c", "kernels/src/core/Attention.c", "kernels/src/cuda/Attention.cu",
            "kernels/src/cuda/Linear.cu", "kernels/src/cuda/Alloc.cu", "kernels/src/cuda/LayerNorm.cu", "kernels/src/cuda/Tensor.cu",
            "kernels/src/cuda/CrossEntropyLoss.cu", "kernels/src/cuda/AdamW.cu", "kernels/src/cuda/GeLU.cu"}


def run(cmd):
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(cmd) + "\n" + res.stdout + res.stderr)


def build(ref: str, out_dir: str, overlay: bool) -> str:
    blas = find_openblas()
    if blas is None:
        raise RuntimeError("no LP64 OpenBLAS shared object found")
    blas_lib, scipy_prefix = blas
    obj_dir = os.path.join(out_dir, "obj")
    os.makedirs(obj_dir, exist_ok=True)
    inc = ["-I", os.path.join(ROOT, "oracle"), "-I", os.path.join(ref, "include"), "-I", os.path.join(ref, "kernels/include"),
           "-I", os.path.join(ref, "kernels/src"), "-I", os.path.join(ROOT, "include")]
    defs = ["-DOMP"] + (["-DREF_BLAS_SCIPY"] if scipy_prefix else [])
    host_flags = ["-O3", "-march=x86-64-v3", "-fopenmp", "-fPIC", "-w"]

    c_srcs, cu_srcs = [], []
    for pat in ("src/*.c", "kernels/src/common/*.c", "kernels/src/core/*.c", "kernels/src/cpu/*.c"):
        c_srcs += sorted(glob.glob(os.path.join(ref, pat)))
    cu_srcs += sorted(glob.glob(os.path.join(ref, "kernels/src/cuda/*.cu")))
    if overlay:
        c_srcs = [s for s in c_srcs if os.path.relpath(s, ref) not in REPLACED]
        cu_srcs = [s for s in cu_srcs if os.path.relpath(s, ref) not in REPLACED]
        c_srcs += [os.path.join(HERE, "src/attention.c"), os.path.join(HERE, "kernels/src/core/Attention.c")]
        cu_srcs += [os.path.join(HERE, "kernels/src/cuda", f) for f in ("Attention.cu", "Linear.cu", "Alloc.cu", "LayerNorm.cu", "Tensor.cu", "CrossEntropyLoss.cu", "AdamW.cu", "GeLU.cu")]
        inc += ["-I", os.path.join(HERE, "kernels/src/cuda")]

    jobs = []
    objs = []
    for s in c_srcs:
        o = os.path.join(obj_dir, os.path.relpath(s, "/").replace("/", "_") + ".o")
        objs.append(o)
        jobs.append(["gcc", *host_flags, *defs, *inc, "-c", s, "-o", o])
    for s in cu_srcs:
        o = os.path.join(obj_dir, os.path.relpath(s, "/").replace("/", "_") + ".o")
        objs.append(o)
        jobs.append(["nvcc", "-ccbin=gcc", "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O3",
                     "--expt-relaxed-constexpr", "-lineinfo", "-Xcompiler", "-fPIC,-w,-O3", *defs, *inc, "-c", s, "-o", o])
    with ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as pool:
        list(pool.map(run, jobs))

    lib = os.path.join(out_dir, "libgpt.so")
    link = ["nvcc", "-ccbin=gcc", "-shared", "-o", lib, *objs, blas_lib, "-Xlinker", "-rpath," + os.path.dirname(blas_lib),
            "-lcublas", "-lgomp", "-lm"]
    if overlay:
        link += [os.path.join(ATTN_LIB_DIR, "libattn_sm100.so"), "-Xlinker", "-rpath," + ATTN_LIB_DIR,
                 "-Xlinker", "-rpath,$ORIGIN/../../../gpt.c_b200/lib"]
    run(link)

    exe_srcs = {"train_gpt": os.path.join(ref, "train_gpt.c"), "infer_gpt": os.path.join(ref, "infer_gpt.c"),
                "layer_driver": os.path.join(HERE, "layer_driver.c")}
    for name, src in exe_srcs.items():
        run(["gcc", *host_flags, *defs, *inc, src, "-o", os.path.join(out_dir, name), lib, "-Wl,-rpath,$ORIGIN",
             "-Wl,-rpath," + out_dir, "-lm", "-lgomp"])
    return out_dir


def build_all(ref: str, only: str | None = None) -> dict:
    out = {}
    base = os.path.join(ROOT, "oracle", "_ref")
    if only in (None, "overlay"):
        out["overlay"] = build(ref, os.path.join(base, "gptc_overlay"), overlay=True)
    if only in (None, "reference"):
        out["reference"] = build(ref, os.path.join(base, "gptc_reference"), overlay=False)
    return out


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("GPTC_REFERENCE_DIR", "/root/reference"))
    ap.add_argument("--only", choices=["overlay", "reference"], default=None)
    a = ap.parse_args()
    print(build_all(a.reference, a.only))
