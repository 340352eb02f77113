"""Build gpt.c with this repository's attention in place of its own (and, beside it, unmodified).

The reference tree is read where it lies (never copied, its Makefile is not run).  The build is
written under ``gpt.c_b200/overlay/_build/`` (git-ignored):

  _build/gptc_overlay/   libgpt.so = reference sources, with src/attention.c,
                         kernels/src/core/Attention.c and kernels/src/cuda/{Attention,Linear,
                         LayerNorm,Tensor,GeLU,CrossEntropyLoss,AdamW,Alloc}.cu taken from
                         gpt.c_b200/overlay/, linked against libattn_sm100.so;
                         plus train_gpt, infer_gpt and layer_driver

``build(ref, out_dir, overlay=False)`` makes the same executables from the unmodified reference (its
cuBLAS + SIMT attention compiled for sm_100a); the checker-side recipe ``oracle/build.py`` uses it for
the GPU baseline it keeps beside the CPU one.

    python gpt.c_b200/overlay/build_libgpt.py --reference DIR      (or GPTC_REFERENCE_DIR=DIR)
"""
from __future__ import annotations

import argparse
import glob
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.abspath(os.path.join(HERE, "..", ".."))
BUILD_DIR = os.path.join(HERE, "_build")
OVERLAY_OUT = os.path.join(BUILD_DIR, "gptc_overlay")


def find_openblas() -> tuple[str, bool] | None:
    """(path, uses_scipy_prefix) of an LP64 OpenBLAS shared object, or None.  gpt.c takes OpenBLAS from a
    submodule that is not vendored; the copies inside the Python wheels are what an offline box has."""
    site = sysconfig.get_paths()["purelib"]
    hits = sorted(glob.glob(os.path.join(site, "scipy.libs", "libscipy_openblas-*.so")))
    if hits:
        return hits[0], True
    for pat in ("opencv_python_headless.libs/libopenblas*.so*", "numpy.libs/libopenblas*.so*"):
        hits = sorted(glob.glob(os.path.join(site, pat)))
        if hits:
            return hits[0], False
    for d in ("/usr/lib/x86_64-linux-gnu", "/usr/lib64", "/usr/local/lib"):
        hits = sorted(glob.glob(os.path.join(d, "libopenblas.so*")))
        if hits:
            return hits[0], False
    return None


def reference_dir(explicit: str | None = None) -> str | None:
    """The gpt.c source tree: --reference, else GPTC_REFERENCE_DIR, else a directory `reference` beside
    this repository.  None when there is none (the builds are then used as they are)."""
    for cand in (explicit, os.environ.get("GPTC_REFERENCE_DIR"), os.path.join(ROOT, "..", "reference")):
        if cand and os.path.isdir(os.path.join(cand, "kernels", "src", "cuda")):
            return os.path.abspath(cand)
    return None

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
    inc = ["-I", HERE, "-I", os.path.join(ref, "include"), "-I", os.path.join(ref, "kernels/include"),
           "-I", os.path.join(ref, "kernels/src"), "-I", os.path.join(ROOT, "include")]
    defs = ["-DOMP"] + (["-DGPTC_BLAS_SCIPY"] if scipy_prefix else [])
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
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    for name, src in exe_srcs.items():
        extra = []
        if name == "layer_driver" and os.path.exists(os.path.join(cuda_home, "lib64", "libcudart.so")):
            # the driver's keep-pool option sets an attribute of the device's default memory pool
            extra = ["-DLAYER_DRIVER_CUDART", "-I", os.path.join(cuda_home, "include"), "-L", os.path.join(cuda_home, "lib64"),
                     "-lcudart", "-Wl,-rpath," + os.path.join(cuda_home, "lib64")]
        run(["gcc", *host_flags, *defs, *inc, src, "-o", os.path.join(out_dir, name), lib, "-Wl,-rpath,$ORIGIN",
             "-Wl,-rpath," + out_dir, "-lm", "-lgomp", *extra])
    return out_dir


def build_overlay(ref: str) -> str:
    return build(ref, OVERLAY_OUT, overlay=True)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=None, help="gpt.c source tree (default: GPTC_REFERENCE_DIR)")
    a = ap.parse_args()
    ref = reference_dir(a.reference)
    if ref is None:
        sys.exit("no gpt.c source tree: pass --reference DIR or set GPTC_REFERENCE_DIR")
    print(build_overlay(ref))
