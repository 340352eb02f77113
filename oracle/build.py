"""Build recipe for the CPU checkers.  TEST INFRASTRUCTURE ONLY.

Two shared libraries are produced:

* ``oracle/liboracle.so`` from ``oracle/attention_oracle.c`` (the plain-C restatement), always;
* ``oracle/_ref/libref_attention.so`` from the reference's own CPU attention sources compiled
  where they lie in the reference tree (``kernels/src/cpu/Attention.c``, ``kernels/src/cpu/Alloc.c``)
  plus ``oracle/ref_driver.c``, linked against an LP64 OpenBLAS found in the Python environment.
  This one is built only when the reference tree is present; the reference's own build system is
  not run and no reference source is copied.

* ``oracle/_ref/libref_ops.so`` from the reference's CPU kernels either side of the attention layer
  (``kernels/src/cpu/{Linear,LayerNorm,CrossEntropyLoss,AdamW,GeLU}.c``) plus ``oracle/ref_ops_driver.c``,
  the same way: they pin the numpy restatements in ``oracle/ops_oracle.py``.
* ``oracle/_ref/gptc_reference/`` the whole unmodified reference (libgpt.so with its own CUDA attention
  compiled for sm_100a, train_gpt, infer_gpt and the layer driver): the GPU baseline.  Compiled with the
  package's gpt.c build recipe (``gpt.c_b200/overlay/build_libgpt.py``), again only when the reference
  tree is present.

The reference tree is taken from ``GPTC_REFERENCE_DIR`` or, failing that, from a directory ``reference``
beside this repository.
Run as ``python oracle/build.py``; ``build_all()`` is what the package-level build calls.
The code is compiled for x86-64-v3 rather than for the building machine so the libraries still
load on a different host CPU.
"""
from __future__ import annotations

import glob
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
REF_DIR = os.environ.get("GPTC_REFERENCE_DIR") or os.path.join(ROOT, "..", "reference")
REF_OUT = os.path.join(HERE, "_ref")
ORACLE_SO = os.path.join(HERE, "liboracle.so")
REF_SO = os.path.join(REF_OUT, "libref_attention.so")
REF_OPS_SO = os.path.join(REF_OUT, "libref_ops.so")

CFLAGS = ["-O3", "-march=x86-64-v3", "-fopenmp", "-fPIC", "-shared", "-Wall", "-Wno-unused-result"]


def _newer(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def find_openblas() -> tuple[str, bool] | None:
    """Return (path, uses_scipy_prefix) of an LP64 OpenBLAS shared object, or None."""
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


def build_oracle(force: bool = False) -> str:
    src = os.path.join(HERE, "attention_oracle.c")
    if force or not _newer(ORACLE_SO, [src]):
        subprocess.check_call(["gcc", *CFLAGS, src, "-o", ORACLE_SO, "-lm"])
    return ORACLE_SO


def build_reference(force: bool = False) -> str | None:
    """Compile the reference CPU attention kernel out of tree.  None when it cannot be built."""
    srcs = [os.path.join(REF_DIR, "kernels/src/cpu/Attention.c"),
            os.path.join(REF_DIR, "kernels/src/cpu/Alloc.c")]
    if not all(os.path.exists(s) for s in srcs):
        return REF_SO if os.path.exists(REF_SO) else None
    blas = find_openblas()
    if blas is None:
        return None
    lib, scipy_prefix = blas
    driver = os.path.join(HERE, "ref_driver.c")
    if not force and _newer(REF_SO, srcs + [driver, os.path.join(HERE, "cblas.h")]):
        return REF_SO
    os.makedirs(REF_OUT, exist_ok=True)
    cmd = ["gcc", *CFLAGS, "-Wno-unknown-pragmas", "-Wno-attributes", "-Wno-discarded-qualifiers",
           "-I", HERE, "-I", os.path.join(REF_DIR, "include"), "-I", os.path.join(REF_DIR, "kernels/src")]
    if scipy_prefix:
        cmd.append("-DREF_BLAS_SCIPY")
    cmd += [driver, *srcs, "-o", REF_SO, lib, "-Wl,-rpath," + os.path.dirname(lib), "-lm"]
    subprocess.check_call(cmd)
    return REF_SO


def build_reference_ops(force: bool = False) -> str | None:
    """Compile the reference CPU kernels of Linear, LayerNorm, cross-entropy, AdamW and GELU out of tree."""
    srcs = [os.path.join(REF_DIR, "kernels/src/cpu", f + ".c") for f in ("Linear", "LayerNorm", "CrossEntropyLoss", "AdamW", "GeLU")]
    srcs.append(os.path.join(REF_DIR, "kernels/src/cpu/Alloc.c"))
    if not all(os.path.exists(s) for s in srcs):
        return REF_OPS_SO if os.path.exists(REF_OPS_SO) else None
    blas = find_openblas()
    if blas is None:
        return None
    lib, scipy_prefix = blas
    driver = os.path.join(HERE, "ref_ops_driver.c")
    if not force and _newer(REF_OPS_SO, srcs + [driver, os.path.join(HERE, "cblas.h")]):
        return REF_OPS_SO
    os.makedirs(REF_OUT, exist_ok=True)
    cmd = ["gcc", *CFLAGS, "-Wno-unknown-pragmas", "-Wno-attributes", "-Wno-discarded-qualifiers", "-Wno-unused-variable",
           "-I", HERE, "-I", os.path.join(REF_DIR, "include"), "-I", os.path.join(REF_DIR, "kernels/src")]
    if scipy_prefix:
        cmd.append("-DREF_BLAS_SCIPY")
    cmd += [driver, *srcs, "-o", REF_OPS_SO, lib, "-Wl,-rpath," + os.path.dirname(lib), "-lm"]
    subprocess.check_call(cmd)
    return REF_OPS_SO


def build_reference_gptc(force: bool = False) -> str | None:
    """The whole unmodified reference, CUDA attention included, as the GPU baseline.  None when the
    reference tree is absent and no earlier build exists."""
    out_dir = os.path.join(REF_OUT, "gptc_reference")
    exe = os.path.join(out_dir, "layer_driver")
    if not os.path.isdir(os.path.join(REF_DIR, "kernels", "src", "cuda")):
        return out_dir if os.path.exists(exe) else None
    if os.path.exists(exe) and not force:
        return out_dir
    import importlib.util

    spec = importlib.util.spec_from_file_location(
        "gptc_b200_overlay_build", os.path.join(ROOT, "gpt.c_b200", "overlay", "build_libgpt.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.build(os.path.abspath(REF_DIR), out_dir, overlay=False)


def build_all(force: bool = False, gptc: bool = False) -> dict:
    out = {"oracle": build_oracle(force), "reference": build_reference(force), "reference_ops": build_reference_ops(force)}
    if gptc:
        out["reference_gptc"] = build_reference_gptc(force)
    return out


if __name__ == "__main__":
    print(build_all(force="--force" in sys.argv, gptc=True))
