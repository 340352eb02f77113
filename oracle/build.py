"""Build recipe for the CPU checkers.  TEST INFRASTRUCTURE ONLY.

Two shared libraries are produced:

* ``oracle/liboracle.so`` from ``oracle/attention_oracle.c`` (the plain-C restatement), always;
* ``oracle/_ref/libref_attention.so`` from the reference's own CPU attention sources compiled
  where they lie in the reference tree (``kernels/src/cpu/Attention.c``, ``kernels/src/cpu/Alloc.c``)
  plus ``oracle/ref_driver.c``, linked against an LP64 OpenBLAS found in the Python environment.
  This one is built only when the reference tree is present; the reference's own build system is
  not run and no reference source is copied.

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
REF_DIR = os.environ.get("GPTC_REFERENCE_DIR", "/root/reference")
REF_OUT = os.path.join(HERE, "_ref")
ORACLE_SO = os.path.join(HERE, "liboracle.so")
REF_SO = os.path.join(REF_OUT, "libref_attention.so")

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


def build_all(force: bool = False) -> dict:
    return {"oracle": build_oracle(force), "reference": build_reference(force)}


if __name__ == "__main__":
    print(build_all(force="--force" in sys.argv))
