"""Stages the reference's own kernels for the GPU-side comparison.

    python baseline/prepare_ref.py /path/to/reference   (or set PYPTX_REFERENCE_DIR)

Copies the reference's ``pyptx/`` package and ``examples/`` tree into ``baseline/_ref/`` (a
git-ignored folder that still travels to the GPU box) and builds its launch shim there with
``g++ -DPYPTX_NO_XLA_FFI`` (the reference's own fallback build, pyptx/_shim/auto_build.py:52-68),
because the shim is written next to its source and the reference tree is read-only.  Nothing is
modified; ``baseline/run_pyptx.py`` imports the copy with ``baseline/jax_stub`` on the path.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")


def main() -> int:
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("PYPTX_REFERENCE_DIR", "")
    if not ref:
        print("usage: prepare_ref.py <reference tree>  (or set PYPTX_REFERENCE_DIR); nothing staged")
        return 0
    if not os.path.isdir(os.path.join(ref, "pyptx")):
        print(f"no reference tree at {ref}; nothing staged")
        return 0
    os.makedirs(DEST, exist_ok=True)
    for sub in ("pyptx", "examples"):
        dst = os.path.join(DEST, sub)
        if os.path.isdir(dst):
            shutil.rmtree(dst)
        shutil.copytree(os.path.join(ref, sub), dst, ignore=shutil.ignore_patterns("__pycache__", "*.pyc", "*.so"))
    shim_dir = os.path.join(DEST, "pyptx", "_shim")
    so = os.path.join(shim_dir, "libpyptx_shim.so")
    # The reference's own Torch-only recipe plus a force-included two-line header (see xla_ns_stub.h);
    # the reference source is compiled as it is.
    cmd = ["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-DPYPTX_NO_XLA_FFI",
           "-include", os.path.join(HERE, "xla_ns_stub.h"),
           os.path.join(shim_dir, "pyptx_launch.cc"), "-o", so, "-ldl"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        print("shim build failed:\n" + r.stderr[-2000:])
        return 1
    print(f"staged {DEST} (shim: {so})")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
