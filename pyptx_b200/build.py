"""``python -m pyptx_b200.build [--force] [--verbose] [--ptxas-info]``: compile the C-ABI library."""
import argparse

from . import _native

if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--ptxas-info", action="store_true", help="print registers / spills / shared memory per kernel")
    a = ap.parse_args()
    print(_native.build(force=a.force, verbose=a.verbose, ptxas_info=a.ptxas_info))
    print(_native.build_torch_ext(force=a.force))
