"""Byte-compiles the reference's own CPU checker for the timed CPU leg of bench.py.  Test/measurement
infrastructure only: nothing in the product path loads what this makes.

The source -- `test/reference.py` of a checkout of SSIGPRO/mamtorch (26 lines of plain torch:
`fullyconnected_reference`, `fullyconnected_backward_reference`) -- is compiled where it lies; it is not
copied.  The output, oracle/_ref/reference_checker.bin, is a build product like the shared objects beside it: it
stays out of version control and travels with the built tree, so that `bench.py --impl reference` and the
`cpu_baseline` leg can time the reference's unmodified CPU path (kind "reference") on a machine that has
no checkout.  Where the file is missing, or was compiled by another Python version, bench.py falls back
to the restatement in oracle/mam_oracle.py (kind "port").

    python oracle/build_ref_py.py [--reference DIR]
"""
from __future__ import annotations

import argparse
import os
import py_compile
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref", "reference_checker.bin")


def build(ref: str | None = None) -> str | None:
    ref = ref or os.environ.get("MAMTORCH_REFERENCE_DIR", "")
    src = os.path.join(ref, "test", "reference.py") if ref else ""
    if not src or not os.path.isfile(src):
        return None
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    py_compile.compile(src, cfile=OUT, dfile="test/reference.py", doraise=True)
    return OUT


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=None, help="checkout of the reference (or MAMTORCH_REFERENCE_DIR)")
    out = build(ap.parse_args().reference)
    if out is None:
        sys.exit("no reference checkout given: pass --reference DIR")
    print(out)
