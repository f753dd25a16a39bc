"""Builds the checker libraries (test infrastructure, not product code).

  oracle/liboracle.so            moe_oracle.cpp  - the double-accumulating CPU restatement (-O2, no FMA contraction)
  oracle/liboracle_fast.so       moe_baseline.cpp - the timed multi-threaded CPU baseline (-O3 -march=native, OpenMP)
  oracle/_ref/libstrix_formats_ref.so   the REFERENCE's formats/q*.cpp compiled unchanged from the reference tree
                                 (only when that tree is mounted; the built file is git-ignored and travels with
                                 the working copy)

Run:  python oracle/build.py [--reference /path/to/strixite]
"""
import argparse
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
# The strixite source tree: STRIXITE_REFERENCE, or a checkout named "reference" beside this repository.
DEFAULT_REF = os.environ.get("STRIXITE_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def _run(cmd):
    print("+", " ".join(cmd), flush=True)
    subprocess.check_call(cmd)


def _stale(out, srcs):
    if not os.path.exists(out):
        return True
    t = os.path.getmtime(out)
    return any(os.path.getmtime(s) > t for s in srcs)


def build(reference=DEFAULT_REF, force=False):
    out = os.path.join(HERE, "liboracle.so")
    src = os.path.join(HERE, "moe_oracle.cpp")
    if force or _stale(out, [src]):
        # -ffp-contract=off: dequantize is "q*s then +m, each rounded separately" (formats/q4.cpp:121-124).
        _run(["g++", "-std=c++17", "-O2", "-ffp-contract=off", "-fPIC", "-shared", src, "-o", out])
    out = os.path.join(HERE, "liboracle_fast.so")
    src = os.path.join(HERE, "moe_baseline.cpp")
    if force or _stale(out, [src]):
        _run(["g++", "-std=c++17", "-O3", "-march=native", "-fopenmp", "-fPIC", "-shared", src, "-o", out])
    ref_dir = os.path.join(HERE, "_ref")
    out = os.path.join(ref_dir, "libstrix_formats_ref.so")
    fmts = [os.path.join(reference, "formats", f + ".cpp") for f in ("q4", "q5", "q6", "q8", "q4_from_q8", "strixw")]
    if all(os.path.exists(f) for f in fmts):
        shims = [os.path.join(HERE, "ref_shim.cpp"), os.path.join(HERE, "ref_strixw_shim.cpp")]
        if force or _stale(out, fmts + shims):
            os.makedirs(ref_dir, exist_ok=True)
            # The reference's own sources, compiled where they lie: no -march/-mfma (keeps q*s+m unfused), C++20.
            _run(["g++", "-std=c++20", "-O2", "-ffp-contract=off", "-Wno-unknown-pragmas", "-pthread", "-fPIC",
                  "-shared", "-I", reference] + fmts + shims + ["-o", out])
    elif not os.path.exists(out):
        print("oracle/build.py: reference tree not mounted at %s and no prebuilt oracle/_ref - the reference-"
              "quantizer checks will be skipped" % reference, file=sys.stderr)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=DEFAULT_REF)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    build(a.reference, a.force)
