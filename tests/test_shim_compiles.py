"""CPU: the reference-side shim (include/strix_kernels_shim.cpp: strixite's kernel functions defined over the C ABI) must compile
against the reference's own headers - every forwarded declaration matched in name, argument types and order. Needs the
reference tree (STRIXITE_REFERENCE, default: a checkout named "reference" beside this repository); skipped where it is
absent. <hip/hip_runtime.h> is a stand-in (tests/stubs) since the check is syntax only."""
import os
import re
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.environ.get("STRIXITE_REFERENCE") or os.path.join(os.path.dirname(ROOT), "reference")
SHIM = os.path.join(ROOT, "include", "strix_kernels_shim.cpp")


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "kernels")) or shutil.which("g++") is None, reason="needs the reference tree and g++")
def test_shim_matches_the_reference_declarations():
    r = subprocess.run(["g++", "-std=c++20", "-fsyntax-only", "-Wall", "-Wextra", "-Werror", "-I", REF, "-I", os.path.join(ROOT, "include"),
                        "-I", os.path.join(ROOT, "tests", "stubs"), SHIM], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-4000:]


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "kernels")), reason="needs the reference tree")
def test_shim_defines_every_function_the_headers_declare():
    """Each function declared in the MoE-path headers (and the dense / tensor projections) has a definition in the shim."""
    headers = ["moe_router.hpp", "moe_grouped.hpp", "linear_q4.hpp", "linear_q5.hpp", "linear_q6.hpp", "linear_q8.hpp", "linear.hpp", "linear_wmma.hpp",
               "swiglu.hpp", "residual.hpp", "hc.hpp", "hc_wmma.hpp"]
    declared = set()
    for h in headers:
        text = re.sub(r"//[^\n]*", "", open(os.path.join(REF, "kernels", h)).read())
        declared |= set(re.findall(r"\b(?:void|size_t)\s+([a-z0-9_]+)\s*\(", text))
    shim = open(SHIM).read()
    expanded = set(re.findall(r"\b(?:void|size_t)\s+([a-z0-9_]+)\s*\(", shim))
    for bits in (4, 5):  # the macro-generated per-slot expert functions
        expanded |= {"linear_q%d_experts_%s" % (bits, k) for k in ("gather", "gather_swiglu", "combine")}
    expanded |= {m.group(1) for m in re.finditer(r"STRIX_SHIM_DENSE2?\((\w+),", shim)}
    missing = declared - expanded
    assert not missing, "the shim does not define %s" % sorted(missing)
