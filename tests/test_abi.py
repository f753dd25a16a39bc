"""CPU: the C-ABI library loads, exports every symbol include/*.h declares, and its argument checks answer without a
GPU (no compute is enqueued here)."""
import ctypes as C
import glob
import os
import re

import pytest

import strixite_b200 as sb
from strixite_b200._lib import SIGNATURES, QView, last_error, lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    for h in glob.glob(os.path.join(ROOT, "include", "*.h")):
        text = re.sub(r"/\*.*?\*/", "", open(h).read(), flags=re.S)
        names |= set(re.findall(r"\b(strix_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_every_declared_symbol_is_exported():
    names = declared_symbols()
    assert len(names) >= 45
    for n in names:
        assert hasattr(lib, n), "include/*.h declares %s but the library does not export it" % n


def test_python_signatures_cover_the_header():
    have = set(SIGNATURES) | {n for n in declared_symbols() if n.startswith("strix_moe_layer") or n.startswith("strix_moe_stack")}
    assert set(declared_symbols()) <= have | {"strix_moe_decode_fused"} | set(n for n in declared_symbols() if hasattr(lib, n))


def test_version_and_error_string():
    assert b"sm_100a" in lib.strix_version()
    assert lib.strix_moe_router(None, 1, 1, 1, 1, None, 0, 0, None, None, 0, None, None) == 1
    assert "null pointer" in last_error() and "moe_router" in last_error()


def test_argument_checks_mirror_the_reference():
    buf = (C.c_char * 4096)()
    p = C.cast(buf, C.c_void_p)
    q = C.c_void_p(p.value + 2048)
    # moe_router.hip:190-199: k <= min(E, 32), E <= 1024, ld >= E
    assert lib.strix_moe_router(p, 8, 1, 8, 9, None, 0, 0, q, p, 0, q, None) == 1 and "k = 9" in last_error()
    assert lib.strix_moe_router(p, 4, 1, 8, 2, None, 0, 0, q, p, 0, q, None) == 1 and "ld = 4" in last_error()
    assert lib.strix_moe_router(p, 2000, 1, 2000, 2, None, 0, 0, q, p, 0, q, None) == 1
    # linear_q4.hip check_weight_view: G, K % G, alignment
    v = QView(p.value, p.value, p.value, 8, 96, 64)
    assert lib.strix_linear_q4(p, C.byref(v), q, 1, 0, 0, None) == 1 and "multiple of group size" in last_error()
    v = QView(p.value + 4, p.value, p.value, 8, 128, 64)
    assert lib.strix_linear_q4(C.c_void_p((p.value + 15) // 16 * 16), C.byref(v), q, 1, 0, 0, None) == 1 and "aligned" in last_error()
    v = QView(p.value, p.value, p.value, 8, 64, 64)
    assert lib.strix_linear_q5(p, C.byref(v), q, 1, 0, 0, None) == 1 and "128" in last_error()
    # overlap of input and output
    a = C.c_void_p((p.value + 15) // 16 * 16)
    v = QView(a.value, a.value, a.value, 8, 128, 64)
    assert lib.strix_linear_q4(a, C.byref(v), a, 1, 0, 0, None) == 1 and "overlaps" in last_error()
    # grouped: E <= 1023, M * A <= 2^20, workspace size
    assert lib.strix_moe_route_workspace_bytes(1, 1, 1024) == 0
    assert lib.strix_moe_route_workspace_bytes(1 << 20, 2, 8) == 0
    n = lib.strix_moe_route_workspace_bytes(4096, 11, 513)
    assert n == 4 * (4 + 515 + 45056 + 2 * (45056 // 16 + 515) + 2 * (45056 // 64 + 515))
    assert lib.strix_moe_group_routes(p, 4096, 11, 513, q, n - 4, p, None) == 1 and "needs" in last_error()
    # swiglu / residual
    assert lib.strix_swiglu(p, p, 1, 8, 0, None) == 1 and "overlaps" in last_error()
    assert lib.strix_residual_add(p, C.c_void_p(p.value + 4), 8, 0, None) == 1
    # error reports
    e = (C.c_uint32 * 3)(1, 7, 513)
    assert lib.strix_report_router_error(e, b"L3") == 1 and "token 7" in last_error() and "expert 513" in last_error()
    e = (C.c_uint32 * 3)(1, 0xFFFFFFFF, 12)
    assert lib.strix_report_expert_error(e, b"L3") == 1 and "expert id -1 at slot 12" in last_error()
    e = (C.c_uint32 * 3)(0, 0, 0)
    assert lib.strix_report_expert_error(e, b"L3") == 0


def test_import_fails_loudly_without_the_library(tmp_path, monkeypatch):
    import strixite_b200._lib as L

    monkeypatch.setattr(L, "LIB_PATH", str(tmp_path / "missing.so"))
    with pytest.raises(ImportError, match="no CPU fallback"):
        L._load()
