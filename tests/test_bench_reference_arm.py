"""CPU: `bench.py --impl reference` - the timed CPU arm - prints one JSON line with the contract's keys and never loads the
CUDA library (the arm must not route through the product)."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

RUNNER = r"""
import io, json, os, sys
sys.argv = ["bench.py", "--impl", "reference", "--workload", "decode1", "--steps", "2", "--warmup", "1"]
sys.path.insert(0, %r)
import bench
bench.main()
maps = open("/proc/self/maps").read()
loaded = "libstrixite_b200" in maps or any(m.startswith("strixite_b200") for m in sys.modules)
sys.stderr.write("PRODUCT_LOADED=%%d\n" %% loaded)
"""


def test_reference_arm_prints_the_contract_line_without_the_product_library():
    r = subprocess.run([sys.executable, "-c", RUNNER % ROOT], capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1, "exactly one line on stdout, got %d" % len(lines)
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "MoE-layer tokens/s" and d["unit"] == "tokens/s" and d["higher_is_better"] is True
    assert d["value"] > 0 and d["ms_per_step"] > 0 and d["gpu_launches"] == 0
    assert d["config"]["workload"] == "decode1"
    cb = d["cpu_baseline"]
    assert cb["kind"] in ("port", "reference") and cb["cores"] >= 1 and cb["value"] == d["value"] and cb["sample"]
    assert d["e2e"] == dict(value=d["value"], unit="tokens/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0)
    assert "PRODUCT_LOADED=0" in r.stderr
