"""Generates tests/golden/demo.strixw and tests/golden/strixw_hashes.json from the REFERENCE's own strixw writer and hash
(strixite formats/strixw.cpp, compiled unchanged by oracle/build.py into oracle/_ref/). Run where the reference tree is
mounted:

    python oracle/build.py && python tests/golden/make_golden_strixw.py

demo.strixw is written by the reference's StrixwWriter through oracle/ref_strixw_shim.cpp (one tensor of every row-major
encoding the MoE path loads, an expert stack with parts, metadata; component bytes from a seeded xorshift the tests
restate). strixw_hashes.json holds strix_hash64 of seeded byte strings of assorted lengths.
"""
import ctypes as C
import json
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
SEED = 7


def main():
    ref = C.CDLL(os.path.join(HERE, "..", "..", "oracle", "_ref", "libstrix_formats_ref.so"))
    ref.ref_hash64.restype, ref.ref_hash64.argtypes = C.c_uint64, [C.c_void_p, C.c_uint64]
    ref.ref_strixw_last_error.restype = C.c_char_p
    path = os.path.join(HERE, "demo.strixw")
    if ref.ref_strixw_write_demo(path.encode(), C.c_uint64(SEED)) != 0:
        raise SystemExit(ref.ref_strixw_last_error().decode())
    hashes = {}
    rng = np.random.default_rng(2026)
    for n in (0, 1, 7, 8, 9, 31, 32, 33, 40, 63, 64, 100, 255, 4096, 4099):
        b = rng.integers(0, 256, n, dtype=np.uint8)
        hashes[str(n)] = dict(seed=2026, hash="%016x" % ref.ref_hash64(b.ctypes.data_as(C.c_void_p), n), first=b[:4].tolist())
    json.dump(dict(note="byte strings are drawn in this order from numpy default_rng(2026).integers(0, 256, n, uint8)", cases=hashes),
              open(os.path.join(HERE, "strixw_hashes.json"), "w"), indent=1)
    print("wrote", path, os.path.getsize(path), "bytes and strixw_hashes.json")


if __name__ == "__main__":
    main()
