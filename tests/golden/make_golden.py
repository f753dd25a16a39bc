"""Generates tests/golden/formats_ref.npz from the REFERENCE's own quantizers (strixite formats/q{4,5,6,8}.cpp and
q4_from_q8.cpp, compiled unchanged by oracle/build.py into oracle/_ref/). Run where the reference tree is mounted:

    python oracle/build.py && python tests/golden/make_golden.py

The fixture holds, per case, the FP32 input and the reference's codes, scales, mins and dequantized values; the
tests check the CPU restatement (and, on a GPU, the CUDA quantizer) against it bit for bit.
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
import oracle  # noqa: E402


def cases():
    """(name, bits, G, w[N, K]) - seeded; includes constant groups (scale 0), half-way ties, wide ranges, negatives."""
    out = []
    for bits in (4, 5, 6, 8):
        for G in (32, 64, 128):
            rng = np.random.default_rng(1000 * bits + G)
            K = 256
            w = (rng.standard_normal((6, K)) * 0.02).astype(np.float32)
            w[1, :G] = 0.25                      # constant group: s == 0, codes 0
            w[2, :] = np.linspace(-1.0, 1.0, K, dtype=np.float32)          # evenly spaced: exact half-way ties
            w[3, :] = (rng.standard_normal(K) * 3e4).astype(np.float32)    # wide range
            w[4, :] = np.abs(w[4, :]) + 1.0      # all positive, offset
            w[5, G:2 * G] = np.float32(-0.0)     # signed zeros in a constant group
            out.append(("q%d_g%d" % (bits, G), bits, G, w))
    return out


def main():
    assert oracle.ref is not None, "oracle/_ref is not built (python oracle/build.py with the reference mounted)"
    blob = {}
    for name, bits, G, w in cases():
        qw = oracle.ref_quantize(bits, w, G)
        blob[name + ".w"] = w
        blob[name + ".q"] = qw.q
        blob[name + ".scale"] = qw.scale
        blob[name + ".minv"] = qw.minv
        blob[name + ".deq"] = oracle.ref_dequantize(qw)
    # Q8 -> Q4 requantization (formats/q4_from_q8.hpp), 1 and 3 worker threads must agree.
    rng = np.random.default_rng(77)
    w = (rng.standard_normal((10, 256)) * 0.02).astype(np.float32)
    q8 = oracle.ref_quantize(8, w, 64)
    q4a, q4b = oracle.ref_q4_from_q8(q8, 128, 1), oracle.ref_q4_from_q8(q8, 128, 3)
    assert np.array_equal(q4a.q, q4b.q) and np.array_equal(q4a.scale, q4b.scale)
    blob["q4_from_q8.w"] = w
    blob["q4_from_q8.q"], blob["q4_from_q8.scale"], blob["q4_from_q8.minv"] = q4a.q, q4a.scale, q4a.minv
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "formats_ref.npz")
    np.savez_compressed(path, **blob)
    print("wrote", path, os.path.getsize(path), "bytes,", len(blob), "arrays")


if __name__ == "__main__":
    main()
