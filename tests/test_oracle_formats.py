"""CPU: the oracle's quantizer restatement and the product's host quantizer against the reference's own quantizers -
the committed golden vectors (made by tests/golden/make_golden.py from strixite formats/q*.cpp) and, when the compiled
reference library travels with the checkout (oracle/_ref), fresh random cases."""
import os

import numpy as np
import pytest

import oracle
from strixite_b200 import StrixError
from strixite_b200 import kernels as K

GOLD = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "formats_ref.npz"))
CASES = [(b, g) for b in (4, 5, 6, 8) for g in (32, 64, 128)]


@pytest.mark.parametrize("bits,G", CASES)
def test_oracle_matches_golden(bits, G):
    n = "q%d_g%d" % (bits, G)
    qw = oracle.quantize(bits, GOLD[n + ".w"], G)
    assert np.array_equal(qw.q, GOLD[n + ".q"])
    assert np.array_equal(qw.scale, GOLD[n + ".scale"]) and np.array_equal(qw.minv, GOLD[n + ".minv"])
    assert np.array_equal(oracle.dequantize(qw).view(np.uint32), GOLD[n + ".deq"].view(np.uint32))


@pytest.mark.parametrize("bits,G", CASES)
def test_product_host_quantizer_matches_golden(bits, G):
    n = "q%d_g%d" % (bits, G)
    w = GOLD[n + ".w"]
    q, s, m = K.quantize(w, bits, G)
    assert np.array_equal(q, GOLD[n + ".q"]) and np.array_equal(s, GOLD[n + ".scale"]) and np.array_equal(m, GOLD[n + ".minv"])
    deq = K.dequantize(bits, q, s, m, w.shape[0], w.shape[1], G)
    assert np.array_equal(deq.view(np.uint32), GOLD[n + ".deq"].view(np.uint32))


def test_golden_edge_cases_present():
    # constant group -> scale bits 0 and codes 0 (formats/q4.cpp:73-76)
    s = GOLD["q4_g32.scale"]
    assert s[1, 0] == 0 and not GOLD["q4_g32.q"][256 // 2 : 256 // 2 + 16].any()


@pytest.mark.skipif(oracle.ref is None, reason="oracle/_ref (the compiled reference quantizers) is not present")
@pytest.mark.parametrize("bits,G", CASES)
def test_oracle_matches_reference_library(bits, G):
    rng = np.random.default_rng(bits * 7 + G)
    for sigma in (0.02, 1.0, 300.0):
        w = (rng.standard_normal((5, 384)) * sigma).astype(np.float32)
        a, b = oracle.quantize(bits, w, G), oracle.ref_quantize(bits, w, G)
        assert np.array_equal(a.q, b.q) and np.array_equal(a.scale, b.scale) and np.array_equal(a.minv, b.minv)
        assert np.array_equal(oracle.dequantize(a).view(np.uint32), oracle.ref_dequantize(b).view(np.uint32))
        q, s, m = K.quantize(w, bits, G)
        assert np.array_equal(q, b.q) and np.array_equal(s, b.scale) and np.array_equal(m, b.minv)


@pytest.mark.skipif(oracle.ref is None, reason="oracle/_ref is not present")
def test_reference_rejects_what_we_reject():
    w = np.zeros((2, 96), np.float32)
    for bits, G, Kdim in ((4, 48, 96), (4, 64, 96), (5, 32, 96), (6, 32, 96)):
        ww = np.zeros((2, Kdim), np.float32)
        with pytest.raises(ValueError):
            oracle.ref_quantize(bits, ww, G)
        assert oracle.quantize_rc(bits, ww, G) != 0
        with pytest.raises(StrixError):
            K.quantize(ww, bits, G)
    w[0, 3] = np.inf
    with pytest.raises(ValueError):
        oracle.ref_quantize(4, w, 32)
    assert oracle.quantize_rc(4, w, 32) == -5
    with pytest.raises(StrixError, match="non-finite"):
        K.quantize(w, 4, 32)


def test_q4_from_q8_golden():
    # formats/q4_from_q8.hpp: dequantize the Q8 rows exactly, then quantize as Q4.
    w = GOLD["q4_from_q8.w"]
    q8 = oracle.quantize(8, w, 64)
    q4 = oracle.quantize(4, oracle.dequantize(q8), 128)
    assert np.array_equal(q4.q, GOLD["q4_from_q8.q"]) and np.array_equal(q4.scale, GOLD["q4_from_q8.scale"])
    assert np.array_equal(q4.minv, GOLD["q4_from_q8.minv"])


@pytest.mark.parametrize("bits", (4, 5, 6, 8))
def test_append_rows_is_exact(bits):
    # formats/q4.hpp:35-38: quantizing row chunks and concatenating == quantizing the whole matrix.
    rng = np.random.default_rng(bits)
    w = (rng.standard_normal((9, 256)) * 0.02).astype(np.float32)
    whole = K.quantize(w, bits, 64)
    parts = [K.quantize(w[a:b], bits, 64) for a, b in ((0, 4), (4, 5), (5, 9))]
    for i in range(3):
        assert np.array_equal(np.concatenate([p[i] for p in parts]), whole[i])


def test_codes_in_range_and_roundtrip_error():
    rng = np.random.default_rng(5)
    w = (rng.standard_normal((8, 512)) * 0.02).astype(np.float32)
    for bits in (4, 5, 6, 8):
        qw = oracle.quantize(bits, w, 128)
        deq = oracle.dequantize(qw)
        step = oracle.bf16_to_f32(qw.scale).repeat(128, axis=1)
        assert np.all(np.abs(deq - w) <= 0.5 * step * 1.02 + 2.0 ** -8 * np.abs(w).max())


def test_bf16_conversion():
    a = np.array([0.0, -0.0, 1.0, 1.00390625, 1.01171875, np.inf, -np.inf, np.nan, 3.3895314e38], np.float32)
    b = oracle.f32_to_bf16(a)
    for x, y in zip(a, b):
        assert int(y) == int(oracle.orc.orc_f32_to_bf16(float(x))) or np.isnan(x)
    assert b[3] == 0x3F80 and b[4] == 0x3F82  # ties to even, both directions
    assert (b[7] & 0x7FC0) == 0x7FC0  # NaN stays a quiet NaN
