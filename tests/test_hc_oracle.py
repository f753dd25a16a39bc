"""CPU: the hyper-connection bracket's oracle (oracle.hc_mix_down / hc_mix_up / to_chunk_major) against an independent
float64 numpy formulation of strixite kernels/hc.hpp:29-50, and the chunk-major layout against the reference's own
to_chunk_major (when the reference's formats are built) and the library's host function."""
import numpy as np
import pytest

import oracle
from helpers import quantized, randn_act
from strixite_b200 import kernels as K

H = 4


def act_f64(x):
    return (oracle.bf16_to_f32(x) if x.dtype == np.uint16 else x).astype(np.float64)


def numpy_down(x, w, d, r, inject, eps):
    X = act_f64(x)
    W = oracle.dequantize(w).astype(np.float64)
    T = X.shape[0]
    Xs = X.reshape(T, H, d)
    inv = 1.0 / np.sqrt((Xs * Xs).mean(axis=2) + eps)
    a = np.einsum("nsj,tsj,ts->tn", W.reshape(-1, H, d), Xs, inv) / H
    h = a[:, :r] / (1.0 + np.exp(-a[:, :r]))
    w_in = 2.0 / (1.0 + np.exp(-a[:, r:])) if inject else None
    return h, w_in, inv


def numpy_up(h, w_up, x, norm_w, inv, d):
    X = act_f64(x)
    T = X.shape[0]
    W = oracle.dequantize(w_up).astype(np.float64)
    z = 1.0 / (1.0 + np.exp(-(h.astype(np.float64) @ W.T)))
    n = X.reshape(T, H, d) * inv.astype(np.float64)[:, :, None] * (1.0 + norm_w.astype(np.float64)).reshape(1, H, d)
    return (z.reshape(T, H, d) * n).sum(axis=1) / H


@pytest.mark.parametrize("bits", (4, 8))
@pytest.mark.parametrize("act", (oracle.F32, oracle.BF16))
@pytest.mark.parametrize("inject", (True, False))
def test_mix_down_matches_the_float64_formula(bits, act, inject):
    rng = np.random.default_rng(7 * bits + act + 2 * inject)
    T, d, r = 5, 96, 40
    x = randn_act(rng, (T, H * d), act)
    w = quantized(rng, bits, r + (H if inject else 0), H * d, 32, sigma=0.05)
    h, w_in, inv = oracle.hc_mix_down(x, w, H, d, r, inject, 1e-6)
    rh, rw, rinv = numpy_down(x, w, d, r, inject, 1e-6)
    assert np.abs(inv - rinv).max() <= 2e-6 * np.abs(rinv).max()
    assert np.abs(h - rh).max() <= 2e-6 * max(np.abs(rh).max(), 1.0)
    if inject:
        assert np.abs(w_in - rw).max() <= 2e-6 * 2.0
    else:
        assert w_in is None


@pytest.mark.parametrize("bits", (4, 8))
@pytest.mark.parametrize("G", (32, 64))
def test_chunk_major_layout(bits, G):
    rng = np.random.default_rng(bits + G)
    w = quantized(rng, bits, 24, 128, G)
    cm = oracle.to_chunk_major(w)
    cb = 32 * bits // 8
    q = w.q.reshape(w.N, w.K // 32, cb)
    assert np.array_equal(cm.q.reshape(w.K // 32, w.N, cb), q.transpose(1, 0, 2))
    assert np.array_equal(cm.scale.reshape(w.K // G, w.N), w.scale.reshape(w.N, -1).T)
    assert np.array_equal(cm.minv.reshape(w.K // G, w.N), w.minv.reshape(w.N, -1).T)
    pq, ps, pm = K.to_chunk_major(bits, w.q, w.scale, w.minv, w.N, w.K, w.G)  # the library's host function
    assert np.array_equal(pq, cm.q) and np.array_equal(ps.ravel(), cm.scale.ravel()) and np.array_equal(pm.ravel(), cm.minv.ravel())
    if oracle.ref is not None and hasattr(oracle.ref, "ref_to_chunk_major"):
        rf = oracle.ref_to_chunk_major(w)
        assert np.array_equal(rf.q, cm.q) and np.array_equal(rf.scale.ravel(), cm.scale.ravel()) and np.array_equal(rf.minv.ravel(), cm.minv.ravel())


@pytest.mark.parametrize("bits", (4, 8))
@pytest.mark.parametrize("act", (oracle.F32, oracle.BF16))
def test_mix_up_matches_the_float64_formula(bits, act):
    rng = np.random.default_rng(11 * bits + act)
    T, d, r = 3, 40, 64
    x = randn_act(rng, (T, H * d), act)
    h = rng.standard_normal((T, r)).astype(np.float32)
    w_up = quantized(rng, bits, H * d, r, 32, sigma=0.2)
    norm_w = (rng.standard_normal(H * d) * 0.1).astype(np.float32)
    inv = (0.5 + rng.random((T, H))).astype(np.float32)
    u = oracle.hc_mix_up(h, oracle.to_chunk_major(w_up), x, norm_w, inv, H, d)
    ref = numpy_up(h, w_up, x, norm_w, inv, d)
    got = act_f64(u)
    tol = 2e-6 if act == oracle.F32 else 2.0 ** -8
    assert np.abs(got - ref).max() <= tol * np.abs(ref).max()
