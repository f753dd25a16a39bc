"""CPU: the in-tree invariants of the layer arithmetic, asserted on the oracle (strixite ships no layer goldens), and
the timed CPU baseline against the double-accumulating oracle."""
import numpy as np
import pytest

import oracle
from helpers import make_layer, make_stack, quantized, randn_act, rel_err_rows


def test_router_picks_topk_and_renormalizes():
    rng = np.random.default_rng(0)
    for E, k in ((1, 1), (31, 5), (32, 32), (33, 10), (512, 10), (1024, 32)):
        logits = rng.standard_normal((7, E + 1)).astype(np.float32)
        ids, coef, err = oracle.moe_router(logits, E, k, shared_col=E, shared_id=E)
        assert err[0] == 0
        order = np.argsort(-logits[:, :E], axis=1, kind="stable")[:, :k]
        assert np.array_equal(ids[:, :k], order.astype(np.int32))
        assert np.allclose(coef[:, :k].sum(1), 1.0, atol=1e-6)
        sm = np.exp(logits[:, :E] - logits[:, :E].max(1, keepdims=True))
        sel = np.take_along_axis(sm, order, 1)
        assert np.allclose(coef[:, :k], sel / sel.sum(1, keepdims=True), rtol=1e-5)
        assert np.all(ids[:, k] == E) and np.allclose(coef[:, k], 1 / (1 + np.exp(-logits[:, E])), rtol=1e-6)


def test_router_ties_go_to_lower_index():
    logits = np.zeros((2, 64), np.float32)
    logits[1, [5, 40, 41]] = 1.0
    ids, coef, _ = oracle.moe_router(logits, 64, 4)
    assert ids[0].tolist() == [0, 1, 2, 3] and ids[1].tolist() == [5, 40, 41, 0]
    assert np.allclose(coef[0], 0.25)


def test_router_nonfinite_fails_the_token():
    logits = np.random.default_rng(1).standard_normal((3, 17)).astype(np.float32)
    logits[1, 9] = np.nan
    logits[1, 4] = np.inf
    logits[2, 16] = -np.inf  # the shared gate
    ids, coef, err = oracle.moe_router(logits, 16, 3, shared_col=16, shared_id=16)
    assert err.tolist() == [1, 1, 4]
    assert np.all(ids[1] == -1) and np.all(np.isnan(coef[1])) and np.all(ids[2] == -1)
    assert ids[0, 3] == 16 and np.all(ids[0, :3] >= 0)


def test_group_routes_layout_and_stability():
    rng = np.random.default_rng(2)
    M, A, E = 37, 5, 19
    ids = rng.integers(0, E, (M, A)).astype(np.int32)
    ids[3, 2], ids[20, 0] = -1, E + 4
    ws, err = oracle.group_routes(ids, E)
    S = M * A
    assert err.tolist() == [1, 0xFFFFFFFF, 3 * A + 2]
    assert ws[1] == S and ws[2] == E
    off = ws[4 : 4 + E + 2]
    slots = ws[4 + E + 2 : 4 + E + 2 + S]
    assert off[0] == 0 and off[E + 1] == S and np.all(np.diff(off) >= 0)
    assert sorted(slots.tolist()) == list(range(S))
    flat = ids.reshape(-1)
    for b in range(E + 1):
        seg = slots[off[b] : off[b + 1]]
        assert np.all(np.diff(seg) > 0)  # ascending inside a bucket: the stable order
        want = [s for s in range(S) if (flat[s] == b if b < E else (flat[s] < 0 or flat[s] >= E))]
        assert seg.tolist() == want
    Tmax = S // 16 + E + 2
    tb = ws[4 + E + 2 + S : 4 + E + 2 + S + Tmax][: ws[0]]
    ts = ws[4 + E + 2 + S + Tmax : 4 + E + 2 + S + 2 * Tmax][: ws[0]]
    assert ws[0] == sum((off[b + 1] - off[b] + 15) // 16 for b in range(E + 1))
    for b, s in zip(tb, ts):
        assert off[b] <= s < off[b + 1] and (s - off[b]) % 16 == 0


@pytest.mark.parametrize("act", (oracle.F32, oracle.BF16))
def test_fused_gather_swiglu_equals_gather_then_swiglu(act):
    # strixite kernels/linear_q4.hpp:53-54: bit-identical.
    rng = np.random.default_rng(3)
    st = make_stack(rng, 6, 64, 128, 32, bits=5)
    x = randn_act(rng, (3, 128), act)
    ids = rng.integers(0, 6, (3, 2)).astype(np.int32)
    fused, _ = oracle.experts_gather(x, st, ids, swiglu=True)
    gu, _ = oracle.experts_gather(x, st, ids, swiglu=False)
    assert np.array_equal(fused.reshape(6, 32), oracle.swiglu(gu, 32))


def test_bad_expert_id_poisons_and_flags():
    rng = np.random.default_rng(4)
    st = make_stack(rng, 4, 32, 64, 32)
    x = randn_act(rng, (2, 64), oracle.F32)
    ids = np.array([[0, 9], [1, 2]], np.int32)
    y, err = oracle.experts_gather(x, st, ids)
    assert err.tolist() == [1, 9, 1] and np.all(np.isnan(y[0, 1])) and not np.isnan(y[1]).any()
    h = randn_act(rng, (2, 2, 64), oracle.F32)
    yc, err = oracle.experts_combine(h, st, ids, np.ones((2, 2), np.float32))
    assert err.tolist() == [1, 9, 1] and np.all(np.isnan(yc[0])) and not np.isnan(yc[1]).any()


def test_shared_add_inject_equals_add_then_inject():
    # strixite kernels/moe_router.hpp:56-60, and the tutorial's CPU reference (tutorial/first-kernel/first_kernel.hip:52-61):
    # x[t, s, c] = fma(w[t, s], moe + shared, x) when the gate is open (sigmoid -> 1 for a large logit).
    rng = np.random.default_rng(5)
    M, N = 3, 40
    for act in (oracle.F32, oracle.BF16):
        y0, s = randn_act(rng, (M, N), act), randn_act(rng, (M, N), act)
        gl = rng.standard_normal((M, 3)).astype(np.float32)
        x0, w_in = randn_act(rng, (M, 4 * N), act), rng.standard_normal((M, 4)).astype(np.float32)
        ya, xa = y0.copy(), x0.copy()
        oracle.moe_shared_add_inject(ya, s, gl, 1, 9, xa, w_in)
        yb, xb = y0.copy(), x0.copy()
        oracle.moe_shared_add(yb, s, gl, 1, 9)
        oracle.hc_inject(xb, yb, w_in)
        assert np.array_equal(ya, yb) and np.array_equal(xa, xb)
    moe, sh = randn_act(rng, (M, N), oracle.F32), randn_act(rng, (M, N), oracle.F32)
    x, w_in = randn_act(rng, (M, 4 * N), oracle.F32), rng.standard_normal((M, 4)).astype(np.float32)
    want = x.copy().reshape(M, 4, N)
    for t in range(M):
        for st in range(4):
            want[t, st] = np.float32(w_in[t, st]) * (moe[t] + sh[t]) + want[t, st]
    y = moe.copy()
    oracle.moe_shared_add_inject(y, sh, np.full((M, 1), 100.0, np.float32), 0, 0, x, w_in)
    assert np.allclose(x.reshape(M, 4, N), want, rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("act", (oracle.F32, oracle.BF16))
def test_cpu_baseline_agrees_with_oracle(act):
    L = make_layer(11, d=256, I=64, E=16, k=4, G=64, router="bf16", shared="separate")
    x = randn_act(np.random.default_rng(12), (9, 256), act)
    y, it = oracle.moe_layer(x, L)
    yf, itf = oracle.moe_layer(x, L, use_fast=True)
    assert np.array_equal(it["ids"], itf["ids"])
    tol = 1e-4 if act == oracle.F32 else 2e-3 + 2.0 ** -8
    assert rel_err_rows(oracle.to_f32(yf), oracle.to_f32(y)) < tol


def test_mixed_format_layer_runs():
    L = make_layer(13, d=256, I=128, E=8, k=2, G=128, shared="stacked", mix=[0.6, 0.15, 0.15, 0.1])
    x = randn_act(np.random.default_rng(14), (2, 256), oracle.F32)
    y, it = oracle.moe_layer(x, L)
    assert np.isfinite(y).all() and it["ids"].shape == (2, 3)
    assert rel_err_rows(oracle.moe_layer(x, L, use_fast=True)[0], y) < 1e-4
