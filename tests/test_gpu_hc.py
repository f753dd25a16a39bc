"""GPU: hc_mix_down / hc_mix_up (strixite kernels/hc.hpp:29-50) through the C ABI against the CPU oracle."""
import numpy as np
import pytest
import torch

import oracle
from helpers import BF16_ULP, quantized, randn_act, to_np_act, to_torch_act, upload
from strixite_b200 import StrixError
from strixite_b200 import kernels as K

pytestmark = pytest.mark.gpu

H = 4
# FP32 chains in a different order than the oracle's double sums (K up to 4 * 512 terms).
TOL = 3e-5


def run_down(x, w, d, r, inject, eps=1e-6):
    T = x.shape[0]
    h = torch.full((T, r), float("nan"), device="cuda")
    w_in = torch.full((T, H), float("nan"), device="cuda") if inject else None
    inv = torch.full((T, H), float("nan"), device="cuda")
    K.hc_mix_down(to_torch_act(x), upload(w), T, H, d, r, inject, eps, h, w_in, inv, oracle.act_of(x))
    torch.cuda.synchronize()
    return h.cpu().numpy(), (w_in.cpu().numpy() if inject else None), inv.cpu().numpy()


@pytest.mark.parametrize("bits", (4, 8))
@pytest.mark.parametrize("act", (oracle.F32, oracle.BF16))
@pytest.mark.parametrize("T,d,r,inject,G", [(1, 64, 32, True, 32), (5, 512, 96, True, 128), (37, 96, 81, False, 32), (6, 256, 320, True, 64)])
def test_mix_down(bits, act, T, d, r, inject, G):
    rng = np.random.default_rng(1000 * bits + 10 * T + act)
    x = randn_act(rng, (T, H * d), act)
    w = quantized(rng, bits, r + (H if inject else 0), H * d, G, sigma=0.05)
    h, w_in, inv = run_down(x, w, d, r, inject)
    rh, rw, rinv = oracle.hc_mix_down(x, w, H, d, r, inject, 1e-6)
    assert np.abs(inv - rinv).max() <= TOL * np.abs(rinv).max()
    assert np.abs(h - rh).max() <= TOL * max(np.abs(rh).max(), 1.0)
    if inject:
        assert np.abs(w_in - rw).max() <= TOL * 2.0


@pytest.mark.parametrize("bits", (4, 8))
@pytest.mark.parametrize("act", (oracle.F32, oracle.BF16))
@pytest.mark.parametrize("T,d,r,G", [(1, 64, 32, 32), (5, 512, 96, 32), (37, 100, 64, 64), (3, 2560, 320, 32)])
def test_mix_up(bits, act, T, d, r, G):
    rng = np.random.default_rng(2000 * bits + 10 * T + act)
    x = randn_act(rng, (T, H * d), act)
    h = rng.standard_normal((T, r)).astype(np.float32)
    w_up = oracle.to_chunk_major(quantized(rng, bits, H * d, r, G, sigma=0.2))
    norm_w = (rng.standard_normal(H * d) * 0.1).astype(np.float32)
    inv = (0.5 + rng.random((T, H))).astype(np.float32)
    u = torch.empty((T, d), dtype=torch.float32 if act == oracle.F32 else torch.bfloat16, device="cuda")
    K.hc_mix_up(torch.from_numpy(h).cuda(), upload(w_up), to_torch_act(x), torch.from_numpy(norm_w).cuda(), torch.from_numpy(inv).cuda(), T, H, d, u, act)
    torch.cuda.synchronize()
    ref = oracle.hc_mix_up(h, w_up, x, norm_w, inv, H, d)
    got = to_np_act(u)
    if act == oracle.BF16:
        got, ref = oracle.bf16_to_f32(got), oracle.bf16_to_f32(ref)
    tol = TOL + (BF16_ULP if act == oracle.BF16 else 0.0)
    assert np.abs(got.astype(np.float64) - ref).max() <= tol * np.abs(ref).max()


def test_bracket_round_trip_with_inject():
    """mix_down -> mix_up -> (a stand-in sublayer) -> hc_inject, the order the runtime drives them in
    (strixite runtime/qwen4exp.cpp), against the same chain on the oracle."""
    rng = np.random.default_rng(5)
    T, d, r = 6, 128, 64
    x = randn_act(rng, (T, H * d), oracle.F32)
    w = quantized(rng, 8, r + H, H * d, 64, sigma=0.05)
    w_up = oracle.to_chunk_major(quantized(rng, 4, H * d, r, 32, sigma=0.2))
    norm_w = (rng.standard_normal(H * d) * 0.1).astype(np.float32)
    rh, rw, rinv = oracle.hc_mix_down(x, w, H, d, r, True, 1e-6)
    ru = oracle.hc_mix_up(rh, w_up, x, norm_w, rinv, H, d)
    rx = x.copy()
    oracle.hc_inject(rx, ru, rw)
    xt = to_torch_act(x)
    h = torch.empty((T, r), device="cuda")
    w_in = torch.empty((T, H), device="cuda")
    inv = torch.empty((T, H), device="cuda")
    u = torch.empty((T, d), device="cuda")
    K.hc_mix_down(xt, upload(w), T, H, d, r, True, 1e-6, h, w_in, inv, oracle.F32)
    K.hc_mix_up(h, upload(w_up), xt, torch.from_numpy(norm_w).cuda(), inv, T, H, d, u, oracle.F32)
    K.hc_inject(xt, u, w_in, T, d, H, oracle.F32)
    torch.cuda.synchronize()
    assert np.abs(xt.cpu().numpy() - rx).max() <= TOL * np.abs(rx).max()


@pytest.mark.parametrize("act", (oracle.F32, oracle.BF16))
def test_inject_inv(act):
    rng = np.random.default_rng(9 + act)
    T, d = 7, 1000
    x = randn_act(rng, (T, H * d), act)
    y = randn_act(rng, (T, d), act)
    w_in = (2.0 * rng.random((T, H))).astype(np.float32)
    rx = x.copy()
    oracle.hc_inject(rx, y, w_in)
    rv = (oracle.bf16_to_f32(rx) if act == oracle.BF16 else rx).astype(np.float64).reshape(T, H, d)
    rinv = 1.0 / np.sqrt((rv * rv).mean(axis=2) + 1e-6)
    xt, inv = to_torch_act(x), torch.empty((T, H), device="cuda")
    K.hc_inject_inv(xt, torch.from_numpy(w_in).cuda(), to_torch_act(y), T, H, d, 1e-6, inv, act)
    torch.cuda.synchronize()
    assert np.array_equal(to_np_act(xt), rx)  # one fma and one rounding per element: bit-exact
    assert np.abs(inv.cpu().numpy() - rinv).max() <= 1e-5 * rinv.max()


def test_argument_errors():
    rng = np.random.default_rng(1)
    w = upload(quantized(rng, 4, 36, 256, 32))
    x = torch.zeros((1, 256), device="cuda")
    h, w_in, inv = torch.zeros((1, 32), device="cuda"), torch.zeros((1, 4), device="cuda"), torch.zeros((1, 4), device="cuda")
    with pytest.raises(StrixError, match="H = 3"):
        K.hc_mix_down(x, w, 1, 3, 64, 32, True, 1e-6, h, w_in, inv, oracle.F32)
    with pytest.raises(StrixError, match="expected \\[32, 256\\]"):
        K.hc_mix_down(x, w, 1, 4, 64, 32, False, 1e-6, h, None, inv, oracle.F32)
    w5 = upload(quantized(rng, 5, 36, 256, 32))
    with pytest.raises(StrixError, match="expected 4 or 8"):
        K.hc_mix_down(x, w5, 1, 4, 64, 32, True, 1e-6, h, w_in, inv, oracle.F32)
