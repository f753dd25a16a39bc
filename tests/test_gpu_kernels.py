"""GPU: every kernel of the library against the CPU oracle, through the C ABI, on seeded inputs.
Bit-exact for integer outputs (codes, ids, permutations, error words); FP outputs within the stated tolerances."""
import numpy as np
import pytest
import torch

import oracle
from helpers import BF16_ULP, make_stack, quantized, randn_act, rel_err_rows, to_np_act, to_torch_act, upload, upload_stack
from strixite_b200 import StrixError
from strixite_b200 import kernels as K

pytestmark = pytest.mark.gpu

ACTS = (oracle.F32, oracle.BF16)
# FP32 accumulation in a different order than the oracle's double sum; BF16 outputs may additionally land one BF16
# step apart where the two sums straddle a rounding boundary.
TOL = {oracle.F32: 2e-5, oracle.BF16: 2e-5 + BF16_ULP}


def dev_err():
    return K.new_err()


def host_err(e):
    return e.cpu().numpy().view(np.uint32)[:3].tolist()


@pytest.mark.parametrize("bits", (4, 5, 6, 8))
@pytest.mark.parametrize("G", (32, 64, 128))
def test_device_quantizer_is_bit_identical(bits, G):
    rng = np.random.default_rng(100 * bits + G)
    w = (rng.standard_normal((37, 512)) * 0.02).astype(np.float32)
    w[1, :G] = 0.5
    w[2] = np.linspace(-1, 1, 512, dtype=np.float32)
    ref = oracle.quantize(bits, w, G)
    qw, err = K.QWeight.quantize_device(torch.from_numpy(w).cuda(), bits, G)
    q, s, m = qw.to_host()
    assert host_err(err)[0] == 0
    assert np.array_equal(q, ref.q) and np.array_equal(s, ref.scale) and np.array_equal(m, ref.minv)


def test_device_quantizer_flags_nonfinite():
    w = torch.zeros((4, 128), device="cuda")
    w[2, 77] = float("nan")
    _, err = K.QWeight.quantize_device(w, 4, 32)
    assert host_err(err) == [1, 2, 77]


@pytest.mark.parametrize("act", ACTS)
@pytest.mark.parametrize("E,k,shared", [(1, 1, False), (31, 5, True), (32, 32, False), (33, 10, True), (512, 10, True), (513, 10, False), (1024, 32, True)])
def test_router_bit_exact(act, E, k, shared):
    rng = np.random.default_rng(E * 37 + k)
    M = 67
    ld = E + (1 if shared else 0) + 3
    logits = randn_act(rng, (M, ld), act)
    ids_ref, coef_ref, _ = oracle.moe_router(logits, E, k, shared_col=E if shared else None, shared_id=E)
    lg = to_torch_act(logits)
    A = k + (1 if shared else 0)
    ids = torch.empty((M, A), dtype=torch.int32, device="cuda")
    coef = torch.empty((M, A), dtype=torch.float32, device="cuda")
    err = dev_err()
    K.moe_router(lg, ld, M, E, k, lg[:, E:] if shared else None, ld, E, ids, coef, act, err)
    assert host_err(err)[0] == 0
    assert np.array_equal(ids.cpu().numpy(), ids_ref)
    # expf differs by an ulp or two between glibc and CUDA: compare the weights to 1e-6 relative.
    assert np.allclose(coef.cpu().numpy(), coef_ref, rtol=2e-6, atol=1e-9)


def test_router_ties_and_nonfinite():
    E, k = 64, 4
    logits = np.zeros((4, E + 1), np.float32)
    logits[1, [5, 40, 41]] = 1.0
    logits[2, 9], logits[2, 4] = np.nan, np.inf
    logits[3, E] = -np.inf
    ids_ref, coef_ref, err_ref = oracle.moe_router(logits, E, k, shared_col=E, shared_id=E)
    lg = torch.from_numpy(logits).cuda()
    ids = torch.empty((4, k + 1), dtype=torch.int32, device="cuda")
    coef = torch.empty((4, k + 1), dtype=torch.float32, device="cuda")
    err = dev_err()
    K.moe_router(lg, E + 1, 4, E, k, lg[:, E:], E + 1, E, ids, coef, K.Act.F32, err)
    assert np.array_equal(ids.cpu().numpy(), ids_ref)
    c = coef.cpu().numpy()
    assert np.array_equal(np.isnan(c), np.isnan(coef_ref)) and np.allclose(c[:2], coef_ref[:2], rtol=2e-6)
    e = host_err(err)
    assert e[0] == 1 and (e[1], e[2]) in ((2, 4), (3, E))  # the first flag wins: either failing token may raise it
    with pytest.raises(StrixError, match="non-finite router logit"):
        K.check_router_error(err, "test")


@pytest.mark.parametrize("act", ACTS)
@pytest.mark.parametrize("bits,G", [(4, 128), (4, 32), (5, 128), (6, 64), (8, 64)])
@pytest.mark.parametrize("M", (1, 3, 6, 11))
def test_linear_q(act, bits, G, M):
    rng = np.random.default_rng(bits * 1000 + G + M)
    qw = quantized(rng, bits, 72, 512, G)
    x = randn_act(rng, (M, 512), act)
    for out_act in ({act, oracle.F32} if act == oracle.BF16 else {act}):
        ref = oracle.linear_q(x, qw, out_act)
        y = torch.empty((M, 72), dtype=K._dtype(out_act), device="cuda")
        getattr(K, "linear_q%d" % bits)(to_torch_act(x), upload(qw), y, M, act, out_act)
        assert rel_err_rows(oracle.to_f32(to_np_act(y)), oracle.to_f32(ref)) < TOL[out_act]


@pytest.mark.parametrize("act", ACTS)
@pytest.mark.parametrize("bits,G", [(4, 128), (4, 32), (5, 128), (6, 64), (8, 64)])
@pytest.mark.parametrize("M", (5, 130, 333))
def test_linear_qw_wmma(act, bits, G, M):
    # the dense projection on the tensor cores (strixite kernels/linear_wmma.hpp:21-24): F16 operands (one rounding of the
    # dequantized weight and of an FP32 activation), FP32 accumulation - far inside the 2e-3 contract, not FP32-FMA exact
    rng = np.random.default_rng(bits * 1000 + G + M)
    N, Kd = 200, 512  # a ragged last tile of weight rows and of tokens
    qw = quantized(rng, bits, N, Kd, G)
    x = randn_act(rng, (M, Kd), act)
    before = K.umma_abort_count()
    for out_act in ({act, oracle.F32} if act == oracle.BF16 else {act}):
        ref = oracle.linear_q(x, qw, out_act)
        y = torch.empty((M, N), dtype=K._dtype(out_act), device="cuda")
        K.linear_qw_wmma(to_torch_act(x), upload(qw), y, M, act, out_act)
        assert rel_err_rows(oracle.to_f32(to_np_act(y)), oracle.to_f32(ref)) < 1e-3 + (BF16_ULP if out_act == oracle.BF16 else 0.0)
    assert K.umma_abort_count() == before


def test_linear_bf16w_wmma_matches_the_fma_kernel():
    rng = np.random.default_rng(11)
    M, N, Kd = 130, 513, 512
    w = oracle.f32_to_bf16((rng.standard_normal((N, Kd)) * 0.02).astype(np.float32))
    x = randn_act(rng, (M, Kd), oracle.BF16)
    ref = oracle.linear_w(x, w, oracle.F32)
    y = torch.empty((M, N), dtype=torch.float32, device="cuda")
    K.linear_bf16w_wmma(to_torch_act(x), torch.from_numpy(w.view(np.int16)).cuda(), y, M, N, Kd, oracle.BF16, oracle.F32)
    assert rel_err_rows(y.cpu().numpy(), ref) < 2e-5
    with pytest.raises(StrixError, match="BF16 tokens with FP32 outputs"):
        K.linear_bf16w_wmma(torch.zeros((M, Kd), device="cuda"), torch.from_numpy(w.view(np.int16)).cuda(), y, M, N, Kd, oracle.F32, oracle.F32)


@pytest.mark.parametrize("act", ACTS)
@pytest.mark.parametrize("wtype", ("f32", "bf16"))
def test_linear_w(act, wtype):
    rng = np.random.default_rng(7)
    M, N, Kd = 5, 130, 1024
    w = (rng.standard_normal((N, Kd)) * 0.02).astype(np.float32)
    wh = w if wtype == "f32" else oracle.f32_to_bf16(w)
    x = randn_act(rng, (M, Kd), act)
    ref = oracle.linear_w(x, wh, oracle.F32)
    y = torch.empty((M, N), dtype=torch.float32, device="cuda")
    if act == oracle.BF16 or True:
        fn = K.linear_f32w if wtype == "f32" else K.linear_bf16w
        if act == oracle.F32:
            fn(to_torch_act(x), to_torch_act(wh), y, M, N, Kd, act)
        else:
            fn(to_torch_act(x), to_torch_act(wh), y, M, N, Kd, act, K.Act.F32)
    assert rel_err_rows(y.cpu().numpy(), ref) < 2e-5


@pytest.mark.parametrize("act", ACTS)
def test_swiglu_residual_inject_bitwise(act):
    rng = np.random.default_rng(8)
    rows, I = 13, 96
    gu = randn_act(rng, (rows, 2 * I), act, 2.0)
    h = torch.empty((rows, I), dtype=K._dtype(act), device="cuda")
    K.swiglu(to_torch_act(gu), h, rows, I, act)
    ref = oracle.swiglu(gu, I)
    got = to_np_act(h)
    # expf(-g) may differ in the last place between glibc and CUDA; everything after it is the same arithmetic.
    assert np.allclose(oracle.to_f32(got), oracle.to_f32(ref), rtol=(1e-6 if act == oracle.F32 else BF16_ULP), atol=1e-7)
    x, y = randn_act(rng, (5, 77), act), randn_act(rng, (5, 77), act)
    xr = x.copy()
    oracle.residual_add(xr, y)
    xt = to_torch_act(x)
    K.residual_add(xt, to_torch_act(y), x.size, act)
    assert np.array_equal(to_np_act(xt), xr)
    w_in = rng.standard_normal((5, 4)).astype(np.float32)
    xs = randn_act(rng, (5, 4 * 77), act)
    xsr = xs.copy()
    oracle.hc_inject(xsr, y, w_in)
    xst = to_torch_act(xs)
    K.hc_inject(xst, to_torch_act(y), torch.from_numpy(w_in).cuda(), 5, 77, 4, act)
    assert np.array_equal(to_np_act(xst), xsr)


@pytest.mark.parametrize("act", ACTS)
def test_shared_add_and_inject(act):
    rng = np.random.default_rng(9)
    M, N = 7, 300
    y0, s = randn_act(rng, (M, N), act), randn_act(rng, (M, N), act)
    gl = rng.standard_normal((M, 5)).astype(np.float32)
    gl[4, 2] = np.nan
    x0, w_in = randn_act(rng, (M, 4 * N), act), rng.standard_normal((M, 4)).astype(np.float32)
    yr, xr = y0.copy(), x0.copy()
    err_ref = oracle.moe_shared_add_inject(yr, s, gl, 2, 33, xr, w_in)
    glt = torch.from_numpy(gl).cuda()
    # fused
    y1, x1, e1 = to_torch_act(y0), to_torch_act(x0), dev_err()
    K.moe_shared_add_inject(y1, to_torch_act(s), glt[:, 2:], 5, M, N, 33, x1, torch.from_numpy(w_in).cuda(), 4, act, e1)
    # the two kernels it replaces
    y2, x2, e2 = to_torch_act(y0), to_torch_act(x0), dev_err()
    K.moe_shared_add(y2, to_torch_act(s), glt[:, 2:], 5, M, N, 33, act, e2)
    K.hc_inject(x2, y2, torch.from_numpy(w_in).cuda(), M, N, 4, act)
    assert torch.equal(y1.view(torch.int16 if act else torch.int32), y2.view(torch.int16 if act else torch.int32))  # bit-identical
    assert torch.equal(x1.view(torch.int16 if act else torch.int32), x2.view(torch.int16 if act else torch.int32))
    assert host_err(e1) == err_ref.tolist() == [1, 4, 33] and host_err(e2) == [1, 4, 33]
    got, want = oracle.to_f32(to_np_act(y1)), oracle.to_f32(yr)
    assert np.all(np.isnan(got[4])) and np.all(np.isnan(want[4]))
    ok = [0, 1, 2, 3, 5, 6]
    assert np.allclose(got[ok], want[ok], rtol=(2e-6 if act == oracle.F32 else BF16_ULP), atol=1e-6)
    assert np.allclose(oracle.to_f32(to_np_act(x1))[ok], oracle.to_f32(xr)[ok], rtol=(2e-6 if act == oracle.F32 else 2 * BF16_ULP), atol=1e-5)


STACKS = [dict(bits=4, G=128), dict(bits=4, G=32), dict(bits=5, G=128), dict(bits=4, G=128, mix=[0.4, 0.2, 0.2, 0.2])]


@pytest.mark.parametrize("act", ACTS)
@pytest.mark.parametrize("cfg", STACKS)
@pytest.mark.parametrize("M,A", [(1, 3), (6, 4)])
def test_experts_per_slot(act, cfg, M, A):
    rng = np.random.default_rng(M * 10 + A)
    E, I, d = 9, 128, 256
    gu_st = make_stack(rng, E, 2 * I, d, cfg["G"], cfg["bits"], cfg.get("mix"))
    dn_st = make_stack(rng, E, d, I, cfg["G"], cfg["bits"], cfg.get("mix"))
    x = randn_act(rng, (M, d), act)
    ids = np.stack([rng.permutation(E)[:A] for _ in range(M)]).astype(np.int32)
    coef = rng.random((M, A)).astype(np.float32)
    gu_d, dn_d = upload_stack(gu_st), upload_stack(dn_st)
    qv = K.qweight(gu_d)
    xt, idt = to_torch_act(x), torch.from_numpy(ids).cuda()
    # gather
    ref, _ = oracle.experts_gather(x, gu_st, ids)
    y = torch.empty((M, A, 2 * I), dtype=K._dtype(act), device="cuda")
    err = dev_err()
    K.linear_qw_experts_gather(xt, qv, E, idt, M, A, y, act, err)
    assert host_err(err)[0] == 0
    assert rel_err_rows(oracle.to_f32(to_np_act(y)), oracle.to_f32(ref)) < TOL[act]
    # fused gather + SwiGLU == gather then swiglu, bitwise (strixite kernels/linear_q4.hpp:53-54)
    h = torch.empty((M, A, I), dtype=K._dtype(act), device="cuda")
    K.linear_qw_experts_gather_swiglu(xt, qv, E, idt, M, A, h, act, err)
    h2 = torch.empty_like(h)
    K.swiglu(y, h2, M * A, I, act)
    assert torch.equal(h.view(torch.int16 if act else torch.int32), h2.view(torch.int16 if act else torch.int32))
    href, _ = oracle.experts_gather(x, gu_st, ids, swiglu=True)
    assert rel_err_rows(oracle.to_f32(to_np_act(h)), oracle.to_f32(href)) < (1e-4 if act == oracle.F32 else 2 * BF16_ULP + 1e-4)
    # combine on the oracle's h, so only this kernel is under test
    yref, _ = oracle.experts_combine(href, dn_st, ids, coef)
    yc = torch.empty((M, d), dtype=K._dtype(act), device="cuda")
    K.linear_qw_experts_combine(to_torch_act(href), K.qweight(dn_d), E, idt, torch.from_numpy(coef).cuda(), M, A, yc, act, err)
    assert rel_err_rows(oracle.to_f32(to_np_act(yc)), oracle.to_f32(yref)) < TOL[act]
    assert host_err(err)[0] == 0


def test_experts_bad_id_flags_and_poisons():
    rng = np.random.default_rng(3)
    E, I, d, M, A = 4, 64, 128, 2, 2
    gu_st, dn_st = make_stack(rng, E, 2 * I, d, 32), make_stack(rng, E, d, I, 32)
    x = randn_act(rng, (M, d), oracle.F32)
    ids = np.array([[0, 9], [1, 2]], np.int32)
    xt, idt = to_torch_act(x), torch.from_numpy(ids).cuda()
    err = dev_err()
    h = torch.empty((M, A, I), device="cuda")
    K.linear_q4_experts_gather_swiglu(xt, upload_stack(gu_st), E, idt, M, A, h, K.Act.F32, err)
    hh = h.cpu().numpy()
    assert host_err(err) == [1, 9, 1] and np.all(np.isnan(hh[0, 1])) and not np.isnan(hh[0, 0]).any() and not np.isnan(hh[1]).any()
    with pytest.raises(StrixError, match="expert id 9 at slot 1"):
        K.check_expert_error(err, "test")
    err = dev_err()
    y = torch.empty((M, d), device="cuda")
    K.linear_q4_experts_combine(torch.zeros((M, A, I), device="cuda"), upload_stack(dn_st), E, idt, torch.ones((M, A), device="cuda"), M, A, y,
                                K.Act.F32, err)
    yy = y.cpu().numpy()
    assert host_err(err) == [1, 9, 1] and np.all(np.isnan(yy[0])) and not np.isnan(yy[1]).any()


@pytest.mark.parametrize("M,A,E", [(1, 1, 1), (6, 11, 513), (37, 5, 19), (512, 11, 513), (4096, 11, 513), (3000, 64, 1023)])
def test_group_routes_bit_exact(M, A, E):
    rng = np.random.default_rng(M + A + E)
    # skewed routing: a few hot experts take most slots; every token routes to distinct experts like the router's output
    p = rng.random(E) ** 4
    p /= p.sum()
    ids = np.stack([rng.choice(E, size=A, replace=False, p=p) if A <= np.count_nonzero(p) else rng.permutation(E)[:A] for _ in range(M)]).astype(np.int32)
    if M > 4:
        ids[3, A // 2], ids[M - 1, 0] = -1, E + 7
    ref, err_ref = oracle.group_routes(ids, E)
    nbytes = K.moe_route_workspace_bytes(M, A, E)
    assert nbytes == ref.size * 4
    ws = torch.full((nbytes // 4,), -7, dtype=torch.int32, device="cuda")
    err = dev_err()
    for _ in range(2):  # the same permutation on every run
        K.moe_group_routes(torch.from_numpy(ids).cuda(), M, A, E, ws, nbytes, err)
        got = ws.cpu().numpy()
        S, Tmax, WTmax = M * A, M * A // 16 + E + 2, M * A // 64 + E + 2
        head = 4 + E + 2 + S
        assert np.array_equal(got[:head], ref[:head])  # header, offsets, the permutation
        nt, nwt = ref[0], ref[3]
        for base, n in ((head, nt), (head + Tmax, nt), (head + 2 * Tmax, nwt), (head + 2 * Tmax + WTmax, nwt)):
            assert np.array_equal(got[base : base + n], ref[base : base + n])
    assert host_err(err) == err_ref.tolist()


@pytest.mark.parametrize("act", ACTS)
@pytest.mark.parametrize("cfg", STACKS)
def test_experts_grouped_f32(act, cfg):
    rng = np.random.default_rng(21)
    E, I, d, M, A = 9, 128, 256, 45, 4
    gu_st = make_stack(rng, E, 2 * I, d, cfg["G"], cfg["bits"], cfg.get("mix"))
    dn_st = make_stack(rng, E, d, I, cfg["G"], cfg["bits"], cfg.get("mix"))
    x = randn_act(rng, (M, d), act)
    ids = np.stack([rng.permutation(E)[:A] for _ in range(M)]).astype(np.int32)
    ids[:, 0] = 2  # a hot expert: several tiles
    coef = rng.random((M, A)).astype(np.float32)
    xt, idt, ct = to_torch_act(x), torch.from_numpy(ids).cuda(), torch.from_numpy(coef).cuda()
    nbytes = K.moe_route_workspace_bytes(M, A, E)
    ws = torch.empty(nbytes // 4, dtype=torch.int32, device="cuda")
    err = dev_err()
    K.moe_group_routes(idt, M, A, E, ws, nbytes, err)
    y = torch.empty((M, A, 2 * I), dtype=K._dtype(act), device="cuda")
    K.linear_qw_experts_gather_grouped(xt, K.qweight(upload_stack(gu_st)), E, ws, nbytes, M, A, y, act, K.MoeMath.F32)
    ref, _ = oracle.experts_gather(x, gu_st, ids)
    assert rel_err_rows(oracle.to_f32(to_np_act(y)), oracle.to_f32(ref)) < TOL[act]
    href, _ = oracle.experts_gather(x, gu_st, ids, swiglu=True)
    yref, _ = oracle.experts_combine(href, dn_st, ids, coef)
    partial = torch.empty((M * A * d,), dtype=torch.float32, device="cuda")
    yc = torch.empty((M, d), dtype=K._dtype(act), device="cuda")
    K.linear_qw_experts_combine_grouped(to_torch_act(href), K.qweight(upload_stack(dn_st)), E, idt, ct, ws, nbytes, partial, M, A, yc, act,
                                        K.MoeMath.F32)
    assert rel_err_rows(oracle.to_f32(to_np_act(yc)), oracle.to_f32(yref)) < TOL[act]
    assert host_err(err)[0] == 0


def test_grouped_bad_id():
    rng = np.random.default_rng(22)
    E, I, d, M, A = 5, 64, 128, 20, 2
    gu_st = make_stack(rng, E, 2 * I, d, 32)
    x = randn_act(rng, (M, d), oracle.F32)
    ids = np.stack([rng.permutation(E)[:A] for _ in range(M)]).astype(np.int32)
    ids[7, 1] = 99
    nbytes = K.moe_route_workspace_bytes(M, A, E)
    ws = torch.empty(nbytes // 4, dtype=torch.int32, device="cuda")
    err = dev_err()
    K.moe_group_routes(torch.from_numpy(ids).cuda(), M, A, E, ws, nbytes, err)
    y = torch.empty((M, A, 2 * I), device="cuda")
    K.linear_q4_experts_gather_grouped(to_torch_act(x), upload_stack(gu_st), E, ws, nbytes, M, A, y, K.Act.F32, K.MoeMath.F32)
    yy = y.cpu().numpy()
    assert host_err(err) == [1, 99, 15] and np.all(np.isnan(yy[7, 1])) and np.isnan(yy).sum() == 2 * I


def test_grouped_refuses_a_workspace_grouped_for_other_sizes():
    """A workspace built for (16 tokens, 4 slots, 16 experts) has the same byte size as one for (12, 4, 20), so the host's size
    check passes - the kernels compare the header with the call's sizes, store nothing and count the refusal."""
    rng = np.random.default_rng(23)
    I, d = 64, 128
    nbytes = K.moe_route_workspace_bytes(16, 4, 16)
    assert nbytes == K.moe_route_workspace_bytes(12, 4, 20)
    ids = np.stack([rng.permutation(16)[:4] for _ in range(16)]).astype(np.int32)
    ws = torch.empty(nbytes // 4, dtype=torch.int32, device="cuda")
    err = dev_err()
    K.moe_group_routes(torch.from_numpy(ids).cuda(), 16, 4, 16, ws, nbytes, err)
    w = upload_stack(make_stack(rng, 20, 2 * I, d, 32))
    x = to_torch_act(randn_act(rng, (12, d), oracle.F32))
    for math in (K.MoeMath.F32, K.MoeMath.WmmaF16):
        before = K.workspace_refusal_count()
        y = torch.full((12, 4, 2 * I), 7.0, device="cuda")
        K.linear_q4_experts_gather_grouped(x, w, 20, ws, nbytes, 12, 4, y, K.Act.F32, math)
        torch.cuda.synchronize()
        assert bool((y == 7.0).all()) and K.workspace_refusal_count() == before + 1


@pytest.mark.parametrize("act", ACTS)
@pytest.mark.parametrize("cfg", STACKS)
@pytest.mark.parametrize("M,A", [(45, 4), (300, 3)])
def test_experts_grouped_tensor_cores(act, cfg, M, A):
    """The tcgen05 grouped GEMM (MoeMath WmmaBf16 / WmmaF16) against the oracle. Weights are rounded to BF16 on the way to
    the tensor cores (and FP32 activations too): the contract is 2e-3 of the row maximum, FP32 accumulation."""
    rng = np.random.default_rng(31 + M)
    E, I, d = 9, 128, 256
    gu_st = make_stack(rng, E, 2 * I, d, cfg["G"], cfg["bits"], cfg.get("mix"))
    dn_st = make_stack(rng, E, d, I, cfg["G"], cfg["bits"], cfg.get("mix"))
    x = randn_act(rng, (M, d), act)
    ids = np.stack([rng.permutation(E)[:A] for _ in range(M)]).astype(np.int32)
    ids[:, 0] = 2  # a hot expert: several 128-token tiles at M = 300
    coef = rng.random((M, A)).astype(np.float32)
    xt, idt, ct = to_torch_act(x), torch.from_numpy(ids).cuda(), torch.from_numpy(coef).cuda()
    nbytes = K.moe_route_workspace_bytes(M, A, E)
    ws = torch.empty(nbytes // 4, dtype=torch.int32, device="cuda")
    err = dev_err()
    K.moe_group_routes(idt, M, A, E, ws, nbytes, err)
    tol = 2e-3 + (BF16_ULP if act == oracle.BF16 else 0.0)
    for math in (K.MoeMath.WmmaBf16, K.MoeMath.WmmaF16):
        y = torch.full((M, A, 2 * I), float("nan"), dtype=K._dtype(act), device="cuda")
        K.linear_qw_experts_gather_grouped(xt, K.qweight(upload_stack(gu_st)), E, ws, nbytes, M, A, y, act, math)
        ref, _ = oracle.experts_gather(x, gu_st, ids)
        assert rel_err_rows(oracle.to_f32(to_np_act(y)), oracle.to_f32(ref)) < tol
        href, _ = oracle.experts_gather(x, gu_st, ids, swiglu=True)
        yref, _ = oracle.experts_combine(href, dn_st, ids, coef)
        partial = torch.empty((M * A * d,), dtype=torch.float32, device="cuda")
        yc = torch.full((M, d), float("nan"), dtype=K._dtype(act), device="cuda")
        K.linear_qw_experts_combine_grouped(to_torch_act(href), K.qweight(upload_stack(dn_st)), E, idt, ct, ws, nbytes, partial, M, A, yc, act, math)
        assert rel_err_rows(oracle.to_f32(to_np_act(yc)), oracle.to_f32(yref)) < tol
    from strixite_b200._lib import lib

    assert lib.strix_umma_abort_count() == 0


def test_grouped_tensor_cores_bad_id_and_k_check():
    rng = np.random.default_rng(23)
    E, I, d, M, A = 5, 64, 128, 20, 2
    gu_st = make_stack(rng, E, 2 * I, d, 32)
    x = randn_act(rng, (M, d), oracle.BF16)
    ids = np.stack([rng.permutation(E)[:A] for _ in range(M)]).astype(np.int32)
    ids[7, 1] = 99
    nbytes = K.moe_route_workspace_bytes(M, A, E)
    ws = torch.empty(nbytes // 4, dtype=torch.int32, device="cuda")
    err = dev_err()
    K.moe_group_routes(torch.from_numpy(ids).cuda(), M, A, E, ws, nbytes, err)
    y = torch.zeros((M, A, 2 * I), dtype=torch.bfloat16, device="cuda")
    K.linear_q4_experts_gather_grouped(to_torch_act(x), upload_stack(gu_st), E, ws, nbytes, M, A, y, K.Act.BF16, K.MoeMath.WmmaBf16)
    yy = y.float().cpu().numpy()
    assert host_err(err) == [1, 99, 15] and np.all(np.isnan(yy[7, 1])) and np.isnan(yy).sum() == 2 * I
    # K must be a multiple of 64 on the tensor path (strixite kernels/moe_grouped.hip:515,528)
    st32 = make_stack(rng, E, 64, 96, 32)
    with pytest.raises(StrixError, match="multiple of 64"):
        K.linear_q4_experts_gather_grouped(torch.zeros((M, 96), dtype=torch.bfloat16, device="cuda"), upload_stack(st32), E, ws, nbytes, M, A,
                                           torch.zeros((M, A, 64), dtype=torch.bfloat16, device="cuda"), K.Act.BF16, K.MoeMath.WmmaBf16)
