"""GPU: the combine whose partial sums live in the library's fixed device array (no buffer passed, nothing allocated)
against the entry point that takes the caller's buffer. Collected last on purpose: it must hold both alone in a fresh
process and after every other test has used the device."""
import numpy as np
import pytest
import torch

import oracle
from helpers import make_stack, randn_act, rel_err_rows, to_np_act, to_torch_act, upload_stack
from strixite_b200 import StrixError
from strixite_b200 import kernels as K

pytestmark = pytest.mark.gpu

TOL = 2e-5  # FP32 accumulation order against the oracle's double sum; both entry points run the same kernels


def _case(seed, E, I, d, M, A, G=32):
    rng = np.random.default_rng(seed)
    dn = make_stack(rng, E, d, I, G, 4)
    h = randn_act(rng, (M * A, I), oracle.F32)
    ids = np.stack([rng.permutation(E)[:A] for _ in range(M)]).astype(np.int32)
    coef = rng.random((M, A)).astype(np.float32)
    yref, _ = oracle.experts_combine(h, dn, ids, coef)
    nbytes = K.moe_route_workspace_bytes(M, A, E)
    ws = torch.empty(nbytes // 4, dtype=torch.int32, device="cuda")
    idt = torch.from_numpy(ids).cuda()
    K.moe_group_routes(idt, M, A, E, ws, nbytes, K.new_err())
    return dict(E=E, M=M, A=A, d=d, w=K.qweight(upload_stack(dn)), h=to_torch_act(h), ids=idt, coef=torch.from_numpy(coef).cuda(), ws=ws,
                nbytes=nbytes, yref=oracle.to_f32(yref))


def _with_buffer(c):
    partial = torch.empty((c["M"] * c["A"] * c["d"],), dtype=torch.float32, device="cuda")
    y = torch.empty((c["M"], c["d"]), dtype=torch.float32, device="cuda")
    K.linear_q4_experts_combine_grouped(c["h"], c["w"].w, c["E"], c["ids"], c["coef"], c["ws"], c["nbytes"], partial, c["M"], c["A"], y, K.Act.F32,
                                        K.MoeMath.F32)
    return y


def test_fixed_scratch_combine_matches_twice_in_a_row():
    a, b = _case(501, E=9, I=128, d=256, M=37, A=3), _case(502, E=6, I=64, d=128, M=11, A=2)
    want_a, want_b = _with_buffer(a), _with_buffer(b)
    ya = torch.empty_like(want_a)
    yb = torch.empty_like(want_b)
    ya2 = torch.empty_like(want_a)
    # a warm-up call resolves the array's address (once per device) before the memory readings
    K.linear_q4_experts_combine_grouped_fixed(b["h"], b["w"].w, b["E"], b["ids"], b["coef"], b["ws"], b["nbytes"], b["M"], b["A"], yb, K.Act.F32,
                                              K.MoeMath.F32)
    torch.cuda.synchronize()
    before = after_outputs = torch.cuda.memory_allocated()
    free_before = torch.cuda.mem_get_info()[0]  # the driver's view: a cudaMalloc inside the library would show here
    # two calls in a row on one stream share the array; the second (another shape) must not disturb a third
    for c, y in ((a, ya), (b, yb), (a, ya2)):
        K.linear_q4_experts_combine_grouped_fixed(c["h"], c["w"].w, c["E"], c["ids"], c["coef"], c["ws"], c["nbytes"], c["M"], c["A"], y, K.Act.F32,
                                                  K.MoeMath.F32)
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == after_outputs >= before  # the calls took nothing from torch's allocator
    assert torch.cuda.mem_get_info()[0] == free_before  # ... and nothing from the device behind its back
    for y, want, c in ((ya, want_a, a), (yb, want_b, b), (ya2, want_a, a)):
        got = to_np_act(y)
        assert rel_err_rows(got, to_np_act(want)) < TOL
        assert rel_err_rows(got, c["yref"]) < TOL


@pytest.mark.parametrize("act", (oracle.F32, oracle.BF16))
def test_fixed_scratch_combine_on_the_tensor_cores(act):
    """The tensor-core route of the same entry (the grouped GEMM writes its partial sums into the fixed array), FP32 and
    BF16 activations, against the entry that takes the caller's buffer: same kernels, same bits."""
    rng = np.random.default_rng(504 + act)
    E, I, d, M, A = 7, 128, 256, 70, 3
    dn = make_stack(rng, E, d, I, 32, 4)
    h = randn_act(rng, (M * A, I), act)
    ids = np.stack([rng.permutation(E)[:A] for _ in range(M)]).astype(np.int32)
    coef = rng.random((M, A)).astype(np.float32)
    yref, _ = oracle.experts_combine(h, dn, ids, coef)
    nbytes = K.moe_route_workspace_bytes(M, A, E)
    ws = torch.empty(nbytes // 4, dtype=torch.int32, device="cuda")
    idt, ct, ht, w = torch.from_numpy(ids).cuda(), torch.from_numpy(coef).cuda(), to_torch_act(h), upload_stack(dn)
    K.moe_group_routes(idt, M, A, E, ws, nbytes, K.new_err())
    partial = torch.empty((M * A * d,), dtype=torch.float32, device="cuda")
    want = torch.empty((M, d), dtype=K._dtype(act), device="cuda")
    got = torch.empty_like(want)
    aborts = K.umma_abort_count()
    K.linear_q4_experts_combine_grouped(ht, w, E, idt, ct, ws, nbytes, partial, M, A, want, act, K.MoeMath.WmmaF16)
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    K.linear_q4_experts_combine_grouped_fixed(ht, w, E, idt, ct, ws, nbytes, M, A, got, act, K.MoeMath.WmmaF16)
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before and K.umma_abort_count() == aborts
    assert torch.equal(got, want)
    assert rel_err_rows(oracle.to_f32(to_np_act(got)), oracle.to_f32(yref)) < 2e-3 + (2.0 ** -7 if act == oracle.BF16 else 0.0)


def test_fixed_scratch_combine_rejects_oversize():
    c = _case(503, E=4, I=64, d=128, M=8, A=2)
    big_M = K.FIXED_PARTIAL_FLOATS // (c["A"] * c["d"]) + 1
    y = torch.empty((c["M"], c["d"]), dtype=torch.float32, device="cuda")
    with pytest.raises(StrixError, match="fixed scratch"):
        K.linear_q4_experts_combine_grouped_fixed(c["h"], c["w"].w, c["E"], c["ids"], c["coef"], c["ws"], c["nbytes"], big_M, c["A"], y, K.Act.F32,
                                                  K.MoeMath.F32)
