"""GPU: the expert-parallel layer (strixite_b200/ep.py over the CUDA library) against the single-device layer object on the
same weights and tokens. One rank in the test process; several ranks emulated on ONE GPU (every rank's backend on the same
device, the all-to-all done by copying blocks) so that the multi-rank kernels are covered on a one-GPU machine; two real ranks
over NCCL as child processes where the machine has two GPUs."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from helpers import gpu_layer, make_layer, randn_act, rel_err_rows, to_np_act, to_torch_act, upload_stack

pytestmark = pytest.mark.gpu

E, K_TOP, D, I, T = 16, 4, 512, 256, 200


def _layer():
    return make_layer(310, d=D, I=I, E=E, k=K_TOP, G=128, router="bf16", shared="stacked", bias_sigma=1.0)


def _tokens():
    return randn_act(np.random.default_rng(311), (T, D), oracle.BF16)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _backend(L, world, rank, place, Tl, chunks=1, device="cuda", peer_group=None):
    from strixite_b200 import ep as EP
    from strixite_b200 import kernels as K

    rw = torch.from_numpy(L["router"].view(np.int16)).to(device).view(torch.bfloat16)
    bias = torch.from_numpy(L["router_bias"]).to(device)
    gu, dn = upload_stack(L["gate_up"]), upload_stack(L["down"])
    return EP.CudaBackend(D, I, E, K_TOP, K.Act.BF16, rw, bias, EP.shard_stack(gu, E, world, rank, place), EP.shard_stack(dn, E, world, rank, place), world,
                          rank, place, Tl, chunks=chunks, peer_group=peer_group)


@pytest.mark.parametrize("P,rank", [(1, 0), (2, 1), (4, 2), (8, 5)])
def test_plan_kernel_matches_its_numpy_restatement(P, rank):
    from strixite_b200 import ep as EP
    from strixite_b200 import kernels as K
    from strixite_b200._lib import call, lib

    rng = np.random.default_rng(P)
    Tn, A, En = 333, 5, 32
    ids = np.stack([rng.permutation(En + 1)[:A] for _ in range(Tn)]).astype(np.int32)  # id En = the shared expert
    ids[7] = -1
    ids[100, 2] = En + 9
    coef = rng.random((Tn, A)).astype(np.float32)
    place = EP.placement(En, P, rng.standard_normal(En).astype(np.float32), 4, balanced=True)
    for Cr, Cs in ((Tn, Tn * A), (40, 90)):  # ample capacity; capacity that overflows (flags, clamped writes)
        want = EP.plan_reference(ids, coef, En, place["owner"], place["local_of"], P, rank, Cr, Cs)
        d_ids, d_coef = torch.from_numpy(ids).cuda(), torch.from_numpy(coef).cuda()  # kept alive across the asynchronous launch
        d_owner, d_local = torch.from_numpy(place["owner"]).cuda(), torch.from_numpy(place["local_of"]).cuda()
        rowtok = torch.zeros((P, Cr), dtype=torch.int32, device="cuda")
        meta = torch.zeros((P, EP.meta_ints(Cr, Cs)), dtype=torch.int32, device="cuda")
        pos = torch.zeros((Tn, P), dtype=torch.int32, device="cuda")
        flags = torch.zeros(2, dtype=torch.int32, device="cuda")
        scratch = torch.empty(int(lib.strix_ep_plan_scratch_ints(Tn)), dtype=torch.int32, device="cuda")
        call("strix_ep_plan", K._p(d_ids), K._p(d_coef), Tn, A, En, K._p(d_owner), K._p(d_local), P, rank, Cr, Cs,
             K._p(rowtok), K._p(meta), K._p(pos), K._p(flags), K._p(scratch), K._s(None))
        assert np.array_equal(flags.cpu().numpy().view(np.uint32), want[3])
        m, wm = meta.cpu().numpy(), want[1]
        assert np.array_equal(m[:, :2], wm[:, :2])
        for r in range(P):
            nr, ns = wm[r, 0], wm[r, 1]
            assert np.array_equal(rowtok.cpu().numpy()[r, :nr], want[0][r, :nr])
            if want[3].any():
                continue  # beyond capacity only the counts, the flags and the kept rows are defined
            assert np.array_equal(m[r, 4: 4 + 2 * nr], wm[r, 4: 4 + 2 * nr])
            assert np.array_equal(m[r, 4 + 2 * Cr: 4 + 2 * Cr + 3 * ns], wm[r, 4 + 2 * Cr: 4 + 2 * Cr + 3 * ns])
        if not want[3].any():
            assert np.array_equal(pos.cpu().numpy(), want[2])


def test_experts_partial_f16_is_the_rounded_fp32_result():
    """strix_moe_layer_experts_partial: the F16 partial sums are the FP32 ones rounded once, and both are the oracle's per-slot
    expert outputs within the tensor-core contract."""
    L, x = _layer(), _tokens()
    layer = gpu_layer(L, oracle.BF16, T, math=2)
    rng = np.random.default_rng(3)
    n = 200
    ids = rng.integers(0, E + 1, n).astype(np.int32)
    ids[5] = -2  # an absent slot: skipped, no error
    rows = rng.integers(0, T, n).astype(np.int32)
    xt = to_torch_act(x)
    p32 = torch.zeros((n, D), dtype=torch.float32, device="cuda")
    p16 = torch.zeros((n, D), dtype=torch.float16, device="cuda")
    layer.experts_partial(xt, torch.from_numpy(ids).cuda(), partial=p32, row_index=torch.from_numpy(rows).cuda())
    layer.experts_partial(xt, torch.from_numpy(ids).cuda(), partial=p16, row_index=torch.from_numpy(rows).cuda())
    torch.cuda.synchronize()
    assert torch.equal(p32.to(torch.float16), p16)
    assert layer.probe("err", 1).cpu().numpy().tolist() == [0] * 6
    keep = ids >= 0
    xs = np.ascontiguousarray(x[rows[keep]])
    gid = ids[keep].reshape(-1, 1)
    h, _ = oracle.experts_gather(xs, L["gate_up"], gid, swiglu=True)
    want, _ = oracle.experts_combine(np.ascontiguousarray(h.reshape(-1, I)), L["down"], gid, np.ones((gid.shape[0], 1), np.float32))
    assert rel_err_rows(p32.cpu().numpy()[keep], oracle.to_f32(want)) < 2e-3 + 2.0 ** -7  # BF16 pipeline: h rounded to BF16 by the oracle


def _single_device(L, x):
    single = gpu_layer(L, oracle.BF16, T, math=2)
    return to_np_act(single.forward(to_torch_act(x)))


def test_one_rank_is_the_single_device_layer_bit_for_bit():
    from strixite_b200 import ep as EP
    from strixite_b200 import kernels as K

    L, x = _layer(), _tokens()
    for chunks in (1, 2):
        be = _backend(L, 1, 0, EP.placement(E, 1, balanced=False), T, chunks=chunks)
        layer = EP.CudaLayer(be, 1, 0)
        y = layer.forward(to_torch_act(x))
        y2 = layer.forward(to_torch_act(x))  # a second pass through the same buffers
        torch.cuda.synchronize()
        layer.check()
        assert torch.equal(y, y2) and K.umma_abort_count() == 0
        assert np.array_equal(to_np_act(y), _single_device(L, x))
        assert layer.launches_per_step() > 0 and layer.received_slots() == T * (K_TOP + 1)


def _emulate_push(P, balanced, L, x):
    """The same with the kernels writing into the "peers'" receive buffers themselves (strix_ep_push_rows,
    strix_ep_row_sum_push): every rank's buffers are on this GPU, so the address tables simply point at them."""
    from strixite_b200 import ep as EP

    Tl = T // P
    place = EP.placement(E, P, L["router_bias"], K_TOP, balanced=balanced)
    bes = [_backend(L, P, r, place, Tl) for r in range(P)]
    for be in bes:
        be.c[0]["back"] = torch.zeros((P, be.Cr, D), dtype=torch.float16, device="cuda")
    table = {n: torch.tensor([be.c[0][n].data_ptr() for be in bes], dtype=torch.int64, device="cuda") for n in ("rows_recv", "meta_recv", "back")}
    xs = [to_torch_act(x[r * Tl:(r + 1) * Tl].copy()) for r in range(P)]
    for r, be in enumerate(bes):
        be.use_peer_tables([table])
        be.begin(xs[r])
        be.route(0, xs[r])
        be.plan_push(0, barrier=False)
    for be in bes:
        be.experts_push(0, barrier=False)
    ys = [to_np_act(be.home(0, be.c[0]["back"])) for be in bes]
    return ys, bes


def _emulate(P, balanced, L, x):
    """Every rank's backend lives on this GPU; the all-to-all is done by hand (block [s -> r] of rank s's send buffer becomes
    block s of rank r's receive buffer). The kernels, capacities and tables are exactly the multi-rank ones."""
    from strixite_b200 import ep as EP

    Tl = T // P
    place = EP.placement(E, P, L["router_bias"], K_TOP, balanced=balanced)
    bes = [_backend(L, P, r, place, Tl) for r in range(P)]
    xs = [to_torch_act(x[r * Tl:(r + 1) * Tl].copy()) for r in range(P)]
    sends = []
    for r, be in enumerate(bes):
        be.begin(xs[r])
        be.route(0, xs[r])
        sends.append([t.clone() for t in be.plan(0)])
    summed = []
    for r, be in enumerate(bes):
        rows = torch.stack([sends[s][0][r] for s in range(P)])
        meta = torch.stack([sends[s][1][r] for s in range(P)])
        be.c[0]["meta_recv"].copy_(meta)
        summed.append(be.experts(0, rows, be.c[0]["meta_recv"]).clone())
    ys = []
    for r, be in enumerate(bes):
        back = torch.stack([summed[s][r] for s in range(P)])
        ys.append(to_np_act(be.home(0, back)))
    return ys, bes


@pytest.mark.parametrize("P,balanced", [(2, False), (4, True)])
def test_several_ranks_emulated_on_one_gpu(P, balanced):
    L, x = _layer(), _tokens()
    Tl = T // P
    ys, bes = _emulate(P, balanced, L, x)
    for be in bes:
        be.check()
    y = np.concatenate(ys)
    want = _single_device(L, x[: Tl * P])
    # one row per (token, rank), summed per rank first: another association of the same FP32 sum - the BF16 outputs differ
    # from the single-device ones in a few elements, by one BF16 step
    assert (y != want).mean() < 0.02
    assert rel_err_rows(oracle.to_f32(y), oracle.to_f32(want)) < 2.0 ** -7
    assert sum(be.received_slots() for be in bes) == Tl * P * (K_TOP + 1)


@pytest.mark.parametrize("P,balanced", [(2, True), (4, False), (8, True)])
def test_peer_store_exchange_emulated_on_one_gpu(P, balanced):
    L, x = _layer(), _tokens()
    Tl = T // P
    ys, bes = _emulate_push(P, balanced, L, x)
    for be in bes:
        be.check()
    y = np.concatenate(ys)
    base, _ = _emulate(P, balanced, L, x)
    want = _single_device(L, x[: Tl * P])
    # against the all-to-all form: the returned sums are F16 here - one more rounding of 2^-11 before the BF16 output's 2^-8
    # moves about one output in sixteen to the neighbouring BF16 value, never further
    assert (y != np.concatenate(base)).mean() < 0.15
    assert rel_err_rows(oracle.to_f32(y), oracle.to_f32(np.concatenate(base))) < 2.0 ** -7
    assert rel_err_rows(oracle.to_f32(y), oracle.to_f32(want)) < 2.0 ** -7
    assert sum(be.received_slots() for be in bes) == Tl * P * (K_TOP + 1)


def test_a_token_with_a_non_finite_logit_poisons_only_itself():
    """strixite kernels/moe_router.hpp: a token whose logits are not finite gets ids -1 and a NaN output row; every other
    token of every rank is untouched, and the home rank's error word names it."""
    from strixite_b200 import StrixError

    L, x = _layer(), _tokens()
    P, bad = 2, 5
    clean, _ = _emulate(P, False, L, x)
    xb = x.copy()
    xb[bad] = oracle.f32_to_bf16(np.full(xb.shape[1], np.nan, np.float32)) if xb.dtype == np.uint16 else np.nan
    ys, bes = _emulate(P, False, L, xb)
    y, want = oracle.to_f32(np.concatenate(ys)), oracle.to_f32(np.concatenate(clean))
    assert np.isnan(y[bad]).all()
    keep = np.arange(y.shape[0]) != bad
    assert np.array_equal(y[keep], want[keep])
    with pytest.raises(StrixError):
        bes[0].check()  # token 5 lives on rank 0
    bes[1].check()


def _run_rank(rank, world, port, out_dir, chunks, peer):
    from strixite_b200 import ep as EP
    from strixite_b200 import kernels as K

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        L, x = _layer(), _tokens()
        Tl = T // world
        place = EP.placement(E, world, L["router_bias"], K_TOP, balanced=True)
        be = _backend(L, world, rank, place, Tl, chunks=chunks, device="cuda:%d" % rank, peer_group=dist.group.WORLD if peer else None)
        assert be.pushes == peer
        layer = EP.CudaLayer(be, world, rank)
        xr = to_torch_act(x[rank * Tl:(rank + 1) * Tl].copy(), device="cuda:%d" % rank)
        y = layer.forward(xr)
        y2 = layer.forward(xr)
        torch.cuda.synchronize()
        layer.check()
        assert torch.equal(y, y2) and K.umma_abort_count() == 0
        np.save(os.path.join(out_dir, "y%d.npy" % rank), to_np_act(y))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("chunks,peer", [(1, False), (2, False), (1, True), (2, True)])
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_over_nccl(tmp_path, chunks, peer):
    """Two processes, a GPU each: the all-to-all exchange and (peer) the exchange by the kernels' own peer stores."""
    mp.spawn(_run_rank, args=(2, _free_port(), str(tmp_path), chunks, peer), nprocs=2, join=True)
    y = np.concatenate([np.load(tmp_path / ("y%d.npy" % r)) for r in range(2)])
    L, x = _layer(), _tokens()
    want = _single_device(L, x)
    # FP32 sums back: another association of the same sum; F16 sums back (peer): one more rounding before the BF16 output
    assert (y != want).mean() < (0.15 if peer else 0.02)
    assert rel_err_rows(oracle.to_f32(y), oracle.to_f32(want)) < 2.0 ** -7
