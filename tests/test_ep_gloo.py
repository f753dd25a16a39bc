"""CPU, gloo ranks: the expert-parallel exchange logic (strixite_b200/ep.py: fixed-capacity blocks, one row per (token, rank),
expert-side and home-side sums) over a host backend made of numpy and the oracle must reproduce the single-process oracle
layer, for one and two ranks, contiguous and balanced placements, one and two chunks per step - and a rank that never joins the
exchange must surface as an error on the others after a host-side timeout, not as a hang."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from helpers import make_layer, randn_act, rel_err_rows
from strixite_b200 import ep as EP

E, K_TOP, D, I, T = 8, 3, 128, 64, 24
A = K_TOP + 1


def _layer():
    return make_layer(77, d=D, I=I, E=E, k=K_TOP, G=32, router="f32", shared="stacked", bias_sigma=1.0)


def _tokens():
    return randn_act(np.random.default_rng(78), (T, D), oracle.F32)


class HostBackend:
    """The compute steps of the exchange on numpy arrays: the plan's numpy restatement, the oracle's router and experts."""

    def __init__(self, L, world, rank, place, Tc, chunks, Cs):
        self.L, self.P, self.rank, self.place, self.chunks = L, world, rank, place, chunks
        self.Cr, self.Cs = Tc, Cs
        self.c = [dict() for _ in range(chunks)]
        inv = np.zeros((world, place["El"]), np.int64)
        for r in range(world):
            inv[r] = place["experts_of"][r]
        self.global_of = inv  # [rank][local] -> id in the full stacks

    def stream(self, c):
        return EP._NoStream()

    def begin(self, x):
        pass

    def end(self, ys):
        return torch.cat(ys, 0)

    def rows_recv(self, c):
        return torch.zeros((self.P, self.Cr, D), dtype=torch.float32)

    def meta_recv(self, c):
        return torch.zeros((self.P, EP.meta_ints(self.Cr, self.Cs)), dtype=torch.int32)

    def back(self, c):
        return torch.zeros((self.P, self.Cr, D), dtype=torch.float32)

    def route(self, c, x):
        L = self.L
        logits = oracle.linear_w(x.numpy(), L["router"], out_act=oracle.F32)
        logits[:, :E] += L["router_bias"]
        ids, coef, _ = oracle.moe_router(np.ascontiguousarray(logits), E, K_TOP, shared_col=E, shared_id=E)
        self.c[c].update(x=x.numpy(), ids=ids, coef=coef)

    def plan(self, c):
        b = self.c[c]
        rowtok, meta, pos, flags = EP.plan_reference(b["ids"], b["coef"], E, self.place["owner"], self.place["local_of"], self.P, self.rank, self.Cr, self.Cs)
        assert not flags.any()
        b["pos"] = pos
        rows = np.zeros((self.P, self.Cr, D), np.float32)
        for r in range(self.P):
            n = meta[r, 0]
            rows[r, :n] = b["x"][rowtok[r, :n]]
        return torch.from_numpy(rows), torch.from_numpy(meta)

    def experts(self, c, rows_recv, meta_recv):
        L, Cr, Cs = self.L, self.Cr, self.Cs
        rows, meta = rows_recv.numpy(), meta_recv.numpy()
        summed = np.zeros((self.P, Cr, D), np.float32)
        for s in range(self.P):
            for i in range(meta[s, 0]):
                first, n = meta[s, 4 + 2 * i], meta[s, 4 + 2 * i + 1]
                acc = np.zeros(D, np.float64)
                for j in range(first, first + n):
                    loc, row, cb = meta[s, 4 + 2 * Cr + 3 * j: 4 + 2 * Cr + 3 * j + 3]
                    assert row == i and 0 <= loc <= self.place["El"]
                    gid = np.array([[E if loc == self.place["El"] else self.global_of[self.rank, loc]]], np.int32)
                    h, _ = oracle.experts_gather(np.ascontiguousarray(rows[s, i:i + 1]), L["gate_up"], gid, swiglu=True)
                    y, _ = oracle.experts_combine(np.ascontiguousarray(h.reshape(1, I)), L["down"], gid, np.ones((1, 1), np.float32))
                    acc += float(np.array([cb], np.int32).view(np.float32)[0]) * y[0].astype(np.float64)
                summed[s, i] = acc
        return torch.from_numpy(summed)

    def home(self, c, back):
        b = self.c[c]
        y = np.zeros((b["ids"].shape[0], D), np.float32)
        for t in range(y.shape[0]):
            acc = np.zeros(D, np.float64)
            for r in range(self.P):
                if b["pos"][t, r] >= 0:
                    acc += back.numpy()[r, b["pos"][t, r]]
            y[t] = acc
        return torch.from_numpy(y)


def _worker(rank, world, port, out_dir, balanced, chunks, absent_rank):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        L, x = _layer(), _tokens()
        Tl = T // world
        place = EP.placement(E, world, L["router_bias"], K_TOP, balanced=balanced)
        be = HostBackend(L, world, rank, place, Tl // chunks, chunks, Cs=(Tl // chunks) * A)
        ep = EP.ExpertParallelMoe(world, rank, be, chunks=chunks, timeout_s=3.0 if absent_rank is not None else None)
        if rank == absent_rank:
            return  # this rank never posts its blocks; it leaves between steps, with nothing of its own in flight
        try:
            y = ep.forward(torch.from_numpy(x[rank * Tl:(rank + 1) * Tl].copy()))
            np.save(os.path.join(out_dir, "y%d.npy" % rank), y.numpy())
        except Exception as e:  # noqa: BLE001
            open(os.path.join(out_dir, "err%d.txt" % rank), "w").write("%s: %s" % (type(e).__name__, e))
    finally:
        if absent_rank is None:
            dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world,balanced,chunks", [(1, False, 1), (2, False, 1), (2, True, 2)])
def test_exchange_reproduces_the_single_process_layer(tmp_path, world, balanced, chunks):
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path), balanced, chunks, None), nprocs=world, join=True)
    y = np.concatenate([np.load(tmp_path / ("y%d.npy" % r)) for r in range(world)])
    want, _ = oracle.moe_layer(_tokens(), _layer())
    assert rel_err_rows(y, want) < 1e-5


def test_a_rank_that_never_joins_is_an_error_not_a_hang(tmp_path):
    # rank 1 leaves before the exchange; rank 0's all-to-all must end with an error after the host-side timeout
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path), False, 1, 1), nprocs=2, join=True)
    assert not (tmp_path / "y0.npy").exists()
    msg = (tmp_path / "err0.txt").read_text()
    assert "did not join" in msg or "imeout" in msg or "closed" in msg.lower() or "Error" in msg


def test_placement_balances_a_skewed_router_and_keeps_shares_equal():
    from strixite_b200 import synth

    bias = synth.zipf_bias(99, 512)
    for world in (2, 4, 8):
        p = EP.placement(512, world, bias, 10, balanced=True)
        assert all(len(e) == 512 // world for e in p["experts_of"])
        assert sorted(np.concatenate(p["experts_of"]).tolist()) == list(range(512))
        for r in range(world):
            assert np.array_equal(p["local_of"][p["experts_of"][r]], np.arange(512 // world))
            assert (p["owner"][p["experts_of"][r]] == r).all()
        # estimated load per rank: within 10 % of the mean (contiguous blocks of this bias are off by far more)
        rng = np.random.default_rng(7)
        logits = rng.standard_normal((4096, 512)).astype(np.float32) * 0.82 + bias[None, :]
        picks = np.argpartition(-logits, 9, axis=1)[:, :10].reshape(-1)
        load = np.bincount(p["owner"][picks], minlength=world)
        assert load.max() / load.mean() < 1.10


def test_plan_reference_keeps_invalid_ids_home_and_counts_overflow():
    ids = np.array([[0, 5, 8], [-1, -1, -1], [3, 99, 8]], np.int32)
    coef = np.ones((3, 3), np.float32)
    p = EP.placement(8, 2, balanced=False)
    rowtok, meta, pos, flags = EP.plan_reference(ids, coef, 8, p["owner"], p["local_of"], 2, 1, 4, 12)
    assert not flags.any()
    # rank 1 is home: expert 0 and 3 go to rank 0; 5, the shared expert 8 and every invalid id stay on rank 1
    assert meta[0, 0] == 2 and meta[0, 1] == 2 and meta[1, 0] == 3 and meta[1, 1] == 7
    assert pos.tolist() == [[0, 0], [-1, 1], [1, 2]]
    slot = lambda r, j: meta[r, 4 + 8 + 3 * j: 4 + 8 + 3 * j + 3].tolist()  # noqa: E731
    assert slot(1, 2)[0] == -1 and slot(1, 5)[0] == -1  # the failed token's ids, the out-of-range id
    _, _, _, flags = EP.plan_reference(ids, coef, 8, p["owner"], p["local_of"], 2, 1, 2, 3)
    assert flags.tolist() == [3, 7]
