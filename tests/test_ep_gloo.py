"""CPU, two gloo ranks: the expert-parallel exchange (strixite_b200/ep.py) with the oracle's functions plugged in as the
compute steps must reproduce the single-process oracle layer, whatever the number of ranks."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from helpers import make_layer, randn_act, rel_err_rows
from strixite_b200.ep import ExpertParallelMoe

E, K_TOP, D, I, T = 8, 3, 128, 64, 26


def _layer():
    return make_layer(77, d=D, I=I, E=E, k=K_TOP, G=32, router="f32", shared="stacked")


def _tokens():
    return randn_act(np.random.default_rng(78), (T, D), oracle.F32)


def _oracle_callables(L, world, rank):
    El = E // world

    def route(x):
        logits = oracle.linear_w(x.numpy(), L["router"], out_act=oracle.F32)
        if L.get("router_bias") is not None:
            logits[:, :E] += L["router_bias"]
        ids, coef, _ = oracle.moe_router(logits, E, K_TOP, shared_col=E, shared_id=E)
        return torch.from_numpy(ids), torch.from_numpy(coef)

    def experts(rows, local_ids, row_index):
        if row_index is not None:
            rows = rows[row_index.to(torch.int64)]
        loc = local_ids.numpy()
        assert ((loc >= 0) & (loc <= El)).all()
        gid = np.where(loc == El, E, rank * El + loc).astype(np.int32).reshape(-1, 1)  # back to ids of the full stacks
        h, _ = oracle.experts_gather(np.ascontiguousarray(rows.numpy()), L["gate_up"], gid, swiglu=True)
        y, _ = oracle.experts_combine(np.ascontiguousarray(h.reshape(-1, I)), L["down"], gid, np.ones_like(gid, dtype=np.float32))
        return torch.from_numpy(y)

    def reduce(partial, pos, ids, coef, out_dtype):
        p = partial.numpy()[pos.numpy().reshape(-1)].astype(np.float64).reshape(ids.shape[0], ids.shape[1], -1)
        return torch.from_numpy((coef.numpy().astype(np.float64)[:, :, None] * p).sum(axis=1).astype(np.float32))

    return route, experts, reduce


def _worker(rank, world, port, out_dir, dedup):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        L, x = _layer(), _tokens()
        lo, hi = rank * T // world, (rank + 1) * T // world  # uneven shares on purpose when T % world != 0
        ep = ExpertParallelMoe(E, K_TOP, world, rank, *_oracle_callables(L, world, rank), dedup=dedup)
        y = ep.forward(torch.from_numpy(x[lo:hi].copy()))
        # plan properties: a permutation of the slots, destinations ascending, slot order kept inside a destination
        order, loc, counts = ep.plan(ep.last["ids"])
        S = (hi - lo) * (K_TOP + 1)
        assert sorted(order.tolist()) == list(range(S)) and int(counts.sum()) == S
        flat = ep.last["ids"].reshape(-1).to(torch.int64)
        dest = torch.where(flat == E, torch.tensor(rank), flat // (E // world))[order]
        assert (dest[1:] >= dest[:-1]).all()
        same = dest[1:] == dest[:-1]
        assert (order[1:][same] > order[:-1][same]).all()
        assert ep.last["sent"] == counts.tolist()
        np.save(os.path.join(out_dir, "y%d.npy" % rank), y.numpy())
        np.save(os.path.join(out_dir, "recv%d.npy" % rank), np.array(ep.last["received"]))
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("dedup", (False, True))
@pytest.mark.parametrize("world", (1, 2))
def test_expert_parallel_exchange_matches_single_process(world, dedup, tmp_path):
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path), dedup), nprocs=world, join=True)
    y = np.concatenate([np.load(tmp_path / ("y%d.npy" % r)) for r in range(world)])
    want, it = oracle.moe_layer(_tokens(), _layer())
    assert y.shape == want.shape
    assert rel_err_rows(y, want) < 1e-5
    # every slot was delivered exactly once: received counts add up to all slots of all ranks
    assert sum(int(np.load(tmp_path / ("recv%d.npy" % r)).sum()) for r in range(world)) == T * (K_TOP + 1)


def test_plan_keeps_invalid_ids_home_and_invalid():
    ep = ExpertParallelMoe(8, 2, 4, 1, None, None, None)
    ids = torch.tensor([[0, 7, 8], [-1, 3, 8], [9, 2, 8]], dtype=torch.int32)
    order, loc, counts = ep.plan(ids)
    flat_dest = [0, 3, 1, 1, 1, 1, 1, 1, 1]  # shared (8) and invalid ids stay on rank 1
    assert counts.tolist() == [flat_dest.count(r) for r in range(4)]
    by_slot = dict(zip(order.tolist(), loc.tolist()))
    assert by_slot[0] == 0 and by_slot[1] == 1 and by_slot[2] == 2 and by_slot[3] == -1 and by_slot[4] == 1 and by_slot[6] == -1 and by_slot[7] == 0


def test_expert_count_must_divide():
    with pytest.raises(ValueError):
        ExpertParallelMoe(10, 2, 4, 0, None, None, None)
