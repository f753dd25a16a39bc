"""GPU: the expert-parallel layer (strixite_b200/ep.py over the CUDA library and NCCL) against the single-device layer
object on the same weights and tokens. One rank in the test process always; two ranks as child processes where the
machine has two GPUs."""
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


def _run_rank(rank, world, port, out_dir, dedup):
    from strixite_b200 import ep as EP
    from strixite_b200 import kernels as K

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        L, x = _layer(), _tokens()
        lo, hi = rank * T // world, (rank + 1) * T // world
        rw = torch.from_numpy(L["router"].view(np.int16)).cuda().view(torch.bfloat16)
        bias = torch.from_numpy(L["router_bias"]).cuda()
        gu, dn = upload_stack(L["gate_up"]), upload_stack(L["down"])
        layer = EP.cuda_layer(D, I, E, K_TOP, K.Act.BF16, rw, bias, EP.shard_stack(gu, E, world, rank), EP.shard_stack(dn, E, world, rank), world,
                              rank, max_local_tokens=hi - lo + 1, dedup=dedup)
        y = layer.forward(to_torch_act(x[lo:hi].copy()))
        y2 = layer.forward(to_torch_act(x[lo:hi].copy()))  # a second pass through the same buffers
        torch.cuda.synchronize()
        assert torch.equal(y, y2)
        assert K.umma_abort_count() == 0
        np.save(os.path.join(out_dir, "y%d.npy" % rank), to_np_act(y))
    finally:
        dist.destroy_process_group()


def _check(world, tmp_path, dedup):
    y = np.concatenate([np.load(tmp_path / ("y%d.npy" % r)) for r in range(world)])
    L, x = _layer(), _tokens()
    single = gpu_layer(L, oracle.BF16, T, math=2)
    want = to_np_act(single.forward(to_torch_act(x)))
    if not dedup:
        # the same kernels on the same rows, summed in the same order: the sharded layer reproduces the single-device bits
        assert np.array_equal(y, want)
    else:
        # one row per (token, rank), summed per rank first: another association of the same FP32 sum - the BF16 outputs
        # differ from the single-device ones in a few elements, by one BF16 step
        assert (y != want).mean() < 0.02
        assert rel_err_rows(oracle.to_f32(y), oracle.to_f32(want)) < 2.0 ** -7
    ref, _ = oracle.moe_layer(x, L)
    assert rel_err_rows(oracle.to_f32(y), oracle.to_f32(ref)) < 2e-3 + 2 ** -6


@pytest.mark.parametrize("dedup", (False, True))
def test_expert_parallel_one_rank_equals_layer(tmp_path, dedup):
    _run_rank(0, 1, _free_port(), str(tmp_path), dedup)
    _check(1, tmp_path, dedup)


@pytest.mark.parametrize("dedup", (False, True))
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_expert_parallel_two_ranks_equal_layer(tmp_path, dedup):
    mp.spawn(_run_rank, args=(2, _free_port(), str(tmp_path), dedup), nprocs=2, join=True)
    _check(2, tmp_path, dedup)
