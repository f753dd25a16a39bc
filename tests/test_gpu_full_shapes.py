"""GPU: parity at the FULL sizes of the measured configurations (E = 512 experts of 2048 x 512, d = 4096 for the stack,
4096- and 16384-token prefill batches), through the same code the benchmark times. The oracle is evaluated on all rows of
the decode / verify workloads and on a seeded 64-row sample of the prefill batches (tokens are independent); routing is
checked on every row. FP32 activations: max |y - oracle| / max |oracle| per row <= 2e-3. BF16 activations: judged against
the evaluation that never rounds to BF16, within max(2e-3 + 2^-9, 1.25 x the oracle's own distance to it)."""
import types

import pytest

import bench

pytestmark = pytest.mark.gpu


def run_single(name, **override):
    import torch

    cfg = dict(bench.WORKLOADS[name])
    cfg.update(override)
    n = cfg["ring"]
    out = bench.measure_single(name, cfg, steps=n, warmup=3, rank=0, world=1, local=0, device="cuda:0", P=bench.peaks(), dist=None,
                               barrier=torch.cuda.synchronize, want_cpu=False, want_parity=True)
    return out["parity"]


@pytest.mark.parametrize("name", ("decode1", "verify6"))
def test_decode_and_verify_at_512_experts(name):
    p = run_single(name, ring=2)
    assert p["ids_equal"] and p["finite"]
    assert p["max_rel_err"] <= 2e-3, p
    assert p["ok"]


def test_stack_of_four_mixed_format_layers_at_d4096():
    p = run_single("stack4", ring=1)
    assert p["ids_equal"] and p["finite"]
    assert p["max_rel_err"] <= 2e-3, p


def test_prefill_4096_tokens_bf16():
    p = run_single("prefill4096", ring=1)
    assert p["ids_equal"] and p["ids_rows_checked"] == 4096 and p["finite"]
    assert p["gpu_vs_unrounded"] <= p["tolerance"], p
    assert p["ok"]


def test_prefill_4096_tokens_fp32_activations():
    """The same batch with FP32 activations (the tensor-core path rounds its operands to F16/BF16 inside; the outputs must
    still hold the 2e-3 contract)."""
    p = run_single("prefill4096", ring=1, act="f32", router="f32")
    assert p["ids_equal"] and p["finite"]
    assert p["max_rel_err"] <= 2e-3, p


def test_expert_parallel_batch_of_16384_tokens_on_one_rank():
    cfg = dict(bench.WORKLOADS["ep_prefill16384"])
    args = types.SimpleNamespace(ep_contiguous=False, ep_chunks=0, ep_all_to_all=False)
    out, _ = bench.run_ep(args, cfg, steps=2, warmup=3, rank=0, world=1, local=0, device="cuda:0", P=bench.peaks(), line={}, want_parity=True)
    p = out["parity"]
    assert p["ids_equal"] and p["ids_rows_checked"] == 16384 and p["finite"]
    assert p["gpu_vs_unrounded"] <= p["tolerance"], p
