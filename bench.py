"""Benchmark of the quantized MoE FFN layer on B200: MoE-layer tokens/s, with the HBM (decode) or tensor (prefill)
roofline of the dominant kernel and the CPU baseline timed beside it.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One "step" = one pass of the MoE layer over one batch of synthetic tokens. Workloads (the benchmark configurations):
  decode1      1 token,  d 2048, I 512, 512 experts top-10 + shared (stacked, gated), q4 G128, FP32 router      [config 1]
  verify6      6 tokens, same shapes, experts q4, router and shared expert (separate) q8 G64                   [config 2]
  ep_prefill16384  16384 BF16 tokens over all ranks, Zipf(1.1) router bias, the 512 experts sharded over the ranks (expert parallel:
               all-to-all dispatch and combine), strong scaling                                                  [config 5]
  prefill4096  4096 BF16 tokens, per-expert router bias N(0, 0.5), q4 experts, shared stacked                 [config 3]
  stack4       4 layers d 4096, I 1024, 6 tokens, per-expert q4/q5/q6/q8 60/15/15/10 %, residual adds          [config 4]
Weights are seeded N(0, 0.02) packed by the library's device quantizer; activations N(0, 1); there are no
checkpoints or datasets involved.

L2 hygiene: a ring of independent (layer weights, token batch) pairs is cycled, one per step, sized so that the
bytes touched between two uses of the same pair exceed the 126 MB L2 many times over (config.l2 says how).
Timing: CUDA events on the launching stream around exactly K steps replayed from CUDA graphs (one per ring entry),
after W warm-up steps; max over ranks.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    #               M     d     I     E    k  act    router  shared      mix                        bias   ring layers
    "decode1": dict(M=1, d=2048, I=512, E=512, k=10, act="f32", router="f32", shared="stacked", mix=None, bias=None, ring=24, layers=1),
    "verify6": dict(M=6, d=2048, I=512, E=512, k=10, act="f32", router="q8", shared="separate", mix=None, bias=None, ring=16, layers=1),
    "prefill4096": dict(M=4096, d=2048, I=512, E=512, k=10, act="bf16", router="bf16", shared="stacked", mix=None, bias=0.5, ring=2, layers=1, math=2),
    "ep_prefill16384": dict(M=16384, d=2048, I=512, E=512, k=10, act="bf16", router="bf16", shared="stacked", mix=None, bias="zipf", ring=2, layers=1,
                            math=2, ep=True),
    # grouped_min: these shapes do not fit the fused decode kernel; of the per-function paths the per-slot kernels measure faster
    # than the grouped ones at six tokens (1.6 ms against 4.9 ms per step), so the grouped path is switched off here
    "stack4": dict(M=6, d=4096, I=1024, E=512, k=10, act="f32", router="f32", shared="stacked", mix=[0.6, 0.15, 0.15, 0.1], bias=None, ring=2,
                   layers=4, grouped_min=1000),
}
G_EXPERTS = 128  # the served choice for the 4-bit classes (strixite docs/weights.md:19-26); not stated by the configs


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        j = json.load(open(p))
        return dict(hbm=float(j["hbm_gbs"]), tensor=float(j["bf16_tflops"]), tensor_sustained=float(j["bf16_tflops_sustained"]), source="measured")
    return dict(hbm=6650.0, tensor=1590.0, tensor_sustained=1400.0, source="fallback")


class ClockSampler:
    """SM clock and throttle reasons during the timed region: NVML polled from a thread every ~5 ms (read-only queries),
    nvidia-smi -lms as the fallback."""

    Q = "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown," \
        "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index):
        self.index, self.rows, self.proc, self.nv, self.stop_flag = index, [], None, None, False
        self.sm, self.mx, self.reason_bits = [], None, 0

    def start(self):
        try:
            import pynvml as nv

            nv.nvmlInit()
            # CUDA_VISIBLE_DEVICES may renumber devices: find the NVML handle by the CUDA device's PCI bus id
            import torch

            bus = torch.cuda.get_device_properties(self.index).pci_bus_id if hasattr(torch.cuda.get_device_properties(self.index), "pci_bus_id") else None
            self.h = None
            if bus is not None:
                for i in range(nv.nvmlDeviceGetCount()):
                    h = nv.nvmlDeviceGetHandleByIndex(i)
                    if nv.nvmlDeviceGetPciInfo(h).bus == bus:
                        self.h = h
            if self.h is None:
                self.h = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.mx = float(nv.nvmlDeviceGetMaxClockInfo(self.h, nv.NVML_CLOCK_SM))
            self.nv = nv
            self.t = threading.Thread(target=self._poll, daemon=True)
            self.t.start()
            return
        except Exception:  # noqa: BLE001  (no NVML binding: fall back to the command-line tool)
            self.nv = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _poll(self):
        nv = self.nv
        while not self.stop_flag:
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                self.reason_bits |= int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
            except Exception:  # noqa: BLE001
                pass
            time.sleep(0.005)

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.nv is not None:
            self.stop_flag = True
            self.t.join(timeout=2)
            nv = self.nv
            names = {"hw_slowdown": nv.nvmlClocksEventReasonHwSlowdown, "hw_thermal_slowdown": nv.nvmlClocksEventReasonHwThermalSlowdown,
                     "sw_thermal_slowdown": nv.nvmlClocksEventReasonSwThermalSlowdown, "sw_power_cap": nv.nvmlClocksEventReasonSwPowerCap}
            reasons = sorted(n for n, bit in names.items() if self.reason_bits & int(bit))
            return dict(sm_mhz=float(np.median(self.sm)) if self.sm else None, sm_max_mhz=self.mx, reasons=reasons, samples=len(self.sm), source="nvml")
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = [float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 9 for n, v in zip(names, r[5:9]) if v.lower().startswith("active")})
        return dict(sm_mhz=float(np.median(sm)) if sm else None, sm_max_mhz=max(mx) if mx else None, reasons=reasons, samples=len(sm), source="nvidia-smi")


def kernel_nodes(graph):
    """Kernel nodes of a captured step = kernels launched per replay."""
    try:
        from cuda.bindings import runtime as rt

        raw = graph.raw_cuda_graph()
        err, _, n = rt.cudaGraphGetNodes(raw, 0)
        err, nodes, n = rt.cudaGraphGetNodes(raw, n)
        k = 0
        for nd in nodes[:n]:
            err, ty = rt.cudaGraphNodeGetType(nd)
            k += int(ty == rt.cudaGraphNodeType.cudaGraphNodeTypeKernel)
        return k
    except Exception:  # noqa: BLE001
        return None


def bytes_of_weight(N, Kdim, bits, G):
    return N * (Kdim * bits // 8 + 4 * (Kdim // G))


def algorithmic_bytes(cfg, layer, ids, info):
    """Bytes one step must read: every DISTINCT active expert's packed weights once, the router, the separate shared
    expert, plus the activations in and out (the benchmark's accounting; padding and re-reads are not work)."""
    d, I, M, E = cfg["d"], cfg["I"], cfg["M"], cfg["E"]
    distinct = np.unique(ids[ids >= 0])
    if cfg["mix"] is None:
        per = bytes_of_weight(2 * I, d, 4, G_EXPERTS) + bytes_of_weight(d, I, 4, G_EXPERTS)
        total = per * len(distinct)
    else:
        gb, db = info["gate_up_bits"], info["down_bits"]
        total = sum(bytes_of_weight(2 * I, d, int(gb[e]), G_EXPERTS) + bytes_of_weight(d, I, int(db[e]), G_EXPERTS) for e in distinct)
    R = layer.router_rows
    total += {"f32": R * d * 4, "bf16": R * d * 2, "q8": bytes_of_weight(R, d, 8, 64)}[cfg["router"]]
    if cfg["shared"] == "separate":
        total += bytes_of_weight(2 * I, d, 8, 64) + bytes_of_weight(d, I, 8, 64)
    es = 4 if cfg["act"] == "f32" else 2
    return int(total + 2 * M * d * es), int(len(distinct))


def flops_of(cfg, A):
    return 2.0 * cfg["M"] * A * 3 * cfg["I"] * cfg["d"] + 2.0 * cfg["M"] * cfg["E"] * cfg["d"]


def build_ring(cfg, rank, device):
    import torch

    from strixite_b200 import kernels as K
    from strixite_b200 import synth

    act = K.Act.F32 if cfg["act"] == "f32" else K.Act.BF16
    ring = []
    g = torch.Generator(device=device)
    for r in range(cfg["ring"]):
        layers = []
        for l in range(cfg["layers"]):
            seed = 1000 * (rank + 1) + 100 * r + 10 * l
            bias = None
            if cfg["bias"] == "zipf":
                bias = synth.zipf_bias(seed + 7, cfg["E"])
            elif cfg["bias"] is not None:
                bias = (np.random.default_rng(seed + 7).standard_normal(cfg["E"]) * cfg["bias"]).astype(np.float32)
            layers.append(synth.make_layer(seed, cfg["d"], cfg["I"], cfg["E"], cfg["k"], act, G=G_EXPERTS, router=cfg["router"], shared=cfg["shared"],
                                           mix=cfg["mix"], bias=bias, max_tokens=cfg["M"], grouped_min_tokens=cfg.get("grouped_min", 6),
                                           math=cfg.get("math", 0), decode_impl=cfg.get("decode_impl", 0), tensor_min_tokens=cfg.get("tensor_min_tokens", 0), device=device))
        g.manual_seed(7000 + 100 * rank + r)
        x = torch.randn((cfg["M"], cfg["d"]), generator=g, device=device, dtype=torch.float32)
        x = x if cfg["act"] == "f32" else x.to(torch.bfloat16)
        ring.append(dict(layers=layers, x=x, y=torch.empty_like(x), tmp=torch.empty_like(x)))
    return ring


def step(entry, stream=None):
    from strixite_b200 import layer as SL

    if len(entry["layers"]) == 1:
        entry["layers"][0].forward(entry["x"], entry["y"], stream)
    else:  # the stack: x <- x + moe_l(x); run on a scratch copy so every step sees the same input
        entry["y"].copy_(entry["x"])
        SL.stack_forward(entry["layers"], entry["y"], entry["tmp"], stream)


def capture(ring):
    import torch

    graphs = []
    for e in ring:
        g = torch.cuda.CUDAGraph(keep_graph=True)
        with torch.cuda.graph(g):
            step(e)
        g.instantiate()
        graphs.append(g)
    return graphs


def time_steps(run_one, n, steps, warmup, barrier):
    import torch

    for i in range(warmup):
        run_one(i % n)
    torch.cuda.synchronize()
    barrier()
    torch.cuda.cudart().cudaProfilerStart()  # lets `ncu --profile-from-start off` see the timed steps only; a no-op otherwise
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        run_one((warmup + i) % n)
    e1.record()
    torch.cuda.synchronize()
    torch.cuda.cudart().cudaProfilerStop()
    barrier()
    return e0.elapsed_time(e1)  # ms


def cpu_layer_from(layer_obj, cfg):
    """The oracle-side twin of one device layer (weights downloaded), for the CPU baseline."""
    import oracle

    w = layer_obj.weights

    def host_q(qw):
        q, s, m = qw.to_host()
        return oracle.QWeight(qw.bits, qw.N, qw.K, qw.G, q, s, m)

    def host_stack(st, E):
        from strixite_b200 import kernels as K

        if isinstance(st, K.QMixStack):
            return oracle.ExpertStack(st.E, st.N, st.K, st.G, st.q.cpu().numpy(), st.scale.cpu().numpy().view(np.uint16),
                                      st.minv.cpu().numpy().view(np.uint16), bits=0, bits_tab=st.bits.cpu().numpy(), q_off=st.q_off.cpu().numpy())
        return oracle.ExpertStack.from_weight(host_q(st), E)

    Es = cfg["E"] + (1 if cfg["shared"] == "stacked" else 0)
    r = w["router"]
    if hasattr(r, "bits"):
        router = host_q(r)
    elif str(r.dtype) == "torch.bfloat16":
        import torch

        router = r.view(torch.int16).cpu().numpy().view(np.uint16)
    else:
        router = r.cpu().numpy()
    L = dict(E=cfg["E"], k=cfg["k"], router=router, shared=cfg["shared"], shared_coef="sigmoid", gate_up=host_stack(w["gate_up"], Es),
             down=host_stack(w["down"], Es))
    if cfg["shared"] == "separate":
        L["sh_gate_up"], L["sh_down"] = host_q(w["sh_gate_up"]), host_q(w["sh_down"])
    if "router_bias" in w:
        L["router_bias"] = w["router_bias"].cpu().numpy()
    return L


def cpu_baseline(ring, cfg, budget_s=12.0, max_tokens=None):
    """The CPU path (oracle/moe_baseline.cpp, all host threads) on a bounded sample of the same workload: the first ring
    entry's layer(s) and tokens, repeated until ~budget_s of CPU work."""
    import oracle

    e = ring[0]
    Ls = [cpu_layer_from(l, cfg) for l in e["layers"]]
    x = e["x"]
    import torch

    xh = x.view(torch.int16).cpu().numpy().view(np.uint16) if x.dtype == torch.bfloat16 else x.cpu().numpy()
    M = xh.shape[0] if max_tokens is None else min(max_tokens, xh.shape[0])
    xh = np.ascontiguousarray(xh[:M])

    def one():
        if len(Ls) == 1:
            return oracle.moe_layer(xh, Ls[0], use_fast=True)[0]
        xr = xh.copy()
        for L in Ls:
            y = oracle.moe_layer(xr, L, use_fast=True)[0]
            oracle.residual_add(xr, y)
        return xr

    one()
    t0, n = time.perf_counter(), 0
    while True:
        one()
        n += 1
        dt = time.perf_counter() - t0
        if dt > budget_s or n >= 200:
            break
    return dict(value=M * n / dt, unit="tokens/s", cores=oracle.fast_threads(), kind="port",
                sample="%d passes of %d token(s) through ring entry 0 (%d layer(s)), %.1f s" % (n, M, len(Ls), dt)), one


def run_ep(args, cfg, rank, world, local, device, dist, barrier, line, P):
    """Config 5: one layer, its routed experts sharded over the ranks, the token batch split evenly (strong scaling)."""
    import torch

    from strixite_b200 import ep as EP
    from strixite_b200 import kernels as K
    from strixite_b200 import synth

    if dist is None:  # one rank: the same code path over a one-rank group
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device(device))
        barrier = lambda: None  # noqa: E731
    d, I, E, k, T = cfg["d"], cfg["I"], cfg["E"], cfg["k"], cfg["M"]
    Tl = T // world
    g = torch.Generator(device=device)
    g.manual_seed(4242)
    rw = (torch.randn((E + 1, d), generator=g, device=device, dtype=torch.float32) * 0.02).to(torch.bfloat16)  # replicated: same seed everywhere
    bias = torch.from_numpy(synth.zipf_bias(99, E)).to(device)
    gu = synth.quantized_normal(501, 4, (E + 1) * 2 * I, d, G_EXPERTS, device=device)
    dn = synth.quantized_normal(502, 4, (E + 1) * d, I, G_EXPERTS, device=device)
    gu_l, dn_l = EP.shard_stack(gu, E, world, rank), EP.shard_stack(dn, E, world, rank)
    del gu, dn
    torch.cuda.empty_cache()
    # capacity: with Zipf routing the hot rank receives several times the mean; 3x the mean plus the shared slots, checked below
    cap = min(T * (k + 1), 3 * T * k // world + Tl + 4096)
    layer = EP.cuda_layer(d, I, E, k, K.Act.BF16, rw, bias, gu_l, dn_l, world, rank, max_local_tokens=Tl, capacity=cap, dedup=not args.ep_exact)
    xs = []
    for r in range(cfg["ring"]):
        g.manual_seed(9000 + 17 * r)
        xs.append(torch.randn((T, d), generator=g, device=device, dtype=torch.float32)[rank * Tl:(rank + 1) * Tl].to(torch.bfloat16).contiguous())
    for i in range(max(3, args.warmup)):
        y = layer.forward(xs[i % len(xs)])
    torch.cuda.synchronize()
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    torch.cuda.cudart().cudaProfilerStart()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    recv = []
    for i in range(args.steps):
        y = layer.forward(xs[i % len(xs)])
        recv.append(sum(layer.last["received"]))
    e1.record()
    torch.cuda.synchronize()
    torch.cuda.cudart().cudaProfilerStop()
    barrier()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1)
    stats = torch.tensor([ms, float(np.mean(recv))], device=device)
    mx = stats.clone()
    dist.all_reduce(mx, op=dist.ReduceOp.MAX)
    sm = stats.clone()
    dist.all_reduce(sm, op=dist.ReduceOp.SUM)
    ms = float(mx[0].item())
    # end to end: host tokens in, host outputs back, every step
    xh = [x.cpu().pin_memory() for x in xs]
    yh = torch.empty_like(xh[0]).pin_memory()
    ke = max(3, args.steps // 4)
    barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for i in range(ke):
        xd = xh[i % len(xh)].to(device, non_blocking=True)
        yh.copy_(layer.forward(xd), non_blocking=True)
        torch.cuda.synchronize()
    dt = torch.tensor([time.perf_counter() - t0], device=device)
    dist.all_reduce(dt, op=dist.ReduceOp.MAX)
    fl = 2.0 * T * (k + 1) * 3 * I * d + 2.0 * T * (E + 1) * d
    step_s = ms * 1e-3 / args.steps
    line["scaling"] = "strong"
    line["config"].update(parallelism="expert parallel x%d (experts e -> rank e / %d, tokens split evenly, shared expert replicated; %s)" % (world, E // world, "one row per slot" if args.ep_exact else "one row per (token, rank), summed on the expert rank"),
                          router_bias="Zipf(1.1)", tokens_per_step=T, l2="two token sets alternate; every step streams far more than the 126 MB L2")
    line.update(value=T / step_s, ms_per_step=ms / args.steps, clocks=clocks)
    line["e2e"] = dict(value=T * ke / float(dt.item()), unit="tokens/s", h2d_bytes_per_step=int(xh[0].numel() * 2 * world), d2h_bytes_per_step=int(yh.numel() * 2 * world),
                       steps=ke, note="pinned host tokens -> device -> expert-parallel layer -> pinned host outputs, per rank, wall clock, max over ranks")
    ach = fl / step_s / 1e12
    line["roofline"] = dict(bound="tensor", achieved=ach, peak=P["tensor"] * world, unit="TFLOP/s", frac=ach / (P["tensor"] * world), traffic=None,
                            peak_source=P["source"], algorithmic_flops_per_step=fl, kernel="whole step, all ranks",
                            load_imbalance_max_over_mean_slots=float(mx[1].item() / (sm[1].item() / world)))
    line["gpu_launches"] = None
    line["gpu_launches_note"] = "per step and rank: 2 router kernels, grouping, tiles, gather, 2 tcgen05 FFN kernels, reduce, plus torch index kernels and 4 NCCL collectives"
    if rank == 0:
        print(json.dumps(line))
    dist.barrier()
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=50)
    ap.add_argument("--workload", default="verify6", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--ring", type=int, default=0, help="override the number of independent (weights, tokens) pairs cycled (a small ring keeps a profiler capture small)")
    ap.add_argument("--tensor-min-tokens", type=int, default=0, help="with --math 2: run forwards of at least this many tokens on the tensor-core path")
    ap.add_argument("--math", type=int, default=-1, choices=[-1, 0, 1, 2], help="override the workload's MoeMath (0 = FP32 kernels, 1/2 = tensor cores)")
    ap.add_argument("--ep-exact", action="store_true", help="expert parallel: one row per slot both ways (bit-identical to one GPU) instead of one per (token, rank)")
    ap.add_argument("--grouped-min", type=int, default=0, help="override the token count from which the grouped expert path runs (reference: 6)")
    ap.add_argument("--decode-impl", type=int, default=0, choices=[0, 1], help="forwards of <= 8 tokens: 0 = the fused kernel, 1 = the per-function kernels")
    args = ap.parse_args()
    cfg = dict(WORKLOADS[args.workload])
    cfg["decode_impl"] = args.decode_impl
    if args.grouped_min > 0:
        cfg["grouped_min"] = args.grouped_min
    cfg["tensor_min_tokens"] = args.tensor_min_tokens
    if args.math >= 0:
        cfg["math"] = args.math
    if args.ring > 0:
        cfg["ring"] = args.ring
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if args.warmup < 3:
        args.warmup = 3

    # torchrun sets OMP_NUM_THREADS=1 for its workers; the CPU legs (rank 0 only) are meant to use every host core
    os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)

    import torch

    import oracle  # noqa: F401  (the CPU legs only)

    if args.impl == "reference" and rank != 0:
        return
    torch.cuda.set_device(local)
    device = "cuda:%d" % local
    if world > 1 and args.impl != "reference":
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device(device))
        barrier = lambda: dist.barrier()  # noqa: E731
    else:
        dist, barrier = None, (lambda: None)

    P = peaks()
    line = dict(metric="MoE-layer tokens/s", unit="tokens/s", n_gpus=args.gpus, steps=args.steps, warmup=args.warmup, higher_is_better=True,
                scaling="weak", vs_baseline=None, dtype="f32" if cfg["act"] == "f32" else "bf16", data="synthetic")
    line["config"] = dict(workload=args.workload, tokens_per_step=cfg["M"], hidden=cfg["d"], intermediate=cfg["I"], experts=cfg["E"], top_k=cfg["k"],
                          shared_expert=cfg["shared"], shared_coef="sigmoid", expert_format="q4" if cfg["mix"] is None else "q4/q5/q6/q8 60/15/15/10",
                          group_size=G_EXPERTS, router=cfg["router"], layers_per_step=cfg["layers"], parallelism="replicas x%d" % world,
                          l2="ring of %d independent (weights, tokens) pairs cycled one per step; bytes between reuses >> 126 MB L2" % cfg["ring"])

    if args.impl == "reference":
        # The reference arm: the CPU path on the host cores, a bounded sample per step.
        cfg["ring"] = 1
        cfg.pop("ep", None)  # the CPU path has no ranks: the whole layer on the host cores
        sample = min(cfg["M"], 256)  # a bounded sample of the batch per pass
        cfg_small = dict(cfg, M=sample, math=0)
        ring = build_ring(cfg_small, 0, device)
        base, one = cpu_baseline(ring, cfg_small, budget_s=3.0)
        for _ in range(max(0, min(args.warmup, 3) - 1)):
            one()
        k = max(1, min(args.steps, 20))
        t0 = time.perf_counter()
        for _ in range(k):
            one()
        dt = time.perf_counter() - t0
        v = sample * k / dt
        line.update(impl="reference", value=v, steps=k, ms_per_step=1e3 * dt / k, n_gpus=args.gpus, gpu_launches=0,
                    cpu_baseline=dict(value=v, unit="tokens/s", cores=base["cores"], kind="port",
                                      sample="%d timed passes of %d token(s) of the batch, one layer set" % (k, sample)),
                    e2e=dict(value=v, unit="tokens/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0))
        print(json.dumps(line))
        return

    if cfg.get("ep"):
        run_ep(args, cfg, rank, world, local, device, dist, barrier, line, P)
        return
    ring = build_ring(cfg, rank, device)
    n = len(ring)
    for e in ring:  # warm every entry once outside any capture (first-call set-up, lazy module loads)
        step(e)
    torch.cuda.synchronize()
    graphs = capture(ring)
    sampler = ClockSampler(local)
    sampler.start()
    ms = time_steps(lambda i: graphs[i].replay(), n, args.steps, args.warmup, barrier)
    clocks = sampler.stop()
    if dist is not None:
        t = torch.tensor([ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    tokens = cfg["M"] * args.steps * world
    line.update(value=tokens / (ms * 1e-3), ms_per_step=ms / args.steps, clocks=clocks)

    # End to end through the host-buffer entry point: pinned staging, H2D, the layer, D2H of y and the error words, one sync.
    e2e = None
    if cfg["layers"] == 1:
        xs = [e["x"].cpu() for e in ring]
        xh = [(x.view(torch.int16).numpy().view(np.uint16) if x.dtype == torch.bfloat16 else x.numpy()) for x in xs]
        yh = np.empty_like(xh[0])
        for i in range(3):
            ring[i % n]["layers"][0].forward_host(xh[i % n], yh)
        barrier()
        ke = max(10, args.steps // 4)
        t0 = time.perf_counter()
        for i in range(ke):
            ring[i % n]["layers"][0].forward_host(xh[i % n], yh)
        dt = time.perf_counter() - t0
        if dist is not None:
            t = torch.tensor([dt], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dt = float(t.item())
        e2e = dict(value=cfg["M"] * ke * world / dt, unit="tokens/s", h2d_bytes_per_step=int(xh[0].nbytes), d2h_bytes_per_step=int(yh.nbytes + 24),
                   steps=ke, note="strix_moe_layer_forward_host: host buffers in and out, copies and the sync inside the timed region (wall clock)")
    line["e2e"] = e2e

    if rank == 0:
        # Roofline of the step: algorithmic bytes (decode) or flops (prefill) over the event-timed step.
        l0 = ring[0]["layers"][0]
        A = l0.A
        per_step_bytes, distinct = [], []
        for e in ring:
            tot = 0
            for l in e["layers"]:
                ids = l.probe("router_ids", cfg["M"]).cpu().numpy()
                b, nd = algorithmic_bytes(cfg, l, ids, getattr(l, "info", {}))
                tot += b
                distinct.append(nd)
            per_step_bytes.append(tot)
        step_s = ms * 1e-3 / args.steps
        if cfg["M"] <= 64:
            ach = float(np.mean(per_step_bytes)) / step_s / 1e9
            line["roofline"] = dict(bound="hbm", achieved=ach, peak=P["hbm"], unit="GB/s", frac=ach / P["hbm"], traffic=None, peak_source=P["source"],
                                    frac_of_nominal_8TBs=ach / 8000.0, algorithmic_bytes_per_step=float(np.mean(per_step_bytes)),
                                    distinct_experts_per_layer=float(np.mean(distinct)), kernel="whole step (all launches of one layer pass)")
        else:
            fl = flops_of(cfg, A)
            ach = fl / step_s / 1e12
            line["roofline"] = dict(bound="tensor", achieved=ach, peak=P["tensor"], unit="TFLOP/s", frac=ach / P["tensor"], traffic=None,
                                    peak_source=P["source"], algorithmic_flops_per_step=fl, kernel="whole step")
        per_step = [kernel_nodes(g) for g in graphs]
        if any(k is None for k in per_step):
            raise RuntimeError("could not count the kernel nodes of the captured steps")
        line["gpu_launches"] = int(sum(per_step[(args.warmup + i) % n] for i in range(args.steps)))
        line["gpu_launches_per_step"] = float(np.mean(per_step))
        if not args.no_cpu_baseline:
            line["cpu_baseline"], _ = cpu_baseline(ring, cfg, max_tokens=256 if cfg["M"] > 256 else None)
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
