"""Benchmark of the quantized MoE FFN layer on B200: MoE-layer tokens/s, with the HBM (decode) or tensor (prefill)
roofline of the step, a parity check of what was timed, and the CPU baseline timed beside it.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One "step" = one pass of the MoE layer over one batch of synthetic tokens. Workloads (the benchmark configurations):
  decode1      1 token,  d 2048, I 512, 512 experts top-10 + shared (stacked, gated), q4 G128, FP32 router      [config 1]
  verify6      6 tokens, same shapes, experts q4, router and shared expert (separate) q8 G64                   [config 2]
  prefill4096  4096 BF16 tokens, per-expert router bias N(0, 0.5), q4 experts, shared stacked                 [config 3]
  stack4       4 layers d 4096, I 1024, 6 tokens, per-expert q4/q5/q6/q8 60/15/15/10 %, residual adds          [config 4]
  ep_prefill16384  16384 BF16 tokens over all ranks, Zipf(1.1) router bias, the 512 experts sharded over the ranks (expert
               parallel: all-to-all dispatch and combine), strong scaling                                      [config 5]
With no --workload the line is ep_prefill16384 - the largest configuration, the only one that shards, the same code path at
every N - and, on one GPU, the other four are measured in the same process and attached under "workloads", each with its
own ms_per_step, roofline, e2e and parity. Weights are seeded N(0, 0.02) packed by the library's device quantizer
(bit-identical to the reference's host quantizer); activations N(0, 1); there are no checkpoints or datasets involved.

L2 hygiene: a ring of independent (layer weights, token batch) pairs is cycled, one per step, sized so that the bytes
touched between two uses of the same pair exceed the 126 MB L2 many times over (config.l2 says how).
Timing: CUDA events on the launching stream around exactly K steps after W warm-up steps; max over ranks. The steps of a
ring are captured in ONE CUDA graph (a step per ring entry, in order), replayed K / ring times, plus a shorter graph for the
remainder: the step-to-step launch gap is the graph's, not Python's.
Parity: outside the timed region, the output of ring entry 0 is compared with the CPU oracle (oracle/) on the same inputs -
every row for the small batches, a seeded sample of rows for the large ones (tokens are independent) - and the routing
ids of ALL rows against the oracle's router run on the GPU-produced logits.
"""
import argparse
import datetime
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
    "decode1": dict(M=1, d=2048, I=512, E=512, k=10, act="f32", router="f32", shared="stacked", mix=None, bias=None, ring=24, layers=1, steps=480),
    "verify6": dict(M=6, d=2048, I=512, E=512, k=10, act="f32", router="q8", shared="separate", mix=None, bias=None, ring=16, layers=1, steps=480),
    "prefill4096": dict(M=4096, d=2048, I=512, E=512, k=10, act="bf16", router="bf16", shared="stacked", mix=None, bias=0.5, ring=2, layers=1, math=2,
                        steps=20),
    "ep_prefill16384": dict(M=16384, d=2048, I=512, E=512, k=10, act="bf16", router="bf16", shared="stacked", mix=None, bias="zipf", ring=2, layers=1,
                            math=2, ep=True, steps=20),
    "stack4": dict(M=6, d=4096, I=1024, E=512, k=10, act="f32", router="f32", shared="stacked", mix=[0.6, 0.15, 0.15, 0.1], bias=None, ring=2,
                   layers=4, steps=100),
}
G_EXPERTS = 128  # the served choice for the 4-bit classes (strixite docs/weights.md:19-26); not stated by the configs
LAYER_TOL = 2e-3  # max |y - oracle| / max |oracle| per row
BF16_STEP = 2.0 ** -9  # half a BF16 step relative to the element: what rounding the output itself to BF16 can move it by

# DRAM bytes (read + write) of the dominant kernel per launch, from ncu captures of small rings of the same workloads; the
# summaries with the full commands are in profiles/. Constants from a profile, not measured in this run.
TRAFFIC = {
    "decode1": dict(bytes=22.68e6, kernel="decode_stream_kernel", source="profiles/decode_stream_kernel_decode1_verify6.md"),
    "verify6": dict(bytes=101.13e6, kernel="decode_stream_kernel", source="profiles/decode_stream_kernel_decode1_verify6.md"),
    "stack4": dict(bytes=479.15e6, kernel="decode_stream_kernel (one launch = one of the 4 layers)", source="profiles/decode_stream_kernel_stack4.md"),
    "prefill4096": dict(bytes=779.07e6, kernel="ffn_umma_kernel<0, 128, 0>", source="profiles/ffn_umma_kernel_prefill4096.md"),
    "ep_prefill16384": dict(bytes=1144.18e6, kernel="ffn_umma_kernel<0, 128, 2> (one GPU, 16384 tokens)", source="profiles/ffn_umma_kernel_ep_prefill16384.md"),
}


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
    """Kernel nodes of a captured graph = kernels launched per replay."""
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
    d, I, M = cfg["d"], cfg["I"], cfg["M"]
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


def capture(entries):
    """One CUDA graph holding a step per entry, in order."""
    import torch

    g = torch.cuda.CUDAGraph(keep_graph=True)
    with torch.cuda.graph(g):
        for e in entries:
            step(e)
    g.instantiate()
    return g


def time_steps(full, rest, n, steps, warmup, barrier):
    """Exactly `steps` steps: steps // n replays of the ring's graph and one of the graph of the first steps % n entries."""
    import torch

    for _ in range((warmup + n - 1) // n):
        full.replay()
    torch.cuda.synchronize()
    barrier()
    torch.cuda.cudart().cudaProfilerStart()  # lets `ncu --profile-from-start off` see the timed steps only; a no-op otherwise
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps // n):
        full.replay()
    if rest is not None:
        rest.replay()
    e1.record()
    torch.cuda.synchronize()
    torch.cuda.cudart().cudaProfilerStop()
    barrier()
    return e0.elapsed_time(e1)  # ms


def host_act(x):
    """A torch activation tensor as the oracle's numpy form (float32, or uint16 BF16 bits)."""
    import torch

    return x.view(torch.int16).cpu().numpy().view(np.uint16) if x.dtype == torch.bfloat16 else x.cpu().numpy()


def cpu_layer_from(layer_obj, cfg):
    """The oracle-side twin of one device layer (weights downloaded), for the CPU baseline and the parity check."""
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


def rel_err_rows(y, ref):
    y, ref = np.asarray(y, np.float64), np.asarray(ref, np.float64)
    return float((np.abs(y - ref).max(axis=1) / np.maximum(np.abs(ref).max(axis=1), 1e-30)).max())


def parity_of(x_rows, y_rows, Ls, logits_all, ids_all, gated_stacked, rows_note):
    """Compares the GPU output rows with the oracle on the same inputs (x_rows / y_rows in the oracle's numpy form; Ls: the
    layer dicts applied in sequence with residual adds when more than one). Routing: the oracle's router on the GPU-produced
    logits of ALL rows (last layer for a stack) must give the same ids bit for bit. BF16 activations: the GPU's and the oracle's
    distances to an evaluation that never rounds to BF16 (FP32 activations, double accumulation) are reported side by side; the
    allowance is the contract plus what rounding the output itself to BF16 moves an element by."""
    import oracle

    bf16 = x_rows.dtype == np.uint16

    def run(x):
        if len(Ls) == 1:
            return oracle.moe_layer(x, Ls[0])
        xr = x.copy()
        it = None
        for L in Ls:
            y, it = oracle.moe_layer(xr, L)
            oracle.residual_add(xr, y)
        return xr, it

    t0 = time.perf_counter()
    want, it = run(x_rows)
    E, k = Ls[-1]["E"], Ls[-1]["k"]
    ids_ref, _, _ = oracle.moe_router(np.ascontiguousarray(logits_all), E, k, shared_col=E if gated_stacked else None, shared_id=E)
    ids_equal = bool(np.array_equal(ids_all[:, : ids_ref.shape[1]], ids_ref))
    got_f, want_f = oracle.to_f32(y_rows), oracle.to_f32(want)
    out = dict(metric="max |y - oracle| / max |oracle| per row", max_rel_err=rel_err_rows(got_f, want_f), rows_checked=int(x_rows.shape[0]),
               rows=rows_note, ids_equal=ids_equal, ids_rows_checked=int(ids_all.shape[0]), finite=bool(np.isfinite(got_f).all()))
    if bf16:
        truth, _ = run(oracle.bf16_to_f32(x_rows))
        g_t, o_t = rel_err_rows(got_f, truth), rel_err_rows(want_f, truth)
        tol = max(LAYER_TOL + BF16_STEP, 1.25 * o_t)
        out.update(gpu_vs_unrounded=g_t, oracle_vs_unrounded=o_t, tolerance=tol,
                   tolerance_note="BF16 activations round gate, up, silu, h and y to BF16 (the reference's arithmetic); that alone puts the oracle "
                                  "oracle_vs_unrounded away from the evaluation that never rounds to BF16, and two pipelines that round cannot agree closer "
                                  "than that. The GPU is judged against the unrounded evaluation: within max(2e-3 + 2^-9, 1.25 x oracle_vs_unrounded)")
        out["ok"] = bool(g_t <= tol and ids_equal and out["finite"])
    else:
        out.update(tolerance=LAYER_TOL)
        out["ok"] = bool(out["max_rel_err"] <= LAYER_TOL and ids_equal and out["finite"])
    out["oracle_seconds"] = round(time.perf_counter() - t0, 2)
    return out


def cpu_baseline(Ls, xh, budget_s=12.0, max_tokens=None):
    """The CPU path (oracle/moe_baseline.cpp, all host threads) on a bounded sample of the workload: the layer(s) of ring
    entry 0 and (a prefix of) its tokens, repeated until ~budget_s of CPU work."""
    import oracle

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


def measure_single(name, cfg, steps, warmup, rank, world, local, device, P, dist, barrier, want_cpu, want_parity):
    """One non-sharded workload on this rank's GPU (N ranks = N independent replicas): the measured fields of its line."""
    import torch

    ring = build_ring(cfg, rank, device)
    n = len(ring)
    for e in ring:  # warm every entry once outside any capture (first-call set-up, lazy module loads)
        step(e)
    torch.cuda.synchronize()
    full = capture(ring)
    rest = capture(ring[: steps % n]) if steps % n else None
    sampler = ClockSampler(local)
    sampler.start()
    ms = time_steps(full, rest, n, steps, warmup, barrier)
    clocks = sampler.stop()
    if dist is not None:
        t = torch.tensor([ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    out = dict(value=cfg["M"] * steps * world / (ms * 1e-3), unit="tokens/s", steps=steps, warmup=warmup, ms_per_step=ms / steps, clocks=clocks,
               dtype="f32" if cfg["act"] == "f32" else "bf16")

    # End to end through the host-buffer entry point: pinned staging, H2D, the layer(s), D2H of y (and the error words), one sync.
    xs = [e["x"].cpu() for e in ring]
    ke = max(10, steps // 4)
    if cfg["layers"] == 1:
        # page-locked host buffers: the entry point copies from and to them directly
        pinned = [x.view(torch.int16).pin_memory() if x.dtype == torch.bfloat16 else x.pin_memory() for x in xs]
        xh = [t.numpy().view(np.uint16) if t.dtype == torch.int16 else t.numpy() for t in pinned]
        y_pin = torch.empty_like(pinned[0]).pin_memory()
        yh = y_pin.numpy().view(np.uint16) if y_pin.dtype == torch.int16 else y_pin.numpy()
        for i in range(3):
            ring[i % n]["layers"][0].forward_host(xh[i % n], yh)
        barrier()
        t0 = time.perf_counter()
        for i in range(ke):
            ring[i % n]["layers"][0].forward_host(xh[i % n], yh)
        dt = time.perf_counter() - t0
        h2d, d2h, note = int(xh[0].nbytes), int(yh.nbytes + 24), "strix_moe_layer_forward_host (page-locked host buffers)"
    else:
        from strixite_b200 import layer as SL

        xp = [x.pin_memory() for x in xs]
        yp = torch.empty_like(xp[0]).pin_memory()

        def one(i):
            e = ring[i % n]
            e["y"].copy_(xp[i % n], non_blocking=True)
            SL.stack_forward(e["layers"], e["y"], e["tmp"])
            yp.copy_(e["y"], non_blocking=True)
            torch.cuda.synchronize()

        for i in range(3):
            one(i)
        barrier()
        t0 = time.perf_counter()
        for i in range(ke):
            one(i)
        dt = time.perf_counter() - t0
        h2d, d2h, note = int(xp[0].numel() * xp[0].element_size()), int(yp.numel() * yp.element_size()), "pinned x -> device, strix_moe_stack_forward, device -> pinned x"
    if dist is not None:
        t = torch.tensor([dt], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt = float(t.item())
    out["e2e"] = dict(value=cfg["M"] * ke * world / dt, unit="tokens/s", h2d_bytes_per_step=h2d, d2h_bytes_per_step=d2h, steps=ke,
                      note=note + ": host buffers in and out, copies and the sync inside the timed region (wall clock)")

    if rank == 0:
        # Roofline of the step: algorithmic bytes (decode) or flops (prefill) over the event-timed step.
        l0 = ring[0]["layers"][0]
        per_step_bytes, distinct = [], []
        for e in ring:
            step(e)
            tot = 0
            for l in e["layers"]:
                ids = l.probe("router_ids", cfg["M"]).cpu().numpy()
                b, nd = algorithmic_bytes(cfg, l, ids, getattr(l, "info", {}))
                tot += b
                distinct.append(nd)
            per_step_bytes.append(tot)
        step_s = ms * 1e-3 / steps
        tr = TRAFFIC.get(name, {})
        traffic = tr.get("bytes")
        traffic_note = None if traffic is None else dict(unit="bytes per launch (dram read + write)", kernel=tr["kernel"],
                                                          source=tr["source"] + " (ncu capture of a small ring of this workload; a constant, not measured in this run)")
        if cfg["M"] <= 64:
            ach = float(np.mean(per_step_bytes)) / step_s / 1e9
            out["roofline"] = dict(bound="hbm", achieved=ach, peak=P["hbm"], unit="GB/s", frac=ach / P["hbm"], traffic=traffic, traffic_note=traffic_note, peak_source=P["source"],
                                   frac_of_nominal_8TBs=ach / 8000.0, algorithmic_bytes_per_step=float(np.mean(per_step_bytes)),
                                   distinct_experts_per_layer=float(np.mean(distinct)), kernel="whole step (all launches of one pass over the layer(s))")
        else:
            fl = flops_of(cfg, l0.A)
            ach = fl / step_s / 1e12
            out["roofline"] = dict(bound="tensor", achieved=ach, peak=P["tensor"], unit="TFLOP/s", frac=ach / P["tensor"], traffic=traffic, traffic_note=traffic_note,
                                   peak_source=P["source"], algorithmic_flops_per_step=fl, kernel="whole step")
        per_ring = kernel_nodes(full)
        if per_ring is None:
            raise RuntimeError("could not count the kernel nodes of the captured steps")
        out["gpu_launches_per_step"] = per_ring / n
        out["gpu_launches"] = int(per_ring * (steps // n) + (kernel_nodes(rest) if rest is not None else 0))
        Ls = None
        if want_parity or want_cpu:
            Ls = [cpu_layer_from(l, cfg) for l in ring[0]["layers"]]
        if want_parity:
            e = ring[0]
            step(e)
            torch.cuda.synchronize()
            M = cfg["M"]
            last = e["layers"][-1]
            logits = last.probe("router_logits", M).cpu().numpy()
            ids = last.probe("router_ids", M).cpu().numpy()
            xh0, yh0 = host_act(e["x"]), host_act(e["y"])
            if M > 64:
                rows = np.sort(np.random.default_rng(5).choice(M, 64, replace=False))
                note = "64 of %d rows (seeded sample; tokens are independent)" % M
            else:
                rows, note = np.arange(M), "all %d" % M
            gated_stacked = cfg["shared"] == "stacked"
            out["parity"] = parity_of(np.ascontiguousarray(xh0[rows]), np.ascontiguousarray(yh0[rows]), Ls, logits, ids, gated_stacked, note)
            if cfg["layers"] > 1:
                out["parity"]["note"] = "the stack's final x after %d layers and residual adds; routing checked on the last layer" % cfg["layers"]
        if want_cpu:
            out["cpu_baseline"], _ = cpu_baseline(Ls, host_act(ring[0]["x"]), max_tokens=256 if cfg["M"] > 256 else None)
    del full, rest, ring
    torch.cuda.empty_cache()
    return out


def config_of(name, cfg, world, ring_note=None):
    return dict(workload=name, tokens_per_step=cfg["M"], hidden=cfg["d"], intermediate=cfg["I"], experts=cfg["E"], top_k=cfg["k"],
                shared_expert=cfg["shared"], shared_coef="sigmoid", expert_format="q4" if cfg["mix"] is None else "q4/q5/q6/q8 60/15/15/10",
                group_size=G_EXPERTS, router=cfg["router"], layers_per_step=cfg["layers"], parallelism="replicas x%d" % world,
                l2=ring_note or "ring of %d independent (weights, tokens) pairs cycled one per step; bytes between reuses >> 126 MB L2" % cfg["ring"])


# ---- the reference arm: the CPU path with weights built on the host, without the product library -------------------------

def cpu_build_layer(cfg, seed, xh):
    """A layer of cfg's shapes in the oracle's dict form, built on the host: N(0, 0.02) weights packed by the reference's
    own quantizer (oracle/_ref) when it was built, else by its restatement. Only the experts the tokens xh route to are
    generated (the others are never read); their weights are windows of one seeded N(0, 0.02) pool, since drawing 1.6 G
    fresh normals on the host would take longer than the measurement."""
    import oracle

    quant = oracle.ref_quantize if oracle.ref is not None else oracle.quantize
    d, I, E, k = cfg["d"], cfg["I"], cfg["E"], cfg["k"]
    rng = np.random.default_rng(seed)
    R = E + 1
    rw = (rng.standard_normal((R, d)) * 0.02).astype(np.float32)
    if cfg["router"] == "bf16":
        router = oracle.f32_to_bf16(rw)
    elif cfg["router"] == "q8":
        router = quant(8, rw, 64)
    else:
        router = rw
    L = dict(E=E, k=k, router=router, shared=cfg["shared"], shared_coef="sigmoid")
    if cfg["bias"] == "zipf":
        rank = rng.permutation(E) + 1
        p = rank.astype(np.float64) ** -1.1
        L["router_bias"] = np.log(p / p.sum()).astype(np.float32)
    elif cfg["bias"] is not None:
        L["router_bias"] = (rng.standard_normal(E) * cfg["bias"]).astype(np.float32)
    logits = oracle.linear_q(xh, router, oracle.F32) if isinstance(router, oracle.QWeight) else oracle.linear_w(xh, router, oracle.F32)
    if "router_bias" in L:
        logits[:, :E] += L["router_bias"][None, :]
    ids, _, _ = oracle.moe_router(np.ascontiguousarray(logits), E, k)
    Es = E + (1 if cfg["shared"] == "stacked" else 0)
    need = sorted(set(int(e) for e in np.unique(ids)) | ({E} if cfg["shared"] == "stacked" else set()))
    pool = (rng.standard_normal(8 << 20) * 0.02).astype(np.float32)
    fmts = rng.choice([4, 5, 6, 8], size=Es, p=cfg["mix"]) if cfg["mix"] is not None else np.full(Es, 4)

    def stack(N, Kd, salt):
        parts = {}
        for e in need:
            off = (e * 2654435761 + salt * 40503) % (pool.size - N * Kd)
            parts[e] = quant(int(fmts[e]), pool[off: off + N * Kd].reshape(N, Kd), G_EXPERTS)
        if cfg["mix"] is None:
            rb = oracle.row_bytes(4, Kd)
            q = np.zeros(Es * N * rb, np.uint8)
            s = np.zeros((Es * N, Kd // G_EXPERTS), np.uint16)
            m = np.zeros((Es * N, Kd // G_EXPERTS), np.uint16)
            for e, pw in parts.items():
                q[e * N * rb: (e + 1) * N * rb] = pw.q
                s[e * N: (e + 1) * N], m[e * N: (e + 1) * N] = pw.scale, pw.minv
            return oracle.ExpertStack(Es, N, Kd, G_EXPERTS, q, s, m, bits=4)
        zero = {b: None for b in (4, 5, 6, 8)}
        full = []
        for e in range(Es):
            if e in parts:
                full.append(parts[e])
            else:
                b = int(fmts[e])
                if zero[b] is None:
                    zero[b] = oracle.QWeight(b, N, Kd, G_EXPERTS, np.zeros(N * oracle.row_bytes(b, Kd), np.uint8), np.zeros((N, Kd // G_EXPERTS), np.uint16),
                                             np.zeros((N, Kd // G_EXPERTS), np.uint16))
                full.append(zero[b])
        return oracle.ExpertStack.from_mixed(full)

    L["gate_up"], L["down"] = stack(2 * I, d, 1), stack(d, I, 2)
    if cfg["shared"] == "separate":
        L["sh_gate_up"] = quant(8, pool[: 2 * I * d].reshape(2 * I, d), 64)
        L["sh_down"] = quant(8, pool[2 * I * d: 2 * I * d + d * I].reshape(d, I), 64)
    return L, ("reference quantizer (oracle/_ref)" if oracle.ref is not None else "quantizer restatement (oracle/)")


def reference_arm(args, name, cfg, line, emit):
    """The reference arm: the CPU implementation of the layer on the host cores, a bounded sample of the batch per step. Never
    touches the product library or a GPU."""
    import oracle

    sample = min(cfg["M"], 256)
    rng = np.random.default_rng(4242)
    x = rng.standard_normal((sample, cfg["d"])).astype(np.float32)
    xh = x if cfg["act"] == "f32" else oracle.f32_to_bf16(x)
    Ls, how = [], None
    for l in range(cfg["layers"]):
        L, how = cpu_build_layer(cfg, 100 + l, xh)
        Ls.append(L)
    base, one = cpu_baseline(Ls, xh, budget_s=3.0)
    for _ in range(max(0, min(args.warmup, 3) - 1)):
        one()
    k = max(1, min(args.steps, 20))
    t0 = time.perf_counter()
    for _ in range(k):
        one()
    dt = time.perf_counter() - t0
    v = sample * k / dt
    line["config"] = config_of(name, cfg, 1, "n/a (host caches)")
    line["config"]["parallelism"] = "host cores (%d threads)" % base["cores"]
    if cfg.get("ep"):  # the same declaration as the GPU arm's line for this workload
        line["scaling"] = "strong"
        line["config"]["router_bias"] = "Zipf(1.1)"
    line.update(impl="reference", value=v, steps=k, ms_per_step=1e3 * dt / k, n_gpus=args.gpus, gpu_launches=0,
                dtype="f32" if cfg["act"] == "f32" else "bf16",
                cpu_baseline=dict(value=v, unit="tokens/s", cores=base["cores"], kind="port",
                                  sample="%d timed passes of %d token(s) of the batch through %d layer(s); weights packed on the host by the %s" % (k, sample, len(Ls), how)),
                e2e=dict(value=v, unit="tokens/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    emit(line)


# ---- config 5: expert parallel ---------------------------------------------------------------------------------------------

def run_ep(args, cfg, steps, warmup, rank, world, local, device, P, line, want_parity):
    """One layer, its routed experts sharded over the ranks, the token batch split evenly (strong scaling). One rank runs the
    same code over a one-rank group. Returns the measured fields on every rank (parity, clocks on rank 0)."""
    import torch
    import torch.distributed as dist

    from strixite_b200 import ep as EP
    from strixite_b200 import kernels as K
    from strixite_b200 import synth

    if world > 1 and not dist.is_initialized():
        # a short timeout: a rank that leaves a collective alone ends the run with an error in minutes, not a silent wait
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(device), timeout=datetime.timedelta(seconds=240))
    barrier = dist.barrier if world > 1 else (lambda: None)  # one rank: the same code, its exchanges are the identity
    d, I, E, k, T = cfg["d"], cfg["I"], cfg["E"], cfg["k"], cfg["M"]
    Tl = T // world
    g = torch.Generator(device=device)
    g.manual_seed(4242)
    rw = (torch.randn((E + 1, d), generator=g, device=device, dtype=torch.float32) * 0.02).to(torch.bfloat16)  # replicated: same seed everywhere
    bias_h = synth.zipf_bias(99, E)
    bias = torch.from_numpy(bias_h).to(device)
    gu = synth.quantized_normal(501, 4, (E + 1) * 2 * I, d, G_EXPERTS, device=device)
    dn = synth.quantized_normal(502, 4, (E + 1) * d, I, G_EXPERTS, device=device)
    host_L = None
    if rank == 0 and want_parity:
        import oracle

        def hq(qw):
            q, s, m = qw.to_host()
            return oracle.QWeight(qw.bits, qw.N, qw.K, qw.G, q, s, m)

        host_L = dict(E=E, k=k, router=rw.view(torch.int16).cpu().numpy().view(np.uint16), shared="stacked", shared_coef="sigmoid",
                      gate_up=oracle.ExpertStack.from_weight(hq(gu), E + 1), down=oracle.ExpertStack.from_weight(hq(dn), E + 1), router_bias=bias_h)
    place = EP.placement(E, world, bias_h, k, balanced=not args.ep_contiguous)
    gu_l, dn_l = EP.shard_stack(gu, E, world, rank, place), EP.shard_stack(dn, E, world, rank, place)
    del gu, dn
    torch.cuda.empty_cache()
    layer = EP.cuda_layer(d, I, E, k, K.Act.BF16, rw, bias, gu_l, dn_l, world, rank, max_local_tokens=Tl, placement=place,
                          chunks=args.ep_chunks, peer_stores=not args.ep_all_to_all)
    xs = []
    for r in range(cfg["ring"]):
        g.manual_seed(9000 + 17 * r)
        xs.append(torch.randn((T, d), generator=g, device=device, dtype=torch.float32)[rank * Tl:(rank + 1) * Tl].to(torch.bfloat16).contiguous())
    for i in range(max(3, warmup)):
        y = layer.forward(xs[i % len(xs)])
    torch.cuda.synchronize()
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    torch.cuda.cudart().cudaProfilerStart()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        y = layer.forward(xs[i % len(xs)])
    e1.record()
    torch.cuda.synchronize()
    torch.cuda.cudart().cudaProfilerStop()
    barrier()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1)
    layer.check()  # the error words and the overflow flags of the timed steps
    recv = float(layer.received_slots())
    stats = torch.tensor([ms, recv], device=device)
    mx, sm = stats.clone(), stats.clone()
    if world > 1:
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
    ms = float(mx[0].item())
    # End to end: every step's tokens come from pinned host memory and its outputs go back to pinned host memory. The copies run on
    # their own streams, two steps' buffers deep, so step i's layer overlaps step i + 1's upload and step i - 1's download (a
    # serving loop's pipeline); the timed region ends when the last output has landed on the host.
    xh = [x.cpu().pin_memory() for x in xs]
    yh = [torch.empty_like(xh[0]).pin_memory() for _ in range(2)]
    xd = [torch.empty_like(xs[0]) for _ in range(2)]
    yd = [torch.empty_like(xs[0]) for _ in range(2)]
    s_in, s_out, cur = torch.cuda.Stream(device=device), torch.cuda.Stream(device=device), torch.cuda.current_stream(device)
    x_free = [torch.cuda.Event() for _ in range(2)]   # the layer has consumed xd[b]
    y_free = [torch.cuda.Event() for _ in range(2)]   # yd[b] has been downloaded
    ke = max(4, steps // 2)

    def e2e_steps(n_steps):
        for b in range(2):
            x_free[b].record(cur), y_free[b].record(cur)
        for i in range(n_steps):
            b = i % 2
            with torch.cuda.stream(s_in):
                s_in.wait_event(x_free[b])
                xd[b].copy_(xh[i % len(xh)], non_blocking=True)
                up = torch.cuda.Event()
                up.record(s_in)
            cur.wait_event(up)
            y = layer.forward(xd[b])
            x_free[b].record(cur)
            cur.wait_event(y_free[b])
            yd[b].copy_(y)  # the layer reuses its output buffer next step
            done = torch.cuda.Event()
            done.record(cur)
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                yh[b].copy_(yd[b], non_blocking=True)
                y_free[b].record(s_out)
        torch.cuda.synchronize()

    e2e_steps(2)
    barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    e2e_steps(ke)
    dt = torch.tensor([time.perf_counter() - t0], device=device)
    if world > 1:
        dist.all_reduce(dt, op=dist.ReduceOp.MAX)
    fl = 2.0 * T * (k + 1) * 3 * I * d + 2.0 * T * (E + 1) * d
    step_s = ms * 1e-3 / steps
    out = dict(value=T / step_s, unit="tokens/s", steps=steps, warmup=warmup, ms_per_step=ms / steps, clocks=clocks, dtype="bf16", scaling="strong")
    out["config"] = config_of("ep_prefill16384", cfg, world, "two token sets alternate; every step streams far more than the 126 MB L2")
    out["config"].update(parallelism="expert parallel x%d (%s placement of the experts over the ranks, tokens split evenly, shared expert replicated; %s; %d chunk(s) per step)"
                         % (world, "contiguous" if args.ep_contiguous else "load-balanced", "one row per (token, rank), summed on the expert rank; " + ("exchange = peer stores of the gather and row-sum kernels over NVLink, F16 sums back, two barriers" if layer.backend.pushes else "exchange = all-to-alls, FP32 sums back" if world > 1 else "no exchange"), layer.chunks),
                         router_bias="Zipf(1.1)")
    out["e2e"] = dict(value=T * ke / float(dt.item()), unit="tokens/s", h2d_bytes_per_step=int(xh[0].numel() * 2 * world), d2h_bytes_per_step=int(yh[0].numel() * 2 * world),
                      steps=ke, note="pinned host tokens -> device -> expert-parallel layer -> pinned host outputs, every step, per rank; uploads and downloads on "
                                     "their own streams two buffers deep (overlapping the neighbouring steps' layers); wall clock from the first upload to the last "
                                     "download landed, max over ranks")
    ach = fl / step_s / 1e12
    tr = TRAFFIC["ep_prefill16384"]
    out["roofline"] = dict(bound="tensor", achieved=ach, peak=P["tensor"] * world, unit="TFLOP/s", frac=ach / (P["tensor"] * world),
                           traffic=None if tr["bytes"] is None else tr["bytes"] / world,
                           traffic_note=dict(unit="bytes per launch and rank (dram read + write)", kernel=tr["kernel"],
                                             source=tr["source"] + (" (ncu capture on one GPU; a constant, not measured in this run" +
                                                                    ("; scaled by 1 / ranks: a rank streams its share of the experts and of the slots)" if world > 1 else ")"))),
                           peak_source=P["source"], algorithmic_flops_per_step=fl, kernel="whole step, all ranks",
                           load_imbalance_max_over_mean_slots=float(mx[1].item() / max(sm[1].item() / world, 1.0)))
    out["load_imbalance"] = out["roofline"]["load_imbalance_max_over_mean_slots"]
    out["gpu_launches_per_step"] = layer.launches_per_step()
    out["gpu_launches"] = int(layer.launches_per_step() * steps)
    out["gpu_launches_note"] = "this library's kernels per step and rank (router, plan, grouping, tiles, gather, FFN, reduce), counted where they are enqueued; NCCL collectives come on top"
    if want_parity:
        y = layer.forward(xs[0])  # every rank: the forward exchanges tokens; only rank 0 then runs the oracle on its rows
        torch.cuda.synchronize()
    if rank == 0 and want_parity:
        rows = np.sort(np.random.default_rng(5).choice(Tl, 64, replace=False))
        out["parity"] = parity_of(np.ascontiguousarray(host_act(xs[0])[rows]), np.ascontiguousarray(host_act(y)[rows]), [host_L], layer.last_logits().cpu().numpy(),
                                  layer.last_ids().cpu().numpy(), True, "64 of rank 0's %d rows (seeded sample; tokens are independent)" % Tl)
    return out, (dist if world > 1 else None)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=0, help="timed steps of the line's workload (0 = the workload's default)")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS), help="default: ep_prefill16384, with the other four attached on one GPU")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity", action="store_true")
    ap.add_argument("--no-workloads", action="store_true", help="default run: do not measure the four other workloads")
    ap.add_argument("--ring", type=int, default=0, help="override the number of independent (weights, tokens) pairs cycled (a small ring keeps a profiler capture small)")
    ap.add_argument("--tensor-min-tokens", type=int, default=0, help="with --math 2: run forwards of at least this many tokens on the tensor-core path")
    ap.add_argument("--math", type=int, default=-1, choices=[-1, 0, 1, 2], help="override the workload's MoeMath (0 = FP32 kernels, 1/2 = tensor cores)")
    ap.add_argument("--ep-contiguous", action="store_true", help="expert parallel: experts e -> rank e / (E / N) instead of the load-balanced placement")
    ap.add_argument("--ep-all-to-all", action="store_true", help="expert parallel: exchange through NCCL all-to-alls instead of the kernels' own peer stores")
    ap.add_argument("--ep-chunks", type=int, default=0, help="expert parallel: token chunks per step whose exchanges overlap the other chunk's kernels (0 = the default)")
    ap.add_argument("--grouped-min", type=int, default=0, help="override the token count from which the grouped expert path runs (reference: 6)")
    ap.add_argument("--decode-impl", type=int, default=0, choices=[0, 1], help="forwards of <= 8 tokens: 0 = the single streaming kernel, 1 = the per-function kernels")
    args = ap.parse_args()
    name = args.workload or "ep_prefill16384"
    cfg = dict(WORKLOADS[name])
    cfg["decode_impl"] = args.decode_impl
    if args.grouped_min > 0:
        cfg["grouped_min"] = args.grouped_min
    cfg["tensor_min_tokens"] = args.tensor_min_tokens
    if args.math >= 0:
        cfg["math"] = args.math
    if args.ring > 0:
        cfg["ring"] = args.ring
    steps = args.steps if args.steps > 0 else cfg["steps"]
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if args.warmup < 3:
        args.warmup = 3

    # torchrun sets OMP_NUM_THREADS=1 for its workers; the CPU legs (rank 0 only) are meant to use every host core
    os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)

    # Libraries (NCCL's version banner, for one) write to stdout; the line is the only thing that may: everything else goes to stderr
    real_stdout = os.dup(1)
    os.dup2(2, 1)

    def emit(obj):
        sys.stdout.flush()
        os.dup2(real_stdout, 1)
        print(json.dumps(obj), flush=True)
        os.dup2(2, 1)

    line = dict(metric="MoE-layer tokens/s", unit="tokens/s", n_gpus=args.gpus, steps=steps, warmup=args.warmup, higher_is_better=True,
                scaling="weak", vs_baseline=None, dtype="f32" if cfg["act"] == "f32" else "bf16", data="synthetic")
    if args.impl == "reference":
        if rank == 0:
            reference_arm(args, name, cfg, line, emit)
        return

    import torch

    import oracle  # noqa: F401  (the CPU legs and the parity check only)

    torch.cuda.set_device(local)
    device = "cuda:%d" % local
    P = peaks()
    want_cpu = not args.no_cpu_baseline and rank == 0 and world == 1
    want_parity = not args.no_parity

    if cfg.get("ep"):
        # The CPU baseline first: before any process group exists (idle ranks spinning in a barrier would take the cores).
        cpu = None
        if want_cpu:
            x = np.random.default_rng(4242).standard_normal((256, cfg["d"])).astype(np.float32)
            xh = oracle.f32_to_bf16(x)
            L, how = cpu_build_layer(cfg, 100, xh)
            cpu, _ = cpu_baseline([L], xh, budget_s=10.0)
            cpu["sample"] += "; weights packed on the host by the " + how
        out, dist = run_ep(args, cfg, steps, args.warmup, rank, world, local, device, P, line, want_parity)
        line.update(out)
        if cpu is not None:
            line["cpu_baseline"] = cpu
        if rank == 0 and args.workload is None and world == 1 and not args.no_workloads:
            line["workloads"] = {}
            for wn in ("decode1", "verify6", "prefill4096", "stack4"):
                wc = dict(WORKLOADS[wn], decode_impl=0, tensor_min_tokens=0)
                w = measure_single(wn, wc, wc["steps"], max(args.warmup, 3), 0, 1, local, device, P, None, lambda: None, not args.no_cpu_baseline, want_parity)
                w["config"] = config_of(wn, wc, 1)
                line["workloads"][wn] = w
        if rank == 0:
            emit(line)
        if dist is not None:
            dist.barrier()
            dist.destroy_process_group()
        return

    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device(device), timeout=datetime.timedelta(seconds=240))
        barrier = lambda: dist.barrier()  # noqa: E731
    else:
        dist, barrier = None, (lambda: None)
    out = measure_single(name, cfg, steps, args.warmup, rank, world, local, device, P, dist, barrier, want_cpu, want_parity and rank == 0)
    line.update(out)
    line["config"] = config_of(name, cfg, world)
    if rank == 0:
        emit(line)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
