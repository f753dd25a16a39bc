"""Expert-parallel MoE sublayer: the routed experts sharded over the ranks of a torch.distributed group, tokens
data-parallel, one all-to-all each way.

strixite itself runs one device (its expert stacks are whole, runtime/qwen4exp.cpp:1126-1186), so this has no
counterpart there; its contract is "the same output as the single-device layer":

  home rank   router projection + moe_router on its own tokens (router weights replicated)       -> ids, coef [T, A]
              every slot (token, a) goes to the rank that owns its expert; the stacked shared expert (id E) is
              replicated and stays home (it is local expert E / P of every rank's stacks)
  exchange    counts, then one activation row + one local expert id per slot (all_to_all_single, uneven splits)
  expert rank partial[i, :] = W_down[e_i] * SwiGLU(W_gate_up[e_i] * row_i), FP32, no coefficient
  exchange    the FP32 rows back, in the order they were sent
  home rank   y[t, :] = sum_a coef[t, a] * partial[t * A + a, :] in ascending a: the reference's ordered combine

A slot's partial row depends on nothing but its own row and expert, and the final sum runs in slot order on the home
rank, so the result does not depend on the number of ranks.

The exchange plumbing is torch (index_select / argsort / all_to_all_single on whatever device the tensors live on);
the three compute steps are callables, by default the CUDA library's. Tests drive the same plumbing over gloo on CPU
tensors with the oracle's functions plugged in.
"""
import torch
import torch.distributed as dist


class ExpertParallelMoe:
    def __init__(self, E, k, world, rank, route_fn, experts_fn, reduce_fn, group=None, shared=True):
        """E routed experts (E % world == 0), top-k; `shared`: a stacked shared expert with id E rides slot k.
        route_fn(x) -> (ids int32 [T, A], coef float32 [T, A]);  experts_fn(rows [n, d], local_ids int32 [n]) -> float32 [n, d];
        reduce_fn(partial float32 [T * A, d], pos int64 [T * A], ids, coef) -> y [T, d], slot (t, a) being row pos[t * A + a]."""
        if E % world != 0:
            raise ValueError("ExpertParallelMoe: %d experts do not divide over %d ranks" % (E, world))
        self.E, self.k, self.world, self.rank, self.group = E, k, world, rank, group
        self.El = E // world
        self.A = k + (1 if shared else 0)
        self.route_fn, self.experts_fn, self.reduce_fn = route_fn, experts_fn, reduce_fn
        self.last = {}

    def plan(self, ids):
        """Slots sorted by destination rank (stable, so a destination sees a home rank's slots in slot order).
        Returns (order int64 [S], local expert ids int32 [S] in that order, counts int64 [world])."""
        flat = ids.reshape(-1).to(torch.int64)
        shared = flat == self.E
        bad = (flat < 0) | (flat > self.E)
        dest = torch.where(shared | bad, torch.full_like(flat, self.rank), torch.div(flat, self.El, rounding_mode="floor"))
        local = torch.where(shared, torch.full_like(flat, self.El), flat - dest * self.El)
        local = torch.where(bad, torch.full_like(flat, -1), local)  # invalid ids stay invalid: the kernels poison those tokens
        order = torch.argsort(dest, stable=True)
        counts = torch.bincount(dest, minlength=self.world)
        return order, local[order].to(torch.int32), counts

    def forward(self, x, timings=None):
        """y [T, d] for this rank's tokens x [T, d]. timings: an optional dict that receives the milliseconds of each phase
        (CUDA events; adds a synchronization at the end)."""
        T, d = x.shape
        marks = []

        def mark(name):
            if timings is not None and x.is_cuda:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                marks.append((name, ev))

        mark("start")
        ids, coef = self.route_fn(x)
        mark("route")
        order, send_ids, counts = self.plan(ids)
        send_rows = x.index_select(0, torch.div(order, self.A, rounding_mode="floor"))
        mark("plan+gather")
        # counts both ways (host integers: all_to_all_single wants split sizes)
        recv_counts = torch.empty_like(counts)
        dist.all_to_all_single(recv_counts, counts, group=self.group)
        out_splits, in_splits = counts.tolist(), recv_counts.tolist()
        mark("counts")
        n_recv = int(sum(in_splits))
        recv_rows = x.new_empty((n_recv, d))
        recv_ids = send_ids.new_empty((n_recv,))
        dist.all_to_all_single(recv_rows, send_rows, in_splits, out_splits, group=self.group)
        dist.all_to_all_single(recv_ids, send_ids, in_splits, out_splits, group=self.group)
        mark("dispatch")
        partial = self.experts_fn(recv_rows, recv_ids) if n_recv else torch.empty((0, d), dtype=torch.float32, device=x.device)
        mark("experts")
        back = torch.empty((T * self.A, d), dtype=torch.float32, device=x.device)
        dist.all_to_all_single(back, partial, out_splits, in_splits, group=self.group)
        mark("combine all-to-all")
        pos = torch.empty_like(order)
        pos[order] = torch.arange(order.numel(), device=order.device)  # slot t * A + a came back as row pos[t * A + a]
        self.last = dict(ids=ids, coef=coef, sent=out_splits, received=in_splits)
        y = self.reduce_fn(back, pos, ids, coef)
        mark("reduce")
        if marks:
            torch.cuda.synchronize()
            for (_, a), (name, b) in zip(marks[:-1], marks[1:]):
                timings[name] = timings.get(name, 0.0) + a.elapsed_time(b)
        return y


def cuda_layer(d, I, E, k, act, router_w, router_bias, gate_up_local, down_local, world, rank, max_local_tokens, capacity=None, group=None,
               math=2):
    """The expert-parallel layer on this rank's GPU. router_w: BF16 or FP32 [E + 1, d] (row E gates the shared expert),
    replicated. gate_up_local / down_local: this rank's E / world routed experts followed by the shared expert
    ([(E / world + 1) * 2I, d] and [(E / world + 1) * d, I], uniform 4-bit). capacity: the most slots this rank accepts in
    one forward (default: every slot of every rank, the worst case)."""
    from . import kernels as K
    from .layer import MoeLayer

    El, A = E // world, k + 1
    cap = capacity if capacity is not None else world * max_local_tokens * A
    dummy_router = torch.zeros((El, d), dtype=torch.float32, device=router_w.device)
    shard = MoeLayer(d, I, El, 1, act, dummy_router, gate_up_local, down_local, shared="stacked", shared_coef="one", max_tokens=(cap + 1) // 2,
                     grouped_min_tokens=1, math=math)
    R = E + 1

    def route(x):
        T = x.shape[0]
        logits = torch.empty((T, R), dtype=torch.float32, device=x.device)
        if router_w.dtype == torch.bfloat16:
            K.linear_bf16w(x, router_w, logits, T, R, d, act, K.Act.F32)
        else:
            K.linear_f32w(x, router_w, logits, T, R, d, act, K.Act.F32)
        if router_bias is not None:
            logits[:, :E] += router_bias
        ids = torch.empty((T, A), dtype=torch.int32, device=x.device)
        coef = torch.empty((T, A), dtype=torch.float32, device=x.device)
        err = K.new_err(x.device)
        K.moe_router(logits, R, T, E, k, logits[:, E:], R, E, ids, coef, K.Act.F32, err)
        return ids, coef

    def experts(rows, local_ids):
        return shard.experts_partial(rows, local_ids)

    def reduce(partial, pos, ids, coef):
        T = ids.shape[0]
        y = torch.empty((T, d), dtype=K._dtype(act), device=partial.device)
        K.moe_combine_reduce(partial, ids, coef, T, A, E + 1, d, y, act, pos=pos)
        return y

    ep = ExpertParallelMoe(E, k, world, rank, route, experts, reduce, group=group)
    ep.shard = shard
    return ep


def shard_stack(full, E, world, rank):
    """This rank's slice of a full stacked weight [(E + 1) * N, K] (kernels.QWeight): its E / world routed experts followed
    by the shared expert (expert E), as a new QWeight."""
    from . import kernels as K

    N = full.N // (E + 1)
    El = E // world
    rb = K.row_bytes(full.bits, full.K)
    rows = torch.cat([torch.arange(rank * El * N, (rank + 1) * El * N, device=full.q.device), torch.arange(E * N, (E + 1) * N, device=full.q.device)])
    q = full.q.view(-1, rb).index_select(0, rows).reshape(-1)
    return K.QWeight(full.bits, rows.numel(), full.K, full.G, q, full.scale.index_select(0, rows), full.minv.index_select(0, rows))
