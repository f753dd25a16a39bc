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

That is the exact mode (dedup=False). The default mode (dedup=True) moves less: a token's row goes ONCE to every rank that
owns one of its experts (with its slots' expert ids and coefficients), the expert rank sums coef * partial over the
token's slots it served (ascending slot order) and returns ONE FP32 row per (token, rank), and the home rank adds those
in ascending rank order. Same arithmetic, another association: results are reproducible for a given number of ranks and
agree with the single-device layer to FP32 rounding, not bit for bit.

The exchange plumbing is torch (index_select / argsort / all_to_all_single on whatever device the tensors live on);
the three compute steps are callables, by default the CUDA library's. Tests drive the same plumbing over gloo on CPU
tensors with the oracle's functions plugged in.
"""
import torch
import torch.distributed as dist


class ExpertParallelMoe:
    def __init__(self, E, k, world, rank, route_fn, experts_fn, reduce_fn, group=None, shared=True, dedup=True):
        """E routed experts (E % world == 0), top-k; `shared`: a stacked shared expert with id E rides slot k.
        route_fn(x) -> (ids int32 [T, A], coef float32 [T, A]);  experts_fn(rows [n, d], local_ids int32 [n]) -> float32 [n, d];
        reduce_fn(partial float32 [R, d], pos int64 [T, W], ids int32 [T, W], coef float32 [T, W], out_dtype) -> [T, d]:
        y[t] = sum over w ascending of coef[t, w] * partial[pos[t, w]] (ids only say valid / invalid), rounded once to
        out_dtype (None = the activation dtype). With dedup, experts_fn(rows, local_ids, row_index int32 [n]) reads slot
        i's activation from rows[row_index[i]]."""
        if E % world != 0:
            raise ValueError("ExpertParallelMoe: %d experts do not divide over %d ranks" % (E, world))
        self.E, self.k, self.world, self.rank, self.group = E, k, world, rank, group
        self.El = E // world
        self.A = k + (1 if shared else 0)
        self.route_fn, self.experts_fn, self.reduce_fn = route_fn, experts_fn, reduce_fn
        self.dedup = dedup
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
        marks = []

        def mark(name):
            if timings is not None and x.is_cuda:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                marks.append((name, ev))

        mark("start")
        y = self._forward_dedup(x, mark) if self.dedup else self._forward_exact(x, mark)
        if marks:
            torch.cuda.synchronize()
            for (_, a), (name, b) in zip(marks[:-1], marks[1:]):
                timings[name] = timings.get(name, 0.0) + a.elapsed_time(b)
        return y

    def _exchange_counts(self, counts):
        """counts int64 [world, c] per destination -> what every source sends here, as host lists (split sizes are host ints)."""
        recv = torch.empty_like(counts)
        dist.all_to_all_single(recv, counts, group=self.group)
        return counts.tolist(), recv.tolist()

    def _forward_exact(self, x, mark):
        T, d = x.shape
        ids, coef = self.route_fn(x)
        mark("route")
        order, send_ids, counts = self.plan(ids)
        send_rows = x.index_select(0, torch.div(order, self.A, rounding_mode="floor"))
        mark("plan+gather")
        out_c, in_c = self._exchange_counts(counts.reshape(-1, 1))
        out_splits, in_splits = [c[0] for c in out_c], [c[0] for c in in_c]
        mark("counts")
        n_recv = int(sum(in_splits))
        recv_rows = x.new_empty((n_recv, d))
        recv_ids = send_ids.new_empty((n_recv,))
        dist.all_to_all_single(recv_rows, send_rows, in_splits, out_splits, group=self.group)
        dist.all_to_all_single(recv_ids, send_ids, in_splits, out_splits, group=self.group)
        mark("dispatch")
        partial = self.experts_fn(recv_rows, recv_ids, None) if n_recv else torch.empty((0, d), dtype=torch.float32, device=x.device)
        mark("experts")
        back = torch.empty((T * self.A, d), dtype=torch.float32, device=x.device)
        dist.all_to_all_single(back, partial, out_splits, in_splits, group=self.group)
        mark("combine all-to-all")
        pos = torch.empty_like(order)
        pos[order] = torch.arange(order.numel(), device=order.device)  # slot t * A + a came back as row pos[t * A + a]
        self.last = dict(ids=ids, coef=coef, sent=out_splits, received=in_splits)
        y = self.reduce_fn(back, pos.reshape(T, self.A), ids, coef, None)
        mark("reduce")
        return y

    def _forward_dedup(self, x, mark):
        T, d = x.shape
        dev = x.device
        W, A = self.world, self.A
        ids, coef = self.route_fn(x)
        mark("route")
        order, send_ids, slot_counts = self.plan(ids)  # slots by destination, (token, slot) order inside a destination
        S = order.numel()
        tok = torch.div(order, A, rounding_mode="floor")
        dest = torch.repeat_interleave(torch.arange(W, device=dev), slot_counts, output_size=S)
        # pairs (destination, token): a new pair starts where either changes along the sorted slots
        new_pair = torch.ones(S, dtype=torch.bool, device=dev)
        new_pair[1:] = (tok[1:] != tok[:-1]) | (dest[1:] != dest[:-1])
        pair_of_slot = torch.cumsum(new_pair.to(torch.int64), 0) - 1          # global pair index of every sorted slot
        first = torch.nonzero(new_pair).reshape(-1)                           # first sorted slot of every pair
        pair_tok, pair_dest = tok[first], dest[first]
        pair_counts = torch.bincount(pair_dest, minlength=W)
        pair_start = torch.cumsum(pair_counts, 0) - pair_counts               # first pair of every destination
        send_rows = x.index_select(0, pair_tok)
        send_rel = (pair_of_slot - pair_start[dest]).to(torch.int32)           # the slot's row inside its destination's block
        send_coef = coef.reshape(-1)[order]
        mark("plan+gather")
        out_c, in_c = self._exchange_counts(torch.stack([slot_counts, pair_counts], 1))
        out_slots, out_pairs = [c[0] for c in out_c], [c[1] for c in out_c]
        in_slots, in_pairs = [c[0] for c in in_c], [c[1] for c in in_c]
        mark("counts")
        n_slots, n_pairs = int(sum(in_slots)), int(sum(in_pairs))
        recv_rows = x.new_empty((n_pairs, d))
        # one message per slot: local expert id, row inside the destination's block, coefficient (bits)
        send_meta = torch.stack([send_ids, send_rel, send_coef.view(torch.int32)], 1).contiguous()
        recv_meta = send_meta.new_empty((n_slots, 3))
        dist.all_to_all_single(recv_rows, send_rows, in_pairs, out_pairs, group=self.group)
        dist.all_to_all_single(recv_meta, send_meta, in_slots, out_slots, group=self.group)
        recv_ids, recv_rel, recv_coef = recv_meta[:, 0].contiguous(), recv_meta[:, 1], recv_meta[:, 2].contiguous().view(torch.float32)
        mark("dispatch")
        # the slot's row among everything received: its source's first row + its row inside the source's block
        in_slots_t, in_pairs_t = torch.tensor(in_slots, device=dev), torch.tensor(in_pairs, device=dev)
        src = torch.repeat_interleave(torch.arange(W, device=dev), in_slots_t, output_size=n_slots)
        row_index = (recv_rel.to(torch.int64) + (torch.cumsum(in_pairs_t, 0) - in_pairs_t)[src])
        if n_slots:
            partial = self.experts_fn(recv_rows, recv_ids, row_index.to(torch.int32))
        else:
            partial = torch.empty((0, d), dtype=torch.float32, device=dev)
        mark("experts")
        # expert-side sum per received row: its slots are consecutive (the source sorted them); a table [rows, k + 1] of slot
        # positions, padded with coefficient 0 on a valid row, feeds the ordered weighted sum
        if n_pairs:
            start = torch.ones(n_slots, dtype=torch.bool, device=dev)
            start[1:] = row_index[1:] != row_index[:-1]
            first_slot = torch.nonzero(start).reshape(-1)                       # one per received row, in row order
            rank_in_row = torch.arange(n_slots, device=dev) - first_slot[row_index]
            pos_t = torch.zeros((n_pairs, A), dtype=torch.int64, device=dev)
            coef_t = torch.zeros((n_pairs, A), dtype=torch.float32, device=dev)
            ids_t = torch.zeros((n_pairs, A), dtype=torch.int32, device=dev)
            pos_t[row_index, rank_in_row] = torch.arange(n_slots, device=dev)
            coef_t[row_index, rank_in_row] = recv_coef
            ids_t[row_index, rank_in_row] = torch.where(recv_ids < 0, recv_ids, torch.zeros_like(recv_ids))  # invalid ids poison the row
            summed = self.reduce_fn(partial, pos_t, ids_t, coef_t, torch.float32)
        else:
            summed = torch.empty((0, d), dtype=torch.float32, device=dev)
        mark("expert-side sum")
        back = torch.empty((int(sum(out_pairs)), d), dtype=torch.float32, device=dev)
        dist.all_to_all_single(back, summed, out_pairs, in_pairs, group=self.group)
        mark("combine all-to-all")
        # home: token t's rows, one per rank that served it, added in ascending rank order
        pos_h = torch.zeros((T, W), dtype=torch.int64, device=dev)
        coef_h = torch.zeros((T, W), dtype=torch.float32, device=dev)
        pos_h[pair_tok, pair_dest] = torch.arange(pair_tok.numel(), device=dev)
        coef_h[pair_tok, pair_dest] = 1.0
        ids_h = torch.zeros((T, W), dtype=torch.int32, device=dev)
        self.last = dict(ids=ids, coef=coef, sent=out_slots, received=in_slots, rows_sent=out_pairs, rows_received=in_pairs)
        y = self.reduce_fn(back, pos_h, ids_h, coef_h, None)
        mark("reduce")
        return y


def cuda_layer(d, I, E, k, act, router_w, router_bias, gate_up_local, down_local, world, rank, max_local_tokens, capacity=None, group=None,
               math=2, dedup=True):
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

    def experts(rows, local_ids, row_index):
        return shard.experts_partial(rows, local_ids, row_index=row_index)

    def reduce(partial, pos, ids, coef, out_dtype):
        T, Wd = ids.shape
        out_act = K.Act.F32 if out_dtype == torch.float32 else act
        y = torch.empty((T, d), dtype=K._dtype(out_act), device=partial.device)
        K.moe_combine_reduce(partial, ids.contiguous(), coef.contiguous(), T, Wd, E + 1, d, y, out_act, pos=pos.contiguous())
        return y

    ep = ExpertParallelMoe(E, k, world, rank, route, experts, reduce, group=group, dedup=dedup)
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
