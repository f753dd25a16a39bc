"""Expert-parallel MoE sublayer: the routed experts spread over the ranks of a torch.distributed group, tokens
data-parallel, one all-to-all each way, no size ever passing through the host.

strixite itself runs one device (its expert stacks are whole, runtime/qwen4exp.cpp:1126-1186), so this has no counterpart
there; its contract is "the same output as the single-device layer" to FP32 rounding (bit for bit on one rank).

  home rank    router projection + moe_router on its own tokens (router weights replicated)          -> ids, coef [T, A]
               plan: a token goes ONCE to every rank that owns one of its experts, with its slots' local expert ids and
               coefficients; the stacked shared expert (id E) is replicated and stays home
  exchange     fixed-capacity blocks per (source, destination): C rows [C, d] and MW int32 of metadata (layout: csrc/ep.cu);
               torch.distributed all_to_all_single with equal splits (NCCL on GPUs) - nothing is sized on the host
  expert rank  partial[slot, :] = W_down[e] * SwiGLU(W_gate_up[e] * row) in FP32 over the received slots (absent slots of a
               pair's capacity are skipped), then one FP32 row per received (token, rank): sum of coef * partial in slot order
  exchange     those rows back
  home rank    y[t, :] = the rows that came back for token t, added in ascending rank order, rounded once

Placement: which rank owns which expert is a table (contiguous blocks, or balanced over a load estimate so that a skewed router
does not make one rank the straggler). A step may be cut into token chunks on separate streams so that one chunk's exchanges
overlap the other's kernels.

The compute steps come from a backend object: CudaBackend (this library's kernels) here; the tests drive the same exchange
logic over gloo with a host backend made of numpy and the oracle.
"""
import ctypes as C

import numpy as np
import torch
import torch.distributed as dist


def meta_ints(Cr, Cs):
    """int32 words of one (source, destination) metadata block for capacities of Cr rows and Cs slots."""
    return 4 + 2 * Cr + 3 * Cs


def placement(E, world, bias=None, k=10, balanced=True, seed=1234, sigma=0.82):
    """owner[e] and local_of[e] for the E routed experts (E % world == 0; every rank holds E / world of them) plus entry E for
    the stacked shared expert (local index E / world on every rank). balanced: experts are dealt in order of an estimated load
    - the share of top-k picks each gets from logits N(0, sigma) + bias, sampled with a fixed seed - always to the rank with
    the least load so far that still has room; else contiguous blocks e -> e // (E / world). Returns a dict of numpy arrays."""
    if E % world != 0:
        raise ValueError("placement: %d experts do not divide over %d ranks" % (E, world))
    El = E // world
    owner = np.zeros(E + 1, np.int32)
    local_of = np.zeros(E + 1, np.int32)
    if balanced and world > 1 and bias is not None:
        rng = np.random.default_rng(seed)
        logits = rng.standard_normal((4096, E)).astype(np.float32) * sigma + np.asarray(bias, np.float32)[None, :]
        picks = np.argpartition(-logits, k - 1, axis=1)[:, :k]
        load = np.bincount(picks.reshape(-1), minlength=E).astype(np.float64) + 1e-3
        order = np.lexsort((np.arange(E), -load))  # descending load, ties by index
        rank_load, room = np.zeros(world), np.full(world, El)
        for e in order:
            cand = [r for r in range(world) if room[r] > 0]
            r = min(cand, key=lambda q: (rank_load[q], q))
            owner[e] = r
            rank_load[r] += load[e]
            room[r] -= 1
    else:
        owner[:E] = np.arange(E) // El
    experts_of = [np.nonzero(owner[:E] == r)[0].astype(np.int64) for r in range(world)]
    for r in range(world):
        local_of[experts_of[r]] = np.arange(El, dtype=np.int32)
    owner[E], local_of[E] = -1, El  # the shared expert: every rank's own
    return dict(owner=owner, local_of=local_of, experts_of=experts_of, El=El)


def plan_reference(ids, coef, E, owner, local_of, P, rank, Cr, Cs):
    """The layout strix_ep_plan writes, restated in numpy (the definition the kernel is tested against):
    rowtok [P, Cr], meta [P, MW], pos [T, P], flags [2]."""
    T, A = ids.shape
    MW = meta_ints(Cr, Cs)
    rowtok = np.zeros((P, Cr), np.int32)
    meta = np.zeros((P, MW), np.int32)
    pos = np.full((T, P), -1, np.int32)
    n_rows, n_slots = np.zeros(P, np.int64), np.zeros(P, np.int64)
    cb = np.ascontiguousarray(coef, np.float32).view(np.int32)
    for t in range(T):
        row_of = {}
        for a in range(A):
            e = int(ids[t, a])
            if 0 <= e <= E:
                r = rank if e == E else int(owner[e])
                loc = int(local_of[e])
            else:
                r, loc = rank, -1
            if r not in row_of:
                row_of[r] = int(n_rows[r])
                n_rows[r] += 1
                if row_of[r] < Cr:
                    rowtok[r, row_of[r]] = t
                    meta[r, 4 + 2 * row_of[r]] = n_slots[r]
            j = int(n_slots[r])
            n_slots[r] += 1
            if j < Cs and row_of[r] < Cr:
                meta[r, 4 + 2 * Cr + 3 * j: 4 + 2 * Cr + 3 * j + 3] = (loc, row_of[r], cb[t, a])
                meta[r, 4 + 2 * row_of[r] + 1] += 1
        for r, i in row_of.items():
            pos[t, r] = i if i < Cr else -1
    flags = np.zeros(2, np.uint32)
    for r in range(P):
        meta[r, 0], meta[r, 1] = min(n_rows[r], Cr), min(n_slots[r], Cs)
        if n_rows[r] > Cr:
            flags[0] = max(flags[0], n_rows[r])
        if n_slots[r] > Cs:
            flags[1] = max(flags[1], n_slots[r])
    return rowtok, meta, pos, flags


class ExpertParallelMoe:
    """The exchange logic over a backend. backend methods, per chunk c (buffers are the backend's, reused every step):
      route(c, x) -> (ids [T, A], coef [T, A]);  plan(c) -> (rows_send [P, Cr, d], meta_send [P, MW]);
      experts(c, rows_recv, meta_recv) -> summed [P, Cr, d] float32;  home(c, back) -> y [T, d]
    and recv buffers rows_recv(c), meta_recv(c), back(c)."""

    def __init__(self, world, rank, backend, group=None, chunks=1, timeout_s=None):
        self.world, self.rank, self.backend, self.group, self.chunks = world, rank, backend, group, chunks
        self.timeout_s = timeout_s

    def _a2a(self, out, inp):
        if self.world == 1:
            return inp
        w = dist.all_to_all_single(out, inp, group=self.group, async_op=self.timeout_s is not None)
        if w is not None and not w.wait(timeout=__import__("datetime").timedelta(seconds=self.timeout_s)):
            raise RuntimeError("expert-parallel exchange: a peer did not join within %.1f s" % self.timeout_s)
        return out

    def forward(self, x):
        """y [T, d] for this rank's tokens x [T, d] (T a multiple of the chunk count)."""
        b, n = self.backend, self.chunks
        T = x.shape[0]
        if T % n != 0:
            raise ValueError("ExpertParallelMoe: %d tokens do not split into %d chunks" % (T, n))
        Tc = T // n
        b.begin(x)
        if getattr(b, "pushes", False):  # the backend's kernels write into the peers' buffers themselves
            for c in range(n):
                with b.stream(c):
                    b.route(c, x[c * Tc:(c + 1) * Tc])
                    b.plan_push(c)
            for c in range(n):
                with b.stream(c):
                    b.experts_push(c)
            ys = []
            for c in range(n):
                with b.stream(c):
                    ys.append(b.home(c, b.back(c)))
            return b.end(ys)
        recv = [None] * n
        for c in range(n):
            with b.stream(c):
                b.route(c, x[c * Tc:(c + 1) * Tc])
                rows_send, meta_send = b.plan(c)
                recv[c] = (self._a2a(b.rows_recv(c), rows_send), self._a2a(b.meta_recv(c), meta_send))
        back = [None] * n
        for c in range(n):
            with b.stream(c):
                summed = b.experts(c, *recv[c])
                back[c] = self._a2a(b.back(c), summed)
        ys = []
        for c in range(n):
            with b.stream(c):
                ys.append(b.home(c, back[c]))
        return b.end(ys)


class _NoStream:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


class CudaBackend:
    """The compute steps on this rank's GPU, over this library's kernels. router_w: BF16 or FP32 [E + 1, d] (row E gates the
    shared expert), replicated. gate_up_local / down_local: this rank's E / world routed experts in placement order followed by
    the shared expert (uniform 4-bit stacks)."""

    def __init__(self, d, I, E, k, act, router_w, router_bias, gate_up_local, down_local, world, rank, place, max_local_tokens, chunks=1, math=2,
                 slot_capacity=None, peer_group=None):
        from . import kernels as K
        from ._lib import lib
        from .layer import MoeLayer

        self.K, self.lib = K, lib
        self.d, self.I, self.E, self.k, self.A, self.act = d, I, E, k, k + 1, K.Act(act)
        self.P, self.rank, self.El = world, rank, E // world
        self.router_w, self.router_bias = router_w, router_bias
        dev = router_w.device
        self.dev = dev
        self.chunks = chunks
        if max_local_tokens % chunks != 0:
            raise ValueError("CudaBackend: %d tokens do not split into %d chunks" % (max_local_tokens, chunks))
        Tc = max_local_tokens // chunks
        self.Tc = Tc
        self.Cr = Tc  # a token sends at most one row to a rank
        if slot_capacity is None:  # 2.5 x the even share of a chunk's slots, or all of them on one or two ranks
            slot_capacity = Tc * self.A if world <= 2 else min(Tc * self.A, int(2.5 * Tc * self.A / world) + 1024)
        self.Cs = int(slot_capacity)
        self.MW = meta_ints(self.Cr, self.Cs)
        self.owner = torch.from_numpy(place["owner"].copy()).to(dev)
        self.local_of = torch.from_numpy(place["local_of"].copy()).to(dev)
        n_cap = world * self.Cs
        dummy_router = torch.zeros((self.El, d), dtype=torch.float32, device=dev)
        self.streams = [torch.cuda.Stream(device=dev) for _ in range(chunks)] if chunks > 1 else [None]
        adt = K._dtype(self.act)
        self.c = []
        self.y_full = torch.empty((Tc * chunks, d), dtype=adt, device=dev)  # the chunks' outputs are views of one buffer
        for ci in range(chunks):
            shard = MoeLayer(d, I, self.El, 1, act, dummy_router, gate_up_local, down_local, shared="stacked", shared_coef="one", max_tokens=(n_cap + 1) // 2,
                             grouped_min_tokens=1, math=math)
            z = lambda *s, dt=torch.int32: torch.zeros(s, dtype=dt, device=dev)  # noqa: E731
            self.c.append(dict(
                shard=shard, logits=z(Tc, E + 1, dt=torch.float32), ids=z(Tc, self.A), coef=z(Tc, self.A, dt=torch.float32), err=K.new_err(dev),
                rowtok=z(world, self.Cr), meta_send=z(world, self.MW), meta_recv=z(world, self.MW), pos=z(Tc, world), flags=z(2),
                plan_scratch=z(int(lib.strix_ep_plan_scratch_ints(Tc))),
                rows_send=z(world, self.Cr, d, dt=adt), rows_recv=z(world, self.Cr, d, dt=adt), slot_ids=z(n_cap), slot_row=z(n_cap),
                partial=torch.empty((n_cap, d), dtype=torch.float16, device=dev), summed=z(world, self.Cr, d, dt=torch.float32),
                back=z(world, self.Cr, d, dt=torch.float32), y=self.y_full[ci * Tc:(ci + 1) * Tc]))
        self.launches = 0
        # peer_group (a process group over the ranks, one GPU each): the receive buffers live in memory every peer has mapped,
        # and the kernels write their blocks straight into the destination's buffers (push_rows / experts_push) - the exchange
        # is part of the gather and of the row sum, the ranks only meet at a barrier. Without it: library all-to-alls.
        self.pushes = False
        if peer_group is not None and world > 1:
            try:
                self._map_peer_buffers(peer_group, adt)
            except Exception as e:  # noqa: BLE001 - no peer mapping on this system: the all-to-all path serves
                import sys

                print("strixite_b200.ep: peer-mapped buffers unavailable (%s: %s); using all-to-alls" % (type(e).__name__, e), file=sys.stderr)
                self.pushes = False

    def _map_peer_buffers(self, group, adt):
        import os

        import torch.distributed._symmetric_memory as symm

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")  # plain peer mappings: the kernels use ordinary stores
        dev, P = self.dev, self.P
        self.peer_group = group
        self.back_dtype = torch.float16  # the sums that travel home: F16, one rounding of each FP32 row sum
        self._sym = []
        for b in self.c:
            tabs = {}
            for name, shape, dt in (("rows_recv", (P, self.Cr, self.d), adt), ("meta_recv", (P, self.MW), torch.int32),
                                    ("back", (P, self.Cr, self.d), self.back_dtype)):
                t = symm.empty(shape, dtype=dt, device=dev)
                t.zero_()
                h = symm.rendezvous(t, group)
                self._sym.append((t, h))
                b[name] = t
                tabs[name] = torch.tensor([int(p) for p in h.buffer_ptrs], dtype=torch.int64, device=dev)
            b["ptrs"] = tabs
            b["token"] = torch.zeros(1, dtype=torch.int32, device=dev)
        self.pushes = True

    def _barrier(self, c):
        """Every rank's kernels enqueued so far on this chunk's stream have finished before any rank's later kernels start: a
        one-element all-reduce (the library's own bounded, abortable wait - no spin of ours)."""
        dist.all_reduce(self.c[c]["token"], group=self.peer_group)

    def use_peer_tables(self, tables, back_dtype=torch.float16):
        """Installs the address tables of the peers' receive buffers for every chunk: tables[c][name] = int64 device tensor of P
        addresses for name in rows_recv / meta_recv / back (how _map_peer_buffers sets them; tests with every rank on one GPU
        build them by hand)."""
        self.back_dtype = back_dtype
        for b, t in zip(self.c, tables):
            b["ptrs"] = t
        self.pushes = True

    def plan_push(self, c, barrier=True):
        """plan(), with the rows and the metadata written into the destinations' receive buffers by the gather itself."""
        from ._lib import call

        K, b = self.K, self.c[c]
        T = b["x"].shape[0]
        call("strix_ep_plan", K._p(b["ids"]), K._p(b["coef"]), T, self.A, self.E, K._p(self.owner), K._p(self.local_of), self.P, self.rank, self.Cr, self.Cs,
             K._p(b["rowtok"]), K._p(b["meta_send"]), K._p(b["pos"]), K._p(b["flags"]), K._p(b["plan_scratch"]), self._sp(c))
        call("strix_ep_push_rows", K._p(b["x"]), self.d, int(self.act), K._p(b["rowtok"]), K._p(b["meta_send"]), self.P, self.rank, self.Cr, self.Cs,
             K._p(b["ptrs"]["rows_recv"]), K._p(b["ptrs"]["meta_recv"]), self._sp(c))
        self.launches += 4
        if barrier:
            self._barrier(c)

    def experts_push(self, c, barrier=True):
        """experts(), with every row sum written into its home rank's `back` buffer by the summing kernel itself."""
        from ._lib import call

        K, b = self.K, self.c[c]
        b["meta_last"] = b["meta_recv"]
        call("strix_ep_unpack", K._p(b["meta_recv"]), self.P, self.Cr, self.Cs, K._p(b["slot_ids"]), K._p(b["slot_row"]), self._sp(c))
        b["shard"].experts_partial(b["rows_recv"].reshape(-1, self.d), b["slot_ids"], partial=b["partial"], stream=self.streams[c], row_index=b["slot_row"])
        call("strix_ep_row_sum_push", K._p(b["partial"]), 1 if b["partial"].dtype == torch.float16 else 0, K._p(b["meta_recv"]), self.P, self.rank, self.Cr, self.Cs,
             self.d, K._p(b["ptrs"]["back"]), 1 if self.back_dtype == torch.float16 else 0, self._sp(c))
        self.launches += 9
        if barrier:
            self._barrier(c)

    # ---- the driver's hooks -------------------------------------------------------------------------------------------------
    def stream(self, c):
        return torch.cuda.stream(self.streams[c]) if self.streams[c] is not None else _NoStream()

    def _sp(self, c):
        return self.K._s(self.streams[c])

    def begin(self, x):
        self.launches = 0
        if self.chunks > 1:
            cur = torch.cuda.current_stream(self.dev)
            for s in self.streams:
                s.wait_stream(cur)

    def end(self, ys):
        if self.chunks > 1:
            cur = torch.cuda.current_stream(self.dev)
            for s in self.streams:
                cur.wait_stream(s)
        if len(ys) == 1:
            return ys[0]
        return self.y_full if all(y.shape[0] == self.Tc for y in ys) else torch.cat(ys, 0)

    def rows_recv(self, c):
        return self.c[c]["rows_recv"]

    def meta_recv(self, c):
        return self.c[c]["meta_recv"]

    def back(self, c):
        return self.c[c]["back"]

    def route(self, c, x):
        K, b, st = self.K, self.c[c], self.streams[c]
        T, R = x.shape[0], self.E + 1
        b["x"] = x
        if self.router_w.dtype == torch.bfloat16:
            K.linear_bf16w(x, self.router_w, b["logits"], T, R, self.d, self.act, K.Act.F32, stream=st)
        else:
            K.linear_f32w(x, self.router_w, b["logits"], T, R, self.d, self.act, K.Act.F32, stream=st)
        if self.router_bias is not None:
            b["logits"][:, : self.E] += self.router_bias
        K.moe_router(b["logits"], R, T, self.E, self.k, b["logits"][:, self.E:], R, self.E, b["ids"], b["coef"], K.Act.F32, b["err"], stream=st)
        self.launches += 2

    def plan(self, c):
        from ._lib import call

        K, b = self.K, self.c[c]
        T = b["x"].shape[0]
        call("strix_ep_plan", K._p(b["ids"]), K._p(b["coef"]), T, self.A, self.E, K._p(self.owner), K._p(self.local_of), self.P, self.rank, self.Cr, self.Cs,
             K._p(b["rowtok"]), K._p(b["meta_send"]), K._p(b["pos"]), K._p(b["flags"]), K._p(b["plan_scratch"]), self._sp(c))
        call("strix_ep_gather_rows", K._p(b["x"]), self.d, int(self.act), K._p(b["rowtok"]), K._p(b["meta_send"]), self.P, self.Cr, self.Cs, K._p(b["rows_send"]),
             self._sp(c))
        self.launches += 4  # the plan is three launches (count, scan, place)
        return b["rows_send"], b["meta_send"]

    def experts(self, c, rows_recv, meta_recv):
        from ._lib import call

        K, b = self.K, self.c[c]
        b["meta_last"] = meta_recv
        call("strix_ep_unpack", K._p(meta_recv), self.P, self.Cr, self.Cs, K._p(b["slot_ids"]), K._p(b["slot_row"]), self._sp(c))
        b["shard"].experts_partial(rows_recv.reshape(-1, self.d), b["slot_ids"], partial=b["partial"], stream=self.streams[c], row_index=b["slot_row"])
        call("strix_ep_row_sum", K._p(b["partial"]), 1 if b["partial"].dtype == torch.float16 else 0, K._p(meta_recv), self.P, self.Cr, self.Cs, self.d, K._p(b["summed"]), self._sp(c))
        self.launches += 9  # unpack, grouping (3), tiles, ordered rows, two FFN kernels, row sum
        return b["summed"]

    def home(self, c, back):
        from ._lib import call

        K, b = self.K, self.c[c]
        T = b["x"].shape[0]
        call("strix_ep_home_sum", K._p(back), 1 if back.dtype == torch.float16 else 0, K._p(b["pos"]), K._p(b["ids"]), T, self.A, self.E, self.P, self.Cr, self.d, K._p(b["y"][:T]), int(self.act), self._sp(c))
        self.launches += 1
        return b["y"][:T]

    # ---- after a step ---------------------------------------------------------------------------------------------------------
    def check(self):
        """Raises if a step overflowed a capacity, a router or expert error word is set, or a tensor-core wait was given up."""
        from ._lib import StrixError

        for i, b in enumerate(self.c):
            f = b["flags"].cpu().numpy().view(np.uint32)
            if f[0] or f[1]:
                raise StrixError("expert-parallel exchange overflowed its fixed capacity in chunk %d: %d rows (capacity %d), %d slots (capacity %d) "
                                 "for one destination; raise slot_capacity" % (i, f[0], self.Cr, f[1], self.Cs))
            self.K.check_router_error(b["err"], "expert-parallel router")
            e = b["shard"].probe("err", 1).cpu().numpy()
            if e[3]:
                raise StrixError("expert-parallel experts: error words %s" % e[3:6].tolist())

    def received_slots(self):
        return float(sum(int(b["meta_last"][:, 1].sum().item()) for b in self.c if "meta_last" in b))


class CudaLayer:
    """ExpertParallelMoe over a CudaBackend: the object bench.py and the GPU tests use."""

    def __init__(self, backend, world, rank, group=None):
        self.backend, self.chunks = backend, backend.chunks
        self.ep = ExpertParallelMoe(world, rank, backend, group=group, chunks=backend.chunks)

    def forward(self, x):
        return self.ep.forward(x)

    def check(self):
        self.backend.check()

    def received_slots(self):
        return self.backend.received_slots()

    def launches_per_step(self):
        return self.backend.launches

    def last_logits(self):
        return torch.cat([b["logits"] for b in self.backend.c], 0)

    def last_ids(self):
        return torch.cat([b["ids"] for b in self.backend.c], 0)


def cuda_layer(d, I, E, k, act, router_w, router_bias, gate_up_local, down_local, world, rank, max_local_tokens, placement=None, group=None, math=2, chunks=0,
               dedup=True, slot_capacity=None, peer_stores=True):
    """The expert-parallel layer on this rank's GPU (see CudaBackend). placement: the dict of placement() (default: contiguous).
    chunks: token chunks per step on separate streams (0 = two from four ranks on while a chunk keeps 2048 tokens, else one). peer_stores: with several ranks, keep the receive buffers in
    peer-mapped memory and let the gather and the row-sum kernels write into the destinations' buffers (False: all-to-alls)."""
    if not dedup:
        raise ValueError("cuda_layer: the one-row-per-slot exchange was removed; rows go once per (token, rank)")
    place = placement if placement is not None else globals()["placement"](E, world, balanced=False)
    if chunks <= 0:
        # measured at 16384 tokens in total: two chunks on two streams hide part of the exchange at 4 ranks (0.86 -> 0.81 ms, chunks of
        # 2048 tokens), change nothing at 2 ranks, and cost 14 % at 8 ranks (chunks of 1024 tokens: the per-chunk launches outweigh
        # the overlap) - so: two chunks from 4 ranks on while a chunk keeps at least 2048 tokens
        chunks = 2 if world >= 4 and max_local_tokens % 2 == 0 and max_local_tokens // 2 >= 2048 else 1
    peer_group = None
    if peer_stores and world > 1:  # peer-mapped receive buffers: the exchange rides on the kernels' own stores
        peer_group = group if group is not None else dist.group.WORLD
    be = CudaBackend(d, I, E, k, act, router_w, router_bias, gate_up_local, down_local, world, rank, place, max_local_tokens, chunks=chunks, math=math,
                     slot_capacity=slot_capacity, peer_group=peer_group)
    return CudaLayer(be, world, rank, group=group)


def shard_stack(full, E, world, rank, place=None):
    """This rank's slice of a full stacked weight [(E + 1) * N, K] (kernels.QWeight): its routed experts in placement order
    followed by the shared expert (expert E), as a new QWeight."""
    from . import kernels as K

    place = place if place is not None else placement(E, world, balanced=False)
    N = full.N // (E + 1)
    rb = K.row_bytes(full.bits, full.K)
    dev = full.q.device
    ex = torch.from_numpy(np.concatenate([place["experts_of"][rank], np.array([E], np.int64)])).to(dev)
    rows = (ex[:, None] * N + torch.arange(N, device=dev)[None, :]).reshape(-1)
    q = full.q.view(-1, rb).index_select(0, rows).reshape(-1)
    return K.QWeight(full.bits, rows.numel(), full.K, full.G, q, full.scale.index_select(0, rows), full.minv.index_select(0, rows))
