"""Expert-parallel MoE layer with the row exchange done by peer stores over NVLink, overlapped with the expert products.

Instead of gather -> NCCL all-to-all -> regroup (``b2g/ep.py``), the token permute and the transfer are one kernel: every
routed row is read from the token matrix on its source rank and written straight into the owner rank's receive buffer,
already grouped by (local expert, source rank); the way back is the mirror image.  The slots follow from the all-gathered
per-rank expert histograms, computed by one small kernel on the device (``build_peer_plan_device``; ``build_peer_plan`` is
the same arithmetic as tensor ops, kept as the checkable statement of it), so no split size is read on the host and nothing
is regrouped afterwards.  Every rank starts its scatter at a different owner's experts, so that the ranks do not all store
to one GPU at a time.

Overlap.  The rank's tokens are cut into ``chunks`` ranges.  The exchanges run on a stream of their own, the expert
products on the caller's stream, and events hand the chunks over, so that chunk ``c+1`` crosses NVLink while chunk ``c``
computes, in both directions of both passes:

    exchange stream :  scatter 0 | scatter 1 |            | return 0 | return 1 |
    compute stream  :            | experts 0 | experts 1  |          | combine 0 | combine 1

The exchange kernels are small enough (128 threads, 48 registers, no shared memory) to sit on the same SMs as the GEMM's
CTA.  The whole layer is ONE autograd node whose backward is written out by hand in the mirrored order, because autograd
would enqueue the two chunks' backward kernels one chunk after the other and undo the overlap.

Buffers are symmetric allocations (one per rank, same size, mapped into every rank): two receive buffers (activations
forward, output gradients backward) and two return buffers of the rank's own routed-row count.  By default a receive
buffer holds the worst case -- every routed row of every rank -- so that no router, however skewed, overflows it; with a
smaller ``capacity_factor`` an overflow is contained (the rows beyond the buffer are dropped, every consumer is clamped to
it) and reported as status 901.  A layer object owns the buffers; its outputs alias them until the next call of the same
layer (a multi-layer model needs one object per layer).  Ranks synchronise after each exchange with a one-element NCCL
all-reduce on the exchange stream (no device-side spin loops of our own); multicast is not used.

Placement.  ``balanced_placement`` spreads the experts over the ranks by measured load (same number of experts per rank,
longest-processing-time first), for routers whose load is skewed but stable; the layer maps the router's expert ids through
that table before it sorts them.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist

from . import _lib, ops


@dataclass
class PeerPlan:
    my_start: torch.Tensor       # int32 [E]   first sorted position of expert e on this rank
    dest_base: torch.Tensor      # int32 [E]   slot at the owner where this rank's rows of expert e start
    blk_start: torch.Tensor      # int32 [E_l*G + 1] owner side: start of block (local expert, source rank)
    src_pos: torch.Tensor        # int32 [E_l*G]     position of that block's first row in the source's sorted order
    local_sizes: torch.Tensor    # int32 [E_l]
    local_offsets: torch.Tensor  # int32 [E_l]


def build_peer_plan(counts: torch.Tensor, rank: int, capacity: Optional[int] = None) -> PeerPlan:
    """counts: int32/int64 [G, E], row g = histogram of rank g's routed rows over all experts.  With ``capacity`` the
    owner-side segments are clamped to that many rows, as the kernel does."""
    g, e = counts.shape
    per = e // g
    c = counts.to(torch.int64)
    total = c.sum(0)
    blocks = total.view(g, per)
    owner_prefix = (blocks.cumsum(1) - blocks).reshape(e)         # rows of the owner's earlier experts
    src_prefix = c.cumsum(0) - c                                   # rows of earlier source ranks, per expert
    my_start_all = c.cumsum(1) - c                                 # where expert e starts in each rank's sorted order
    lo, hi = rank * per, (rank + 1) * per
    blk_counts = c[:, lo:hi].t().contiguous().reshape(-1)          # (local expert, source rank) order
    blk_start = torch.cat([blk_counts.new_zeros(1), blk_counts.cumsum(0)])
    local_offsets = total[lo:hi].cumsum(0)
    if capacity is not None:
        blk_start = blk_start.clamp(max=capacity)
        local_offsets = local_offsets.clamp(max=capacity)
    local_sizes = torch.diff(local_offsets, prepend=local_offsets.new_zeros(1))
    i32 = torch.int32
    return PeerPlan(my_start=my_start_all[rank].to(i32).contiguous(), dest_base=(owner_prefix + src_prefix[rank]).to(i32).contiguous(),
                    blk_start=blk_start.to(i32).contiguous(), src_pos=my_start_all[:, lo:hi].t().contiguous().reshape(-1).to(i32),
                    local_sizes=local_sizes.to(i32).contiguous(), local_offsets=local_offsets.to(i32).contiguous())


def _plan_views(buf: torch.Tensor, g: int, e: int) -> PeerPlan:
    per = e // g
    return PeerPlan(*torch.split(buf, [e, e, per * g + 1, per * g, per, per]))


def _plan_words(g: int, e: int) -> int:
    per = e // g
    return 2 * e + (per * g + 1) + per * g + 2 * per


def _launch_plan(counts: torch.Tensor, stride: int, g: int, e: int, rank: int, plan: PeerPlan, capacity: int) -> None:
    dev = counts.device
    with torch.cuda.device(dev):
        _lib.call("b2g_ep_peer_plan", C.c_void_p(counts.data_ptr()), int(stride), g, e, int(rank),
                  *(C.c_void_p(t.data_ptr()) for t in (plan.my_start, plan.dest_base, plan.blk_start, plan.src_pos, plan.local_sizes,
                                                       plan.local_offsets)),
                  int(capacity), C.c_void_p(ops.status_word(dev).data_ptr()), C.c_void_p(torch.cuda.current_stream(dev).cuda_stream))


def build_peer_plan_device(counts: torch.Tensor, rank: int, capacity: Optional[int] = None) -> PeerPlan:
    """The same plan as :func:`build_peer_plan` in one kernel launch (``counts``: int32 [G, E] on the GPU)."""
    g, e = counts.shape
    plan = _plan_views(torch.empty(_plan_words(g, e), dtype=torch.int32, device=counts.device), g, e)
    _launch_plan(counts, e, g, e, rank, plan, (1 << 31) - 1 if capacity is None else capacity)
    return plan


# ---- static load-aware expert placement ---------------------------------------------------------------------------------
def balanced_placement(load: torch.Tensor, world: int) -> torch.Tensor:
    """Placed id of every expert, int64 [E]: rank ``placed // (E / world)`` owns it as its local expert ``placed % (E / world)``.

    ``load[e]`` is the measured number of rows routed to expert ``e`` (a histogram over one or more batches).  Experts are
    taken from the heaviest down and each goes to the rank with the least load so far among the ranks that still have a
    free slot, every rank ending with exactly ``E / world`` experts.  Deterministic: ties go to the smaller expert id and
    the smaller rank, so every rank derives the same table from the same (all-reduced) histogram."""
    e = load.numel()
    if e % world:
        raise ValueError(f"{e} experts do not divide over {world} ranks")
    per = e // world
    weights = [float(v) for v in load.detach().cpu().double().tolist()]
    order = sorted(range(e), key=lambda i: (-weights[i], i))
    rank_load, rank_fill = [0.0] * world, [0] * world
    placed = [0] * e
    for ex in order:
        g = min((r for r in range(world) if rank_fill[r] < per), key=lambda r: (rank_load[r], r))
        placed[ex] = g * per + rank_fill[g]
        rank_fill[g] += 1
        rank_load[g] += weights[ex]
    return torch.tensor(placed, dtype=torch.int64)


def contiguous_placement(num_experts: int) -> torch.Tensor:
    return torch.arange(num_experts, dtype=torch.int64)


def experts_of_rank(placement: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Original ids of the experts rank ``rank`` holds, in its local order (the inverse of the placement on its block)."""
    e = placement.numel()
    per = e // world
    inverse = torch.empty(e, dtype=torch.int64)
    inverse[placement.cpu()] = torch.arange(e, dtype=torch.int64)
    return inverse[rank * per:(rank + 1) * per]


def rank_loads(load: torch.Tensor, placement: torch.Tensor, world: int) -> torch.Tensor:
    """Rows per rank under a placement, float64 [world]."""
    per = load.numel() // world
    out = torch.zeros(world, dtype=torch.float64)
    out.index_add_(0, placement.cpu() // per, load.detach().cpu().double())
    return out


# ---- buffers and exchange kernels -----------------------------------------------------------------------------------------
class PeerExchange:
    """Symmetric receive / return buffers of one MoE layer, its exchange stream and the two exchange kernels."""

    MAX_BUFFER_BYTES = 16 << 30      # all four buffers of a layer together; a worst-case size beyond this is cut down to it

    def __init__(self, rows_local: int, hidden: int, num_experts: int, group=None, capacity_factor: Optional[float] = None,
                 device: Optional[torch.device] = None, chunks: int = 1, placement: Optional[torch.Tensor] = None):
        import torch.distributed._symmetric_memory as symm

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.rows_local, self.hidden, self.num_experts = int(rows_local), int(hidden), int(num_experts)
        if num_experts % self.world:
            raise ValueError(f"{num_experts} experts do not divide over {self.world} ranks")
        self.experts_per_rank = num_experts // self.world
        self.chunks = max(1, int(chunks))
        self.placement = None if placement is None else placement.to(device=self.device, dtype=torch.int64).contiguous()
        # rows per chunk are bounded by ceil(rows_local / chunks) rounded up to a whole token; the receive side of a chunk holds,
        # in the worst case, that many rows from every rank
        self.chunk_rows = -(-self.rows_local // self.chunks)
        factor = float(self.world) if capacity_factor is None else float(capacity_factor)
        cap = int(self.chunk_rows * min(factor, float(self.world)))
        row_bytes = 2 * hidden
        budget_rows = (self.MAX_BUFFER_BYTES // row_bytes - 2 * self.rows_local) // (2 * self.chunks)
        cap = max(512, min(cap, budget_rows))
        self.capacity = (cap + 511) // 512 * 512                  # rows of ONE chunk's receive buffer
        self.recv, self.ret, self._recv_ptrs, self._ret_ptrs = [], [], [], []
        for _ in range(2):
            for store, ptrs, rows in ((self.recv, self._recv_ptrs, self.capacity * self.chunks), (self.ret, self._ret_ptrs, max(1, self.rows_local))):
                t = symm.empty((rows, hidden), dtype=torch.bfloat16, device=self.device)
                h = symm.rendezvous(t, self.group)
                store.append(t)
                ptrs.append([int(p) for p in h.buffer_ptrs])
        self._flag = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.stream = torch.cuda.Stream(device=self.device, priority=-1)
        words = _plan_words(self.world, num_experts)
        self._plan_buf = torch.empty(self.chunks, words, dtype=torch.int32, device=self.device)
        self.plans = [_plan_views(self._plan_buf[c], self.world, num_experts) for c in range(self.chunks)]
        self.counts_mine = torch.zeros(self.chunks, num_experts, dtype=torch.int32, device=self.device)
        self.counts_all = torch.zeros(self.world, self.chunks, num_experts, dtype=torch.int32, device=self.device)
        self.local_ids = torch.arange(self.experts_per_rank, device=self.device, dtype=torch.int64)
        self._ptr_cache: dict[tuple[int, int, int], torch.Tensor] = {}
        self.events = {name: [torch.cuda.Event() for _ in range(self.chunks)] for name in
                       ("sent", "computed", "returned", "g_ready", "g_sent", "g_computed", "g_returned")}
        self.ev_plan = torch.cuda.Event()
        self.profile = False
        self.trace: list = []

    def phase_ms(self) -> dict[str, float]:
        """Summed device time per phase name of the spans recorded since ``trace`` was last cleared (synchronises)."""
        torch.cuda.synchronize(self.device)
        out: dict[str, float] = {}
        for name, a, b in self.trace:
            out[name] = out.get(name, 0.0) + a.elapsed_time(b)
        return out

    # -- geometry ---------------------------------------------------------------------------------------------------------
    def token_bounds(self, tokens: int) -> list[tuple[int, int]]:
        """Token range of every chunk: equal parts, the first ``tokens % chunks`` one token longer."""
        base, extra = divmod(tokens, self.chunks)
        out, t0 = [], 0
        for c in range(self.chunks):
            t1 = t0 + base + (1 if c < extra else 0)
            out.append((t0, t1))
            t0 = t1
        return out

    def recv_view(self, which: int, chunk: int) -> torch.Tensor:
        return self.recv[which][chunk * self.capacity:(chunk + 1) * self.capacity]

    def _peer_table(self, kind: int, which: int, row0: int) -> torch.Tensor:
        """Device array of every rank's address of row ``row0`` of a buffer (kind 0 = receive, 1 = return)."""
        key = (kind, which, row0)
        t = self._ptr_cache.get(key)
        if t is None:
            base = (self._recv_ptrs if kind == 0 else self._ret_ptrs)[which]
            t = torch.tensor([p + row0 * self.hidden * 2 for p in base], dtype=torch.int64, device=self.device)
            self._ptr_cache[key] = t
        return t

    # -- pieces (each runs on the CURRENT stream) ---------------------------------------------------------------------------
    def sync(self) -> None:
        """All ranks' earlier work on this stream is complete before any rank continues on it."""
        dist.all_reduce(self._flag, group=self.group)

    def gather_counts(self) -> None:
        dist.all_gather_into_tensor(self.counts_all.view(-1), self.counts_mine.view(-1), group=self.group)

    def plan_chunk(self, chunk: int) -> PeerPlan:
        _launch_plan(self.counts_all[0, chunk], self.chunks * self.num_experts, self.world, self.num_experts, self.rank, self.plans[chunk],
                     self.capacity)
        return self.plans[chunk]

    def scatter(self, src: torch.Tensor, perm: Optional[torch.Tensor], top_k: int, sorted_expert: torch.Tensor, chunk: int, which: int):
        """Rows of ``src`` (gathered through ``perm`` when given) into the owners' receive buffers of this chunk."""
        rows = sorted_expert.numel()
        plan = self.plans[chunk]
        peers = self._peer_table(0, which, chunk * self.capacity)
        with torch.cuda.device(self.device):
            _lib.call("b2g_ep_scatter_rows", C.c_void_p(src.data_ptr()), None if perm is None else C.c_void_p(perm.data_ptr()), int(top_k),
                      C.c_void_p(sorted_expert.data_ptr()), C.c_void_p(plan.my_start.data_ptr()), C.c_void_p(plan.dest_base.data_ptr()),
                      C.c_void_p(peers.data_ptr()), self.experts_per_rank, rows, self.hidden, self.capacity,
                      ((self.rank + 1) % self.world) * self.experts_per_rank,      # start with the next rank's experts
                      C.c_void_p(ops.status_word(self.device).data_ptr()), C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream))

    def give_back(self, rows: torch.Tensor, chunk: int, which: int, row0: int) -> None:
        """Rows of this rank's receive-side result back to their sources, at ``row0`` + sorted position of their return buffer."""
        plan = self.plans[chunk]
        peers = self._peer_table(1, which, row0)
        with torch.cuda.device(self.device):
            _lib.call("b2g_ep_return_rows", C.c_void_p(rows.data_ptr()), C.c_void_p(plan.blk_start.data_ptr()), C.c_void_p(plan.src_pos.data_ptr()),
                      C.c_void_p(peers.data_ptr()), self.world, self.experts_per_rank * self.world, self.hidden, self.capacity,
                      C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream))


class _Span:
    """Optional timing of one phase on one stream: a pair of timing events appended to ``xchg.trace`` while
    ``xchg.profile`` is set (the benchmark's phase table); free otherwise."""

    def __init__(self, xchg: "PeerExchange", name: str, stream: torch.cuda.Stream):
        self.on = xchg.profile
        if self.on:
            self.xchg, self.name, self.stream = xchg, name, stream
            self.a, self.b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def __enter__(self):
        if self.on:
            self.a.record(self.stream)

    def __exit__(self, *exc):
        if self.on:
            self.b.record(self.stream)
            self.xchg.trace.append((self.name, self.a, self.b))


class _PeerMoe(torch.autograd.Function):
    """The whole expert-parallel layer as one node: chunked, exchanges on their own stream, backward in mirrored order."""

    @staticmethod
    def forward(ctx, xchg: PeerExchange, hidden, top_k_index, top_k_weights, gate_p, up_p, down_p, quant_type, inter_dim, scaling,
                gu_a, gu_b, down_a, down_b):
        from . import autograd as ag

        tokens, top_k = top_k_index.shape
        if tokens * top_k > xchg.rows_local or hidden.shape[1] != xchg.hidden:
            raise ValueError(f"the exchange buffers hold {xchg.rows_local} routed rows of width {xchg.hidden}; got {tokens * top_k} x {hidden.shape[1]}")
        dev = hidden.device
        cs, xs, ev = torch.cuda.current_stream(dev), xchg.stream, xchg.events
        bounds = xchg.token_bounds(tokens)
        hidden = hidden.contiguous()
        weights = top_k_weights.contiguous()
        ids = top_k_index if xchg.placement is None else xchg.placement[top_k_index.long()]

        routes = []                                      # per chunk: (sorted expert ids, permutation, inverse, first row of the chunk)
        row0 = 0
        with _Span(xchg, "plan", cs):
            for c, (t0, t1) in enumerate(bounds):
                sorted_e, perm, inverse, sizes, _ = ops.route_plan(ids[t0:t1].contiguous(), xchg.num_experts)
                xchg.counts_mine[c].copy_(sizes)
                routes.append((sorted_e, perm, inverse, row0))
                row0 += (t1 - t0) * top_k
        xchg.ev_plan.record(cs)

        with torch.cuda.stream(xs):
            xs.wait_event(xchg.ev_plan)
            with _Span(xchg, "plan_exchange", xs):
                xchg.gather_counts()
                for c in range(xchg.chunks):
                    xchg.plan_chunk(c)
            for c, (t0, t1) in enumerate(bounds):
                sorted_e, perm, _, _ = routes[c]
                # No wait is needed before writing a receive buffer: its last readers (the previous call's backward) were
                # enqueued before that call's final sync(), which every rank has passed to get here.
                with _Span(xchg, "dispatch", xs):
                    xchg.scatter(hidden[t0:t1], perm, top_k, sorted_e, c, 0)
                    xchg.sync()                          # every source has delivered chunk c
                ev["sent"][c].record(xs)

        lora = gu_a is not None
        saved, outs = [], []
        for c in range(xchg.chunks):
            cs.wait_event(ev["sent"][c])
            plan = xchg.plans[c]
            with _Span(xchg, "experts_forward", cs):
                out_c, sv = ag.expert_block_forward(xchg.recv_view(0, c), gate_p, up_p, down_p, quant_type, quant_type, inter_dim,
                                                    xchg.local_ids, plan.local_offsets, plan.local_offsets, gu_a if lora else None,
                                                    gu_b if lora else None, down_a if lora else None, down_b if lora else None, scaling, 0.0)
            ev["computed"][c].record(cs)
            saved.append(sv)
            outs.append(out_c)

        with torch.cuda.stream(xs):
            for c in range(xchg.chunks):
                xs.wait_event(ev["computed"][c])
                with _Span(xchg, "return", xs):
                    xchg.give_back(outs[c], c, 0, routes[c][3])
                    xchg.sync()
                ev["returned"][c].record(xs)

        out = torch.empty(tokens, xchg.hidden, dtype=torch.bfloat16, device=dev)
        returned = []
        for c, (t0, t1) in enumerate(bounds):
            cs.wait_event(ev["returned"][c])
            rows_c = xchg.ret[0][routes[c][3]:routes[c][3] + (t1 - t0) * top_k]
            with _Span(xchg, "combine", cs):
                ops.route_combine(rows_c, weights[t0:t1], routes[c][2], out=out[t0:t1])
            returned.append(rows_c)
        # `outs` were read by the exchange stream; the compute stream has waited for the last of those reads above, so the
        # allocator may hand their memory to later work of the compute stream
        ctx.xchg, ctx.saved, ctx.routes, ctx.bounds, ctx.top_k = xchg, saved, routes, bounds, top_k
        ctx.returned, ctx.weights, ctx.lora = returned, weights, lora
        return out

    @staticmethod
    def backward(ctx, grad_out):
        from . import autograd as ag

        xchg, routes, bounds, top_k = ctx.xchg, ctx.routes, ctx.bounds, ctx.top_k
        dev = grad_out.device
        cs, xs, ev = torch.cuda.current_stream(dev), xchg.stream, xchg.events
        grad_out = grad_out.contiguous()
        d_weights = torch.empty_like(ctx.weights)
        d_rows = []
        for c, (t0, t1) in enumerate(bounds):
            with _Span(xchg, "combine_backward", cs):
                d_out_c, d_w_c = ops.route_combine_bwd(ctx.returned[c], ctx.weights[t0:t1], routes[c][1], grad_out[t0:t1])
                d_weights[t0:t1].copy_(d_w_c)
            ev["g_ready"][c].record(cs)
            d_rows.append(d_out_c)

        with torch.cuda.stream(xs):
            for c in range(xchg.chunks):
                xs.wait_event(ev["g_ready"][c])
                with _Span(xchg, "dispatch_backward", xs):
                    xchg.scatter(d_rows[c], None, 1, routes[c][0], c, 1)
                    xchg.sync()
                ev["g_sent"][c].record(xs)

        grads, d_sel = [], []
        for c in range(xchg.chunks):
            cs.wait_event(ev["g_sent"][c])
            with _Span(xchg, "experts_backward", cs):
                g = ag.expert_block_backward(ctx.saved[c], xchg.recv_view(1, c))
            ev["g_computed"][c].record(cs)
            d_sel.append(g[0])
            grads.append(g[1:])

        with torch.cuda.stream(xs):
            for c in range(xchg.chunks):
                xs.wait_event(ev["g_computed"][c])
                with _Span(xchg, "return_backward", xs):
                    xchg.give_back(d_sel[c], c, 1, routes[c][3])
                    xchg.sync()
                ev["g_returned"][c].record(xs)

        d_hidden = torch.empty(grad_out.shape[0], xchg.hidden, dtype=torch.bfloat16, device=dev)
        for c, (t0, t1) in enumerate(bounds):
            cs.wait_event(ev["g_returned"][c])
            rows_c = xchg.ret[1][routes[c][3]:routes[c][3] + (t1 - t0) * top_k]
            with _Span(xchg, "gather_backward", cs):
                ops.route_gather_bwd(rows_c, routes[c][2], t1 - t0, top_k, out=d_hidden[t0:t1])
        factor_grads = [None, None, None, None]
        if ctx.lora:
            factor_grads = list(grads[0])
            for more in grads[1:]:
                factor_grads = [a + b for a, b in zip(factor_grads, more)]
        ctx.saved = None
        return (None, d_hidden, None, d_weights, None, None, None, None, None, None, *factor_grads)


def peer_moe_layer(xchg: PeerExchange, hidden: torch.Tensor, top_k_index: torch.Tensor, top_k_weights: torch.Tensor,
                   gate_payload: torch.Tensor, up_payload: torch.Tensor, down_payload: torch.Tensor, quant_type: int, inter_dim: int,
                   lora: Optional[dict] = None, scaling: float = 1.0) -> torch.Tensor:
    """Expert-parallel layer; payloads / LoRA factors hold this rank's experts only (in the order of the exchange's placement),
    ``top_k_index`` carries the router's global ids."""
    lo = lora or {}
    return _PeerMoe.apply(xchg, hidden, top_k_index, top_k_weights, gate_payload, up_payload, down_payload, int(quant_type), int(inter_dim),
                          float(scaling), lo.get("gate_up_a"), lo.get("gate_up_b"), lo.get("down_a"), lo.get("down_b"))
