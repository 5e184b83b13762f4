"""Expert-parallel MoE layer with the row exchange done by peer stores over NVLink, overlapped with the expert products.

Instead of gather -> NCCL all-to-all -> regroup (``b2g/ep.py``), the token permute and the transfer are one kernel: every
routed row is read from the token matrix on its source rank and written straight into the owner rank's receive buffer,
already grouped by (local expert, source rank); the way back is the mirror image.  The slots follow from the all-gathered
per-rank expert histograms, computed by one small kernel on the device (``build_peer_plan_device``; ``build_peer_plan`` is
the same arithmetic as tensor ops, kept as the checkable statement of it), so no split size is read on the host and nothing
is regrouped afterwards.  Every rank starts its scatter at a different owner's experts, so that the ranks do not all store
to one GPU at a time.

Overlap.  Every rank's experts are cut into ``chunks`` EXPERT GROUPS (the same ranges of local expert indices on every
rank).  The rows of one group are exchanged by one launch; the exchanges run on a stream of their own, the expert products
on the caller's stream, and events hand the groups over, so that group ``c+1`` crosses NVLink while group ``c`` computes, in
both directions of both passes:

    exchange stream :  scatter 0 | scatter 1 | scatter 2 |  return 0 | return 1  | return 2 |
    compute stream  :            | experts 0 | experts 1 | experts 2 |           |          | combine

Cutting by experts rather than by tokens keeps every expert's rows together (its packed weight is unpacked once per 512 rows
whatever the number of groups), needs one routing plan per step, and lets each group write its own rows of shared
activation buffers and its own experts' factor gradients.  The exchange kernels are small enough (128 threads, 32 registers,
no shared memory, one CTA per SM) to sit on the same SMs as the GEMM's CTA.  The whole layer is ONE autograd node whose
backward is written out by hand in the mirrored order.

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
def group_ranges(experts_per_rank: int, chunks: int) -> list[tuple[int, int]]:
    """The expert groups of a rank: ``chunks`` contiguous ranges of local expert indices, equal parts, the first
    ``experts_per_rank % chunks`` one expert longer."""
    chunks = max(1, min(int(chunks), experts_per_rank))
    base, extra = divmod(experts_per_rank, chunks)
    out, lo = [], 0
    for c in range(chunks):
        hi = lo + base + (1 if c < extra else 0)
        out.append((lo, hi))
        lo = hi
    return out


def _fill_bins(items: list[int], weights: list[float], capacities: list[int]) -> list[list[int]]:
    """Longest-processing-time first into bins of fixed capacities: ``items`` (heaviest first) each go to the bin with the least
    weight so far among those with a free slot; ties to the smaller bin."""
    load, bins = [0.0] * len(capacities), [[] for _ in capacities]
    for it in items:
        b = min((i for i in range(len(capacities)) if len(bins[i]) < capacities[i]), key=lambda i: (load[i], i))
        bins[b].append(it)
        load[b] += weights[it]
    return bins


def balanced_placement(load: torch.Tensor, world: int, chunks: int = 1) -> torch.Tensor:
    """Placed id of every expert, int64 [E]: rank ``placed // (E / world)`` owns it as its local expert ``placed % (E / world)``.

    ``load[e]`` is the measured number of rows routed to expert ``e`` (a histogram over one or more batches).  Experts are
    taken from the heaviest down and each goes to the rank with the least load so far among the ranks that still have a
    free slot, every rank ending with exactly ``E / world`` experts.  Within a rank the same rule spreads its experts over the
    ``chunks`` expert groups of the exchange pipeline (``group_ranges``), so that the groups carry equal loads too.
    Deterministic: ties go to the smaller expert id and the smaller bin, so every rank derives the same table from the same
    (all-reduced) histogram."""
    e = load.numel()
    if e % world:
        raise ValueError(f"{e} experts do not divide over {world} ranks")
    per = e // world
    weights = [float(v) for v in load.detach().cpu().double().tolist()]
    order = sorted(range(e), key=lambda i: (-weights[i], i))
    ranges = group_ranges(per, chunks)
    placed = [0] * e
    for g, members in enumerate(_fill_bins(order, weights, [per] * world)):
        slot = 0
        for group in _fill_bins(members, weights, [hi - lo for lo, hi in ranges]):
            for ex in group:
                placed[ex] = g * per + slot
                slot += 1
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
                 device: Optional[torch.device] = None, chunks: int = 1, placement: Optional[torch.Tensor] = None, exchange_tpcs: int = 0):
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
        self.placement = None if placement is None else placement.to(device=self.device, dtype=torch.int64).contiguous()
        self.groups = group_ranges(self.experts_per_rank, chunks)
        self.chunks = len(self.groups)
        # Where an exchange runs while expert products of another group compute: 0 = on the same SMs (a small kernel beside the
        # GEMM's CTA); n > 0 = on n TPCs (2n SMs) of its own, which the GEMM is told to leave free
        self.exchange_tpcs = int(exchange_tpcs) if self.chunks > 1 else 0
        # a receive buffer holds, in the worst case, the routed rows of every rank
        factor = float(self.world) if capacity_factor is None else float(capacity_factor)
        cap = int(self.rows_local * min(factor, float(self.world)))
        row_bytes = 2 * hidden
        budget_rows = (self.MAX_BUFFER_BYTES // row_bytes - 2 * self.rows_local) // 2
        cap = max(512, min(cap, budget_rows))
        self.capacity = (cap + 511) // 512 * 512
        self.recv, self.ret, self._recv_ptrs, self._ret_ptrs = [], [], [], []
        for _ in range(2):
            for store, ptrs, rows in ((self.recv, self._recv_ptrs, self.capacity), (self.ret, self._ret_ptrs, max(1, self.rows_local))):
                t = symm.empty((rows, hidden), dtype=torch.bfloat16, device=self.device)
                h = symm.rendezvous(t, self.group)
                store.append(t)
                ptrs.append(torch.tensor([int(p) for p in h.buffer_ptrs], dtype=torch.int64, device=self.device))
        self._flag = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.stream = torch.cuda.Stream(device=self.device, priority=-1)
        self.plan = _plan_views(torch.empty(_plan_words(self.world, num_experts), dtype=torch.int32, device=self.device), self.world, num_experts)
        self.counts_mine = torch.zeros(num_experts, dtype=torch.int32, device=self.device)
        self.counts_all = torch.zeros(self.world, num_experts, dtype=torch.int32, device=self.device)
        self.local_ids = torch.arange(self.experts_per_rank, device=self.device, dtype=torch.int64)
        # first row and end row of every group inside the receive buffer: one-element views of the plan's cumulative ends
        off = self.plan.local_offsets
        self.group_first = [None if lo == 0 else off[lo - 1:lo] for lo, _ in self.groups]
        self.group_end = [off[hi - 1:hi] for _, hi in self.groups]
        self.events = {name: [torch.cuda.Event() for _ in range(self.chunks)] for name in
                       ("sent", "computed", "returned", "g_sent", "g_computed", "g_returned")}
        self.ev_plan, self.ev_ready = torch.cuda.Event(), torch.cuda.Event()
        self.profile = False
        self.trace: list = []

    def phase_ms(self) -> dict[str, float]:
        """Summed device time per phase name of the spans recorded since ``trace`` was last cleared (synchronises)."""
        torch.cuda.synchronize(self.device)
        out: dict[str, float] = {}
        for name, a, b in self.trace:
            out[name] = out.get(name, 0.0) + a.elapsed_time(b)
        return out

    def timeline(self) -> list[tuple[str, float, float]]:
        """(phase, start ms, end ms) of every recorded span, relative to the first one (synchronises)."""
        torch.cuda.synchronize(self.device)
        if not self.trace:
            return []
        origin = self.trace[0][1]
        return [(name, origin.elapsed_time(a), origin.elapsed_time(b)) for name, a, b in self.trace]

    # -- pieces (each runs on the CURRENT stream) ---------------------------------------------------------------------------
    def sync(self) -> None:
        """All ranks' earlier work on this stream is complete before any rank continues on it."""
        dist.all_reduce(self._flag, group=self.group)

    def make_plan(self) -> PeerPlan:
        """All-gather of the per-rank expert histograms (``counts_mine``) and the slot plan from them, one launch each."""
        dist.all_gather_into_tensor(self.counts_all.view(-1), self.counts_mine, group=self.group)
        _launch_plan(self.counts_all, self.num_experts, self.world, self.num_experts, self.rank, self.plan, self.capacity)
        return self.plan

    ALONE = 8                        # CTAs per SM of the small kernel for an exchange that nothing computes beside

    def _beside(self) -> int:
        """Launch shape of an exchange that runs while experts compute: the wide kernel on TPCs of its own, or one small CTA per SM."""
        return -self.exchange_tpcs if self.exchange_tpcs else 1

    def gemm_margin(self, on: bool) -> None:
        """The GEMMs launched from here on leave the exchange's SMs free (or, ``on = False``, use the whole GPU again)."""
        if self.exchange_tpcs:
            _lib.call("b2g_set_gemm_sm_margin", 2 * self.exchange_tpcs if on else 0)

    def scatter(self, src: torch.Tensor, perm: Optional[torch.Tensor], top_k: int, sorted_expert: torch.Tensor, chunk: int, which: int) -> None:
        """Rows of ``src`` (gathered through ``perm`` when given) that belong to expert group ``chunk`` into the owners' receive
        buffers.  The first group's scatter has nothing to hide behind (the experts wait for it), so it takes the whole GPU; the
        others run beside the previous group's expert products."""
        lo, hi = self.groups[chunk]
        with torch.cuda.device(self.device):
            _lib.call("b2g_ep_scatter_rows", C.c_void_p(src.data_ptr()), None if perm is None else C.c_void_p(perm.data_ptr()), int(top_k),
                      C.c_void_p(sorted_expert.data_ptr()), C.c_void_p(self.plan.my_start.data_ptr()), C.c_void_p(self.plan.dest_base.data_ptr()),
                      C.c_void_p(self._recv_ptrs[which].data_ptr()), self.experts_per_rank, self.world, self.rank, lo, hi,
                      sorted_expert.numel(), self.hidden, self.capacity, self.ALONE if chunk == 0 else self._beside(),
                      C.c_void_p(ops.status_word(self.device).data_ptr()), C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream))

    def give_back(self, rows: torch.Tensor, chunk: int, which: int) -> None:
        """Rows of expert group ``chunk`` of this rank's receive-side result back to their sources' return buffers (the last
        group's return runs after all expert products, alone)."""
        lo, hi = self.groups[chunk]
        with torch.cuda.device(self.device):
            _lib.call("b2g_ep_return_rows", C.c_void_p(rows.data_ptr()), C.c_void_p(self.plan.blk_start.data_ptr()),
                      C.c_void_p(self.plan.src_pos.data_ptr()), C.c_void_p(self._ret_ptrs[which].data_ptr()), self.world, lo * self.world,
                      hi * self.world, self.hidden, self.capacity, self.ALONE if chunk == self.chunks - 1 else self._beside(),
                      C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream))


class _Span:
    """Optional timing of one phase on one stream: a pair of timing events appended to ``xchg.trace`` while
    ``xchg.profile`` is set (the benchmark's phase table); free otherwise."""

    def __init__(self, xchg: PeerExchange, name: str, stream: torch.cuda.Stream):
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


def _bf16(rows: int, cols: int, dev) -> torch.Tensor:
    return torch.empty(rows, cols, dtype=torch.bfloat16, device=dev)


class _PeerMoe(torch.autograd.Function):
    """The whole expert-parallel layer as one node: expert groups, exchanges on their own stream, backward in mirrored order."""

    @staticmethod
    def forward(ctx, xchg: PeerExchange, hidden, top_k_index, top_k_weights, gate_p, up_p, down_p, quant_type, inter_dim, scaling,
                gu_a, gu_b, down_a, down_b):
        tokens, top_k = top_k_index.shape
        rows = tokens * top_k
        if rows > xchg.rows_local or hidden.shape[1] != xchg.hidden:
            raise ValueError(f"the exchange buffers hold {xchg.rows_local} routed rows of width {xchg.hidden}; got {rows} x {hidden.shape[1]}")
        dev = hidden.device
        cs, xs, ev = torch.cuda.current_stream(dev), xchg.stream, xchg.events
        hidden = hidden.contiguous()
        weights = top_k_weights.contiguous()
        ids = top_k_index if xchg.placement is None else xchg.placement[top_k_index.long()]
        e_local, cap, plan = xchg.experts_per_rank, xchg.capacity, xchg.plan
        lora = gu_a is not None
        r = gu_a.shape[1] if lora else 0

        with _Span(xchg, "plan", cs):
            sorted_e, perm, inverse, sizes, _ = ops.route_plan(ids.contiguous(), xchg.num_experts)
            xchg.counts_mine.copy_(sizes)
        xchg.ev_plan.record(cs)
        # activations of all groups live in shared buffers (every group writes its own rows); allocated on the compute stream
        gate, up, z, out_e = _bf16(cap, inter_dim, dev), _bf16(cap, inter_dim, dev), _bf16(cap, inter_dim, dev), _bf16(cap, xchg.hidden, dev)
        xa = xas = za = zas = gu_a_c = gu_b16 = down_a_c = down_b16 = None
        if lora:
            xa, xas, za, zas = (_bf16(cap, ops.LORA_PAD, dev) for _ in range(4))
            gu_a_c, down_a_c = gu_a.contiguous(), down_a.contiguous()
            gu_b16, down_b16 = ops.pad_rank_cols(gu_b), ops.pad_rank_cols(down_b)

        n = xchg.chunks

        def send(c):                                     # exchange stream: rows of group c to their owners
            # No wait is needed before writing the receive buffer: its last readers (the previous call's backward) were
            # enqueued before that call's final sync(), which every rank has passed to get here.
            with torch.cuda.stream(xs), _Span(xchg, "dispatch", xs):
                xchg.scatter(hidden, perm, top_k, sorted_e, c, 0)
                xchg.sync()                              # every source has delivered group c
            ev["sent"][c].record(xs)

        def bring_back(c):                               # exchange stream: results of group c back to their sources
            with torch.cuda.stream(xs):
                xs.wait_event(ev["computed"][c])
                with _Span(xchg, "return", xs):
                    xchg.give_back(out_e, c, 0)
                    xchg.sync()
            ev["returned"][c].record(xs)

        with torch.cuda.stream(xs):
            xs.wait_event(xchg.ev_plan)
            with _Span(xchg, "plan_exchange", xs):
                xchg.make_plan()
        # The exchange stream runs S0 S1 S2 R0 S3 R1 ... R(n-1): while group c computes, group c+1 (already) and c+2 arrive and
        # group c-1 goes home.  An event must be recorded (host side) before another stream is told to wait for it, hence the
        # order of the calls below.
        send(0)
        if n > 1:
            send(1)
        x = xchg.recv[0]
        tiles = []
        xchg.gemm_margin(True)
        try:
            for c, (lo, hi) in enumerate(xchg.groups):
                cs.wait_event(ev["sent"][c])
                first, end = xchg.group_first[c], xchg.group_end[c]
                with _Span(xchg, "experts_forward", cs):
                    t = ops.grouped_schedule(xchg.local_ids[lo:hi], plan.local_offsets[lo:hi], cap, first)
                    if lora:
                        ops.grouped_lora_down(x, None, gu_a_c, False, scaling, r, t, zero=False, out=(xa, xas))
                    ops.grouped_fwd(x, gate_p.reshape(-1), up_p.reshape(-1), quant_type, inter_dim, e_local, t, xas, gu_b16, out0=gate, out1=up)
                    ops.swiglu_fwd(gate, up, 0.0, first, end, out=z)
                    if lora:
                        ops.grouped_lora_down(z, None, down_a_c, False, scaling, r, t, zero=False, out=(za, zas))
                    ops.grouped_fwd(z, down_p.reshape(-1), None, quant_type, xchg.hidden, e_local, t, zas, down_b16, out0=out_e)
                ev["computed"][c].record(cs)
                tiles.append(t)
                if c + 2 < n:
                    send(c + 2)
                bring_back(c)
        finally:
            xchg.gemm_margin(False)

        cs.wait_event(ev["returned"][-1])                 # the exchange stream is in order: the last group's return is the last
        returned = xchg.ret[0][:rows]
        with _Span(xchg, "combine", cs):
            out = ops.route_combine(returned, weights, inverse)
        # `out_e` was read by the exchange stream; the compute stream has waited for the last of those reads, so the allocator may
        # hand its memory to later work of the compute stream
        ctx.xchg, ctx.geometry, ctx.lora = xchg, (tokens, top_k, int(quant_type), int(inter_dim), float(scaling), r), lora
        ctx.saved = (sorted_e, perm, inverse, weights, returned, tiles, gate, up, z, xa, za, gate_p, up_p, down_p, gu_a_c, gu_b, down_a_c, down_b)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        xchg, lora = ctx.xchg, ctx.lora
        tokens, top_k, quant_type, inter_dim, scaling, r = ctx.geometry
        sorted_e, perm, inverse, weights, returned, tiles, gate, up, z, xa, za, gate_p, up_p, down_p, gu_a, gu_b, down_a, down_b = ctx.saved
        dev = grad_out.device
        cs, xs, ev = torch.cuda.current_stream(dev), xchg.stream, xchg.events
        e_local, cap, plan, hid = xchg.experts_per_rank, xchg.capacity, xchg.plan, xchg.hidden
        with _Span(xchg, "combine_backward", cs):
            d_rows, d_weights = ops.route_combine_bwd(returned, weights, perm, grad_out.contiguous())
        xchg.ev_ready.record(cs)
        dz, d_gate, d_up, d_sel = _bf16(cap, inter_dim, dev), _bf16(cap, inter_dim, dev), _bf16(cap, inter_dim, dev), _bf16(cap, hid, dev)
        dob = dobs = dgb = dgbs = down_bt = gu_bt = down_a16 = gu_a16 = None
        grads = [None, None, None, None]
        if lora:
            dob, dobs, dgb, dgbs = (_bf16(cap, ops.LORA_PAD, dev) for _ in range(4))
            down_bt, gu_bt = down_b.transpose(1, 2).contiguous(), gu_b.transpose(1, 2).contiguous()
            down_a16, gu_a16 = ops.pad_rank_rows(down_a), ops.pad_rank_rows(gu_a)
            grads = [torch.empty_like(gu_a), torch.empty_like(gu_b), torch.empty_like(down_a), torch.empty_like(down_b)]

        n = xchg.chunks

        def send(c):
            with torch.cuda.stream(xs), _Span(xchg, "dispatch_backward", xs):
                xchg.scatter(d_rows, None, 1, sorted_e, c, 1)
                xchg.sync()
            ev["g_sent"][c].record(xs)

        def bring_back(c):
            with torch.cuda.stream(xs):
                xs.wait_event(ev["g_computed"][c])
                with _Span(xchg, "return_backward", xs):
                    xchg.give_back(d_sel, c, 1)
                    xchg.sync()
            ev["g_returned"][c].record(xs)

        xs.wait_event(xchg.ev_ready)
        send(0)
        if n > 1:
            send(1)
        x, d_out = xchg.recv[0], xchg.recv[1]
        xchg.gemm_margin(True)
        try:
            for c, (lo, hi) in enumerate(xchg.groups):
                cs.wait_event(ev["g_sent"][c])
                first, end, t, offs = xchg.group_first[c], xchg.group_end[c], tiles[c], plan.local_offsets[lo:hi]
                with _Span(xchg, "experts_backward", cs):
                    if lora:
                        # down projection: dZ = dOut.deq(Wd) + s.(dOut.Bd).Ad ; dAd = s.(dOut.Bd)^T.Z ; dBd = s.dOut^T.(Z.Ad^T)
                        ops.grouped_lora_down(d_out, None, down_bt, False, scaling, r, t, zero=False, out=(dob, dobs))
                    ops.grouped_dgrad(d_out, None, down_p.reshape(-1), None, quant_type, inter_dim, e_local, t, dobs, down_a16, out=dz)
                    if lora:
                        ops.grouped_lora_wgrad(dob, z, scaling, r, offs, grads[2][lo:hi], False, 0, first)
                        ops.grouped_lora_wgrad(za, d_out, scaling, r, offs, grads[3][lo:hi], True, 0, first)
                    ops.swiglu_bwd(gate, up, dz, 0.0, first, end, out=(d_gate, d_up))
                    if lora:
                        # gate|up: dX = dG.deq(Wg) + dU.deq(Wu) + s.([dG|dU].Bgu).Agu
                        ops.grouped_lora_down(d_gate, d_up, gu_bt, False, scaling, r, t, zero=False, out=(dgb, dgbs))
                    ops.grouped_dgrad(d_gate, d_up, gate_p.reshape(-1), up_p.reshape(-1), quant_type, hid, e_local, t, dgbs, gu_a16, out=d_sel)
                    if lora:
                        ops.grouped_lora_wgrad(dgb, x, scaling, r, offs, grads[0][lo:hi], False, 0, first)
                        ops.grouped_lora_wgrad(xa, d_gate, scaling, r, offs, grads[1][lo:hi], True, 0, first)
                        ops.grouped_lora_wgrad(xa, d_up, scaling, r, offs, grads[1][lo:hi], True, inter_dim, first)
                ev["g_computed"][c].record(cs)
                if c + 2 < n:
                    send(c + 2)
                bring_back(c)
        finally:
            xchg.gemm_margin(False)

        cs.wait_event(ev["g_returned"][-1])
        with _Span(xchg, "gather_backward", cs):
            d_hidden = ops.route_gather_bwd(xchg.ret[1][:tokens * top_k], inverse, tokens, top_k)
        ctx.saved = None
        return (None, d_hidden, None, d_weights, None, None, None, None, None, None, *grads)


def peer_moe_layer(xchg: PeerExchange, hidden: torch.Tensor, top_k_index: torch.Tensor, top_k_weights: torch.Tensor,
                   gate_payload: torch.Tensor, up_payload: torch.Tensor, down_payload: torch.Tensor, quant_type: int, inter_dim: int,
                   lora: Optional[dict] = None, scaling: float = 1.0) -> torch.Tensor:
    """Expert-parallel layer; payloads / LoRA factors hold this rank's experts only (in the order of the exchange's placement),
    ``top_k_index`` carries the router's global ids."""
    lo = lora or {}
    return _PeerMoe.apply(xchg, hidden, top_k_index, top_k_weights, gate_payload, up_payload, down_payload, int(quant_type), int(inter_dim),
                          float(scaling), lo.get("gate_up_a"), lo.get("gate_up_b"), lo.get("down_a"), lo.get("down_b"))
