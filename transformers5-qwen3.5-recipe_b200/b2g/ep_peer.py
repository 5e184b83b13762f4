"""Expert-parallel MoE layer with the row exchange done by peer stores over NVLink.

Instead of gather -> NCCL all-to-all -> regroup (``b2g/ep.py``), the token permute and the transfer are one
kernel: every routed row is read from the token matrix on its source rank and written straight into the owner
rank's receive buffer, already grouped by (local expert, source rank); the way back is the mirror image.  The
slots follow from the all-gathered per-rank expert histograms, computed by one small kernel on the device
(``build_peer_plan_device``; ``build_peer_plan`` is the same arithmetic as tensor ops, kept as the checkable
statement of it), so no split size is read on the host and nothing is regrouped afterwards.  Every rank starts
its scatter at a different owner's experts, so that the ranks do not all store to one GPU at a time.

Buffers are symmetric allocations (one per rank, same size, mapped into every rank): two receive buffers of
``capacity`` rows (activations forward, output gradients backward) and two return buffers of the rank's own
routed-row count.  A layer object owns them; its outputs alias them until the next call of the same layer.
Ranks synchronise on the stream after each exchange with a one-element NCCL all-reduce (no device-side spin
loops of our own); multicast is not used.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist

from . import _lib, ops, routing


@dataclass
class PeerPlan:
    my_start: torch.Tensor       # int32 [E]   first sorted position of expert e on this rank
    dest_base: torch.Tensor      # int32 [E]   slot at the owner where this rank's rows of expert e start
    blk_start: torch.Tensor      # int32 [E_l*G + 1] owner side: start of block (local expert, source rank)
    src_pos: torch.Tensor        # int32 [E_l*G]     position of that block's first row in the source's sorted order
    local_sizes: torch.Tensor    # int32 [E_l]
    local_offsets: torch.Tensor  # int32 [E_l]


def build_peer_plan(counts: torch.Tensor, rank: int) -> PeerPlan:
    """counts: int32/int64 [G, E], row g = histogram of rank g's routed rows over all experts."""
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
    local_sizes = total[lo:hi]
    i32 = torch.int32
    return PeerPlan(my_start=my_start_all[rank].to(i32).contiguous(), dest_base=(owner_prefix + src_prefix[rank]).to(i32).contiguous(),
                    blk_start=blk_start.to(i32).contiguous(), src_pos=my_start_all[:, lo:hi].t().contiguous().reshape(-1).to(i32),
                    local_sizes=local_sizes.to(i32).contiguous(), local_offsets=local_sizes.cumsum(0).to(i32).contiguous())


def build_peer_plan_device(counts: torch.Tensor, rank: int) -> PeerPlan:
    """The same plan as :func:`build_peer_plan` in one kernel launch (``counts``: int32 [G, E] on the GPU)."""
    g, e = counts.shape
    per = e // g
    dev = counts.device
    buf = torch.empty(2 * e + (per * g + 1) + per * g + 2 * per, dtype=torch.int32, device=dev)
    my_start, dest_base, blk_start, src_pos, local_sizes, local_offsets = torch.split(buf, [e, e, per * g + 1, per * g, per, per])
    with torch.cuda.device(dev):
        _lib.call("b2g_ep_peer_plan", C.c_void_p(counts.data_ptr()), g, e, int(rank), *(C.c_void_p(t.data_ptr()) for t in
                  (my_start, dest_base, blk_start, src_pos, local_sizes, local_offsets)), C.c_void_p(torch.cuda.current_stream().cuda_stream))
    return PeerPlan(my_start, dest_base, blk_start, src_pos, local_sizes, local_offsets)


class PeerExchange:
    """Symmetric receive / return buffers of one MoE layer and the two exchange kernels."""

    def __init__(self, rows_local: int, hidden: int, num_experts: int, group=None, capacity_factor: float = 1.5,
                 device: Optional[torch.device] = None):
        import torch.distributed._symmetric_memory as symm

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.rows_local, self.hidden, self.num_experts = rows_local, hidden, num_experts
        self.experts_per_rank = num_experts // self.world
        cap = rows_local if self.world == 1 else int(rows_local * capacity_factor)
        self.capacity = (cap + 511) // 512 * 512
        self.recv, self.ret, self._recv_ptrs, self._ret_ptrs = [], [], [], []
        for _ in range(2):
            for store, ptrs, rows in ((self.recv, self._recv_ptrs, self.capacity), (self.ret, self._ret_ptrs, rows_local)):
                t = symm.empty((rows, hidden), dtype=torch.bfloat16, device=self.device)
                h = symm.rendezvous(t, self.group)
                store.append(t)
                ptrs.append(torch.tensor([int(p) for p in h.buffer_ptrs], dtype=torch.int64, device=self.device))
        self._flag = torch.zeros(1, dtype=torch.int32, device=self.device)

    def sync(self) -> None:
        """All ranks' earlier work on their streams is complete before any rank continues."""
        dist.all_reduce(self._flag, group=self.group)

    def gather_counts(self, group_sizes: torch.Tensor) -> torch.Tensor:
        counts = torch.empty(self.world, self.num_experts, dtype=torch.int32, device=self.device)
        dist.all_gather_into_tensor(counts, group_sizes.to(torch.int32).contiguous(), group=self.group)
        return counts

    def scatter(self, src: torch.Tensor, perm: Optional[torch.Tensor], top_k: int, sorted_expert: torch.Tensor, plan: PeerPlan, which: int):
        rows = sorted_expert.numel()
        # No synchronisation is needed before writing: the last reads of this receive buffer (expert forward / backward of
        # the previous call) were enqueued before that call's final sync(), which every rank has passed to get here.
        with torch.cuda.device(self.device):
            _lib.call("b2g_ep_scatter_rows", C.c_void_p(src.data_ptr()), None if perm is None else C.c_void_p(perm.data_ptr()), int(top_k),
                      C.c_void_p(sorted_expert.data_ptr()), C.c_void_p(plan.my_start.data_ptr()), C.c_void_p(plan.dest_base.data_ptr()),
                      C.c_void_p(self._recv_ptrs[which].data_ptr()), self.experts_per_rank, rows, self.hidden, self.capacity,
                      ((self.rank + 1) % self.world) * self.experts_per_rank,      # start with the next rank's experts
                      C.c_void_p(ops.status_word(self.device).data_ptr()), C.c_void_p(torch.cuda.current_stream().cuda_stream))
        self.sync()          # every source has delivered
        return self.recv[which]

    def give_back(self, rows: torch.Tensor, plan: PeerPlan, which: int):
        # Same argument as in scatter(): every earlier read of the return buffers is separated from this write by at
        # least one sync() that both ranks took part in.
        with torch.cuda.device(self.device):
            _lib.call("b2g_ep_return_rows", C.c_void_p(rows.data_ptr()), C.c_void_p(plan.blk_start.data_ptr()), C.c_void_p(plan.src_pos.data_ptr()),
                      C.c_void_p(self._ret_ptrs[which].data_ptr()), self.world, self.experts_per_rank * self.world, self.hidden, self.capacity,
                      C.c_void_p(torch.cuda.current_stream().cuda_stream))
        self.sync()
        return self.ret[which]


class _PeerDispatch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, perm, inverse, sorted_expert, plan, xchg, top_k):
        ctx.plan, ctx.xchg, ctx.geometry = plan, xchg, (hidden.shape[0], top_k)
        ctx.save_for_backward(inverse)
        return xchg.scatter(hidden, perm, top_k, sorted_expert, plan, 0)

    @staticmethod
    def backward(ctx, grad_rows):
        (inverse,) = ctx.saved_tensors
        tokens, top_k = ctx.geometry
        back = ctx.xchg.give_back(grad_rows.contiguous(), ctx.plan, 1)
        return ops.route_gather_bwd(back, inverse, tokens, top_k), None, None, None, None, None, None


class _PeerReturn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, expert_rows, sorted_expert, plan, xchg):
        ctx.plan, ctx.xchg = plan, xchg
        ctx.save_for_backward(sorted_expert)
        return xchg.give_back(expert_rows.contiguous(), plan, 0)

    @staticmethod
    def backward(ctx, grad_sorted):
        (sorted_expert,) = ctx.saved_tensors
        return ctx.xchg.scatter(grad_sorted.contiguous(), None, 1, sorted_expert, ctx.plan, 1), None, None, None


def peer_moe_layer(xchg: PeerExchange, hidden: torch.Tensor, top_k_index: torch.Tensor, top_k_weights: torch.Tensor,
                   gate_payload: torch.Tensor, up_payload: torch.Tensor, down_payload: torch.Tensor, quant_type: int, inter_dim: int,
                   lora: Optional[dict] = None, scaling: float = 1.0) -> torch.Tensor:
    """Expert-parallel layer; payloads / LoRA factors hold this rank's experts only, indices are global ids."""
    from . import autograd as ag

    top_k = top_k_index.shape[1]
    sorted_e, perm, inverse, sizes, _ = ops.route_plan(top_k_index.contiguous(), xchg.num_experts)
    plan = build_peer_plan_device(xchg.gather_counts(sizes), xchg.rank)
    local_rows = _PeerDispatch.apply(hidden, perm, inverse, sorted_e, plan, xchg, top_k)
    idx = torch.arange(xchg.experts_per_rank, device=hidden.device, dtype=torch.int64)
    lo = lora or {}
    local_out = ag.grouped_lora_experts(local_rows, gate_payload, up_payload, down_payload, quant_type, quant_type, inter_dim, idx,
                                        plan.local_offsets, plan.local_offsets, lo.get("gate_up_a"), lo.get("gate_up_b"),
                                        lo.get("down_a"), lo.get("down_b"), scaling, 0.0)
    returned = _PeerReturn.apply(local_out, sorted_e, plan, xchg)
    return routing._RouteCombine.apply(returned, top_k_weights.contiguous(), perm, inverse)
