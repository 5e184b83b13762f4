"""Expert-parallel execution of the grouped MoE path over one process per GPU.

The reference runs the whole model on one device and states that expert parallelism is
unsupported (``docs/plan_qwen3.5.md:23``); this module is therefore new design, not a restatement.
Experts shard naturally: rank ``g`` of ``G`` owns the contiguous block of ``E/G`` experts
``[g*E/G, (g+1)*E/G)`` (packed payloads and LoRA factors of other experts are never needed), and
tokens stay data-parallel.  Per layer and direction there is exactly one exchange each way:

    local top-k  ->  stable sort by global expert id (rows come out grouped by destination rank,
    then expert)  ->  per-(rank, expert) row counts exchanged (one small all-to-all)  ->
    DISPATCH all-to-all of the routed rows  ->  regroup by local expert  ->  grouped expert block
    on the owner  ->  inverse regroup  ->  COMBINE all-to-all back  ->  weighted un-permute.

Backward mirrors it through the two autograd functions below; factor gradients stay on the
expert's owner (every expert has exactly one), so no all-reduce is needed.

The index logic (split sizes, regroup permutation) is plain integer tensor code that runs on any
device, which is how the multi-rank behaviour is tested on CPU ranks with gloo; the row payload
always moves with ``torch.distributed.all_to_all_single`` (NCCL over NVLink on the GPU box).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.distributed as dist


@dataclass
class ExpertParallelPlan:
    send_splits: list[int]            # rows this rank sends to each rank (dispatch direction)
    recv_splits: list[int]            # rows this rank receives from each rank
    regroup: torch.Tensor             # int64 [R_recv]: received order (source rank, expert) -> (expert, source rank)
    regroup_inverse: torch.Tensor     # int64 [R_recv]
    local_sizes: torch.Tensor         # int32 [E/G] rows per local expert
    local_offsets: torch.Tensor       # int32 [E/G] cumulative ends
    experts_per_rank: int


def expert_owner_ranges(num_experts: int, world: int) -> list[tuple[int, int]]:
    if num_experts % world:
        raise ValueError(f"{num_experts} experts do not divide over {world} ranks")
    per = num_experts // world
    return [(g * per, (g + 1) * per) for g in range(world)]


def regroup_permutation(recv_counts: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """recv_counts [G, E_local]: rows received from source rank g for local expert e, laid out in
    (g, e) order.  Returns the gather index that reorders them to (e, g) order, and its inverse."""
    g, e = recv_counts.shape
    counts = recv_counts.to(torch.int64)
    starts_ge = (torch.cumsum(counts.reshape(-1), 0) - counts.reshape(-1)).reshape(g, e)   # where block (g,e) starts on arrival
    counts_eg = counts.t().contiguous().reshape(-1)                                        # block sizes in (e,g) order
    starts_eg = starts_ge.t().contiguous().reshape(-1)
    total = int(counts.sum())
    block_of_row = torch.repeat_interleave(torch.arange(g * e, device=counts.device), counts_eg, output_size=total)
    first_of_block = torch.cumsum(counts_eg, 0) - counts_eg
    within = torch.arange(total, device=counts.device) - first_of_block[block_of_row]
    perm = starts_eg[block_of_row] + within
    inverse = torch.empty_like(perm)
    inverse[perm] = torch.arange(total, device=counts.device)
    return perm, inverse


def build_plan(group_sizes: torch.Tensor, group: Optional[dist.ProcessGroup] = None) -> ExpertParallelPlan:
    """From this rank's histogram over ALL experts (int32 [E]) to the exchange plan.
    One small all-to-all of counts and one device-to-host read of the split sizes."""
    world = dist.get_world_size(group)
    e_total = group_sizes.numel()
    per = e_total // world
    if per * world != e_total:
        raise ValueError(f"{e_total} experts do not divide over {world} ranks")
    send_counts = group_sizes.reshape(world, per).contiguous()
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts, group=group)
    both = torch.stack([send_counts.sum(1), recv_counts.sum(1)]).cpu()          # the one host read of the layer
    send_splits, recv_splits = both[0].tolist(), both[1].tolist()
    if min(send_splits + recv_splits) < 0:
        raise RuntimeError("negative split size in the expert-parallel plan")
    regroup, inverse = regroup_permutation(recv_counts)
    local_sizes = recv_counts.sum(0).to(torch.int32)
    local_offsets = torch.cumsum(local_sizes, 0).to(torch.int32)
    return ExpertParallelPlan(send_splits, recv_splits, regroup, inverse, local_sizes, local_offsets, per)


class _AllToAllRows(torch.autograd.Function):
    """Row exchange with per-rank split sizes; the backward is the same exchange with the splits swapped."""

    @staticmethod
    def forward(ctx, rows, send_splits, recv_splits, group):
        ctx.splits = (send_splits, recv_splits)
        ctx.group = group
        out = rows.new_empty((sum(recv_splits),) + tuple(rows.shape[1:]))
        dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=recv_splits, input_split_sizes=send_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, grad):
        send_splits, recv_splits = ctx.splits
        out = grad.new_empty((sum(send_splits),) + tuple(grad.shape[1:]))
        dist.all_to_all_single(out, grad.contiguous(), output_split_sizes=send_splits, input_split_sizes=recv_splits, group=ctx.group)
        return out, None, None, None


class _PermuteRows(torch.autograd.Function):
    """y = x[index]; ``index`` is a permutation, so the backward is the inverse gather (no scatter-add)."""

    @staticmethod
    def forward(ctx, x, index, inverse):
        ctx.save_for_backward(index, inverse)
        return x.index_select(0, index)

    @staticmethod
    def backward(ctx, grad):
        _, inverse = ctx.saved_tensors
        return grad.index_select(0, inverse), None, None


def dispatch(selected_rows: torch.Tensor, plan: ExpertParallelPlan, group=None) -> torch.Tensor:
    """Rows sorted by global expert id -> rows of this rank's experts, grouped by local expert."""
    arrived = _AllToAllRows.apply(selected_rows, plan.send_splits, plan.recv_splits, group)
    return _PermuteRows.apply(arrived, plan.regroup, plan.regroup_inverse)


def combine(expert_rows: torch.Tensor, plan: ExpertParallelPlan, group=None) -> torch.Tensor:
    """Inverse of ``dispatch``: expert outputs back to the rank, in its sorted-by-expert order."""
    back = _PermuteRows.apply(expert_rows, plan.regroup_inverse, plan.regroup)
    return _AllToAllRows.apply(back, plan.recv_splits, plan.send_splits, group)


ExpertFn = Callable[[torch.Tensor, torch.Tensor, torch.Tensor], torch.Tensor]


def expert_parallel_moe(hidden: torch.Tensor, top_k_index: torch.Tensor, top_k_weights: torch.Tensor, expert_fn: ExpertFn,
                        num_experts: int, route_plan_fn, gather_fn, combine_fn, group=None, always_exchange: bool = False) -> torch.Tensor:
    """One expert-parallel MoE layer.

    ``route_plan_fn(top_k_index, num_experts)`` -> (perm, inverse, group_sizes) of the stable sort;
    ``gather_fn(hidden, perm, inverse)`` / ``combine_fn(rows, weights, perm, inverse)`` are the token
    permute and weighted un-permute; ``expert_fn(rows, local_sizes, local_offsets)`` computes the
    outputs of this rank's experts for rows grouped by local expert.  All are differentiable.
    """
    perm, inverse, group_sizes = route_plan_fn(top_k_index, num_experts)
    selected = gather_fn(hidden, perm, inverse)
    if dist.get_world_size(group) == 1 and not always_exchange:
        # one rank owns every expert: rows are already grouped by expert, nothing to exchange
        sizes = group_sizes.to(torch.int32)
        local_out = expert_fn(selected, sizes, torch.cumsum(sizes, 0).to(torch.int32))
        return combine_fn(local_out, top_k_weights, perm, inverse)
    plan = build_plan(group_sizes, group)
    local_rows = dispatch(selected, plan, group)
    local_out = expert_fn(local_rows, plan.local_sizes, plan.local_offsets)
    returned = combine(local_out, plan, group)
    return combine_fn(returned, top_k_weights, perm, inverse)


# ---- the CUDA instantiation ------------------------------------------------------------------------
def cuda_moe_layer(hidden: torch.Tensor, top_k_index: torch.Tensor, top_k_weights: torch.Tensor, gate_payload: torch.Tensor,
                   up_payload: torch.Tensor, down_payload: torch.Tensor, quant_type: int, inter_dim: int, num_experts: int,
                   lora: Optional[dict] = None, scaling: float = 1.0, group=None, always_exchange: bool = False) -> torch.Tensor:
    """Expert-parallel layer on the libb2g kernels.  Payloads / LoRA factors hold only THIS rank's experts
    ([E/G, ...]); ``top_k_index`` carries global expert ids."""
    from . import autograd as ag
    from . import ops, routing

    def route_plan_fn(idx, e):
        _, perm, inverse, sizes, _ = ops.route_plan(idx.contiguous(), e)
        return perm, inverse, sizes

    def gather_fn(h, perm, inverse):
        return routing._RouteGather.apply(h, perm, inverse)

    def combine_fn(rows, weights, perm, inverse):
        return routing._RouteCombine.apply(rows.contiguous(), weights.contiguous(), perm, inverse)

    def expert_fn(rows, local_sizes, local_offsets):
        idx = torch.arange(local_sizes.numel(), device=rows.device, dtype=torch.int64)
        lo = lora or {}
        return ag.grouped_lora_experts(rows.contiguous(), gate_payload, up_payload, down_payload, quant_type, quant_type, inter_dim,
                                       idx, local_offsets, local_offsets, lo.get("gate_up_a"), lo.get("gate_up_b"),
                                       lo.get("down_a"), lo.get("down_b"), scaling, 0.0)

    return expert_parallel_moe(hidden, top_k_index, top_k_weights, expert_fn, num_experts, route_plan_fn, gather_fn, combine_fn, group,
                               always_exchange)
