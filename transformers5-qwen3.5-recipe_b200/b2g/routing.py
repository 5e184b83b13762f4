"""Routing plan and the two permute autograd functions (token gather, weighted combine).

Restates the behaviour of the reference's ``fast_moe_routing.py`` (``prepare_expert_routing`` :379-428,
``_RouteGather`` :229-285, ``_RouteCombine`` :288-347) on top of the libb2g kernels: a stable
counting sort replaces ``torch.sort`` + the inverse-permutation kernel, and the same pass produces
the expert histogram (group sizes and cumulative offsets) that the grouped products consume.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from . import ops


@dataclass(frozen=True)
class ExpertRoutingPlan:
    selected_hidden_states: torch.Tensor
    expert_indices: torch.Tensor          # sorted flat expert ids [R]
    routing_weights: torch.Tensor
    permutation: torch.Tensor
    inverse_permutation: torch.Tensor
    num_tokens: int
    num_top_k: int
    hidden_dim: int
    # produced by the same sort; the reference gets these from GGUFExperts._prepare_expert_execution
    group_sizes: Optional[torch.Tensor] = None    # int32 [E]
    group_offsets: Optional[torch.Tensor] = None  # int32 [E], cumulative ends


class _RouteGather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden_states, permutation, inverse_permutation):
        num_tokens = hidden_states.shape[0]
        top_k = permutation.numel() // num_tokens
        ctx.save_for_backward(inverse_permutation)
        ctx.geometry = (num_tokens, top_k)
        return ops.route_gather(hidden_states, permutation, top_k)

    @staticmethod
    def backward(ctx, grad_selected):
        if not ctx.needs_input_grad[0]:
            return None, None, None
        (inverse_permutation,) = ctx.saved_tensors
        num_tokens, top_k = ctx.geometry
        return ops.route_gather_bwd(grad_selected.contiguous(), inverse_permutation, num_tokens, top_k), None, None


class _RouteCombine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, expert_output, routing_weights, permutation, inverse_permutation):
        ctx.save_for_backward(expert_output, routing_weights, permutation)
        return ops.route_combine(expert_output, routing_weights, inverse_permutation)

    @staticmethod
    def backward(ctx, grad_final):
        expert_output, routing_weights, permutation = ctx.saved_tensors
        d_out, d_w = ops.route_combine_bwd(expert_output, routing_weights, permutation, grad_final.contiguous())
        return (d_out if ctx.needs_input_grad[0] else None, d_w if ctx.needs_input_grad[1] else None, None, None)


def build_plan(hidden_states: torch.Tensor, top_k_index: torch.Tensor, top_k_weights: torch.Tensor,
               num_experts: int = 256) -> ExpertRoutingPlan:
    num_tokens, hidden_dim = hidden_states.shape
    top_k = top_k_index.shape[1]
    sorted_e, perm, inv, sizes, offsets = ops.route_plan(top_k_index.contiguous(), num_experts)
    selected = _RouteGather.apply(hidden_states, perm, inv)
    return ExpertRoutingPlan(selected_hidden_states=selected, expert_indices=sorted_e, routing_weights=top_k_weights.contiguous(),
                             permutation=perm, inverse_permutation=inv, num_tokens=num_tokens, num_top_k=top_k,
                             hidden_dim=hidden_dim, group_sizes=sizes, group_offsets=offsets)


def combine(output: torch.Tensor, plan: ExpertRoutingPlan) -> torch.Tensor:
    return _RouteCombine.apply(output, plan.routing_weights, plan.permutation, plan.inverse_permutation)
