"""Token permute / un-permute for the MoE expert path (B200 build).

Public surface of the reference module of this name: ``ExpertRoutingPlan``,
``prepare_expert_routing``, ``finalize_expert_routing``, the geometry allow-list and the launch
helpers its tests import.  The sort is a stable counting sort on the device (one pass also yields
the expert histogram), the permutes are 16-byte-vector streaming kernels; see ``b2g/routing.py``.
"""
from __future__ import annotations

import torch

from b2g.routing import ExpertRoutingPlan, _RouteCombine, _RouteGather, build_plan  # noqa: F401

# (top_k, hidden) pairs of the production models plus the two small regression geometries.
_SUPPORTED_ROUTING_GEOMETRIES = frozenset({(8, 2048), (6, 4096), (4, 2048), (1, 256)})
# The reference stops at 16 x 2048 tokens; one B200 also runs the 65,536-token expert-parallel
# baseline point, so the cap is raised once and stays fail-closed beyond it.
_MAX_TOKENS = 32 * 2048


def _is_supported_routing_geometry(num_tokens: int, num_top_k: int, hidden_dim: int) -> bool:
    return 0 < num_tokens <= _MAX_TOKENS and (num_top_k, hidden_dim) in _SUPPORTED_ROUTING_GEOMETRIES


def _routing_gather_forward_launch(num_tokens: int, top_k: int, hidden_dim: int) -> tuple[int, int]:
    """(columns per block, warps) of the gather kernel: one 256-thread block moves a whole row."""
    del num_tokens, top_k
    return hidden_dim, 8


def _routing_combine_forward_launch(num_tokens: int, top_k: int, hidden_dim: int) -> tuple[int, int]:
    del num_tokens, top_k
    return hidden_dim, 8


def _routing_launch_warps(num_tokens: int, num_top_k: int = 8, hidden_dim: int = 2048) -> tuple[int, int]:
    del num_tokens, num_top_k, hidden_dim
    return 8, 8


def _validate_optimized_routing(hidden_states: torch.Tensor, top_k_index: torch.Tensor, top_k_weights: torch.Tensor) -> None:
    num_tokens, hidden_dim = hidden_states.shape
    if not _is_supported_routing_geometry(num_tokens, top_k_index.shape[1], hidden_dim):
        raise RuntimeError("Unsupported optimized expert-routing geometry. Production requires Qwen top-8/hidden-2048 or "
                           f"DeepSeek top-6/hidden-4096 with at most {_MAX_TOKENS:,} tokens.")
    if hidden_states.device.type != "cuda":
        raise RuntimeError("Optimized expert routing requires CUDA tensors.")
    if hidden_states.dtype != torch.bfloat16 or not hidden_states.is_contiguous():
        raise RuntimeError("Optimized expert routing requires contiguous BF16 hidden states.")
    if top_k_index.device != hidden_states.device:
        raise RuntimeError("Expert indices must be on the hidden-state device.")
    if top_k_weights.device != hidden_states.device:
        raise RuntimeError("Routing weights must be on the hidden-state device.")
    if top_k_index.dtype not in (torch.int32, torch.int64):
        raise RuntimeError("Expert indices must use int32 or int64.")
    if top_k_weights.dtype not in (torch.bfloat16, torch.float32):
        raise RuntimeError("Routing weights must use BF16 or FP32.")


def prepare_expert_routing(hidden_states: torch.Tensor, top_k_index: torch.Tensor, top_k_weights: torch.Tensor,
                           num_experts: int = 256) -> ExpertRoutingPlan:
    if hidden_states.ndim != 2:
        raise ValueError(f"Expert routing expects hidden states [tokens, hidden], got {hidden_states.shape}.")
    if top_k_index.ndim != 2 or top_k_weights.shape != top_k_index.shape:
        raise ValueError("Expert routing expects matching top-k index and weight matrices.")
    if top_k_index.shape[0] != hidden_states.shape[0]:
        raise ValueError("Expert routing token count does not match the hidden-state token count.")
    _validate_optimized_routing(hidden_states, top_k_index, top_k_weights.contiguous())
    return build_plan(hidden_states, top_k_index, top_k_weights, num_experts)


def finalize_expert_routing(output: torch.Tensor, hidden_states: torch.Tensor, routing_plan: ExpertRoutingPlan,
                            output_mask: torch.Tensor | None) -> torch.Tensor:
    if output_mask is not None:
        raise RuntimeError("Optimized expert routing does not support output masks.")
    expected = (routing_plan.num_tokens * routing_plan.num_top_k, routing_plan.hidden_dim)
    if output.device.type != "cuda" or output.dtype != torch.bfloat16 or not output.is_contiguous() or tuple(output.shape) != expected:
        raise RuntimeError(f"Optimized expert combine requires contiguous CUDA BF16 output with shape {expected}, "
                           f"got {tuple(output.shape)}.")
    result = _RouteCombine.apply(output, routing_plan.routing_weights, routing_plan.permutation, routing_plan.inverse_permutation)
    return result.to(hidden_states.dtype)
