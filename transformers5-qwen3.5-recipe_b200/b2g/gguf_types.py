"""GGUF tensor / module types the reference takes from an un-vendored transformers fork.

When that fork is installed (``transformers.integrations.gguf`` with ``GGUFLinear`` etc.) its own
classes are re-exported unchanged, so models loaded by it work directly.  Otherwise the small
stand-ins below provide exactly the attributes and hooks the hot path consumes
(``fast_lora.py:137-162``, ``fast_moe_lora.py:536-545,698-769``): packed payload tensors that carry
``quant_type`` and ``logical_shape``, a packed linear, and a packed expert bank with the
``_prepare_expert_*`` / ``_apply_split_gate`` hooks and the implementation registry.
"""
from __future__ import annotations

from dataclasses import dataclass
from types import SimpleNamespace
from typing import Any, Callable, Optional

import torch

from . import autograd as ag
from . import ops

try:  # the fork, when present
    from transformers.integrations.gguf import (ALL_GGUF_EXPERTS_FUNCTIONS, DeepseekV4GGUFExperts, GGUFExperts,  # type: ignore
                                                GGUFGroupedLinear, GGUFLinear)
    from transformers.integrations.gguf_dequant import GGUFQuantizedTensor, dequantize_gguf_tensor  # type: ignore

    HAVE_FORK = True
except Exception:  # stock transformers, or none
    HAVE_FORK = False

    class GGUFQuantizedTensor(torch.Tensor):
        """uint8 payload in GGUF block layout plus its type id and logical shape."""

        @staticmethod
        def __new__(cls, payload: torch.Tensor, quant_type: int = 0, logical_shape: tuple[int, ...] = ()):
            t = torch.Tensor._make_subclass(cls, payload, False)
            t.quant_type = int(quant_type)
            t.logical_shape = tuple(int(v) for v in logical_shape)
            return t

        def __init__(self, *args: Any, **kwargs: Any) -> None:
            super().__init__()

        @classmethod
        def __torch_function__(cls, func, types, args=(), kwargs=None):
            with torch._C.DisableTorchFunctionSubclass():
                return func(*args, **(kwargs or {}))

    def dequantize_gguf_tensor(payload: torch.Tensor, quant_type: int, dtype: torch.dtype = torch.bfloat16,
                               device: Optional[torch.device] = None) -> torch.Tensor:
        """Logical weight of a packed payload [..., rows, row_bytes] (native types only)."""
        qt = int(quant_type)
        blk, nbytes = ops._BLOCK[qt]
        k = payload.shape[-1] // nbytes * blk
        src = payload.as_subclass(torch.Tensor) if isinstance(payload, GGUFQuantizedTensor) else payload
        if device is not None:
            src = src.to(device)
        out = ops.dequantize(src.contiguous(), qt, (*payload.shape[:-1], k))
        return out.to(dtype)

    class GGUFLinear(torch.nn.Module):
        """Frozen packed linear: ``weight`` is a GGUFQuantizedTensor of logical shape [out, in]."""

        def __init__(self, in_features: int, out_features: int, bias: bool = False, device=None, dtype=None,
                     compute_dtype: torch.dtype = torch.bfloat16) -> None:
            super().__init__()
            self.in_features, self.out_features = in_features, out_features
            self.compute_dtype = compute_dtype
            self.weight: Any = None
            self.bias = torch.nn.Parameter(torch.zeros(out_features, device=device, dtype=compute_dtype)) if bias else None
            self.input_permutation = None
            self.output_permutation = None

        def forward(self, x: torch.Tensor) -> torch.Tensor:
            # a module takes strided activations like nn.Linear does (e.g. the kept positions ``hidden[:, -1:, :]``); the
            # operator underneath does not, so the one copy is made here, where it is visible
            w = self.weight
            x = x.to(self.compute_dtype)
            y = ag.mmq(x if x.is_contiguous() else x.contiguous(), w.as_subclass(torch.Tensor), int(w.quant_type), self.out_features)
            return y if self.bias is None else y + self.bias.to(y.dtype)

    class GGUFGroupedLinear(torch.nn.Module):
        """Frozen packed projection in ``n_groups`` independent groups: ``[..., n_groups, in_features]`` ->
        ``[..., n_groups, out_features / n_groups]``; ``weight`` is a GGUFQuantizedTensor holding the groups' rows one
        after the other (``[out_features, row bytes]``).  The stock forward materialises every group's logical weight;
        ``deepseek_v4_lora.configure_deepseek_v4_grouped_mmq`` replaces it with the native fixed-group product."""

        def __init__(self, in_features: int, out_features: int, n_groups: int, device=None, dtype=None,
                     compute_dtype: torch.dtype = torch.bfloat16) -> None:
            super().__init__()
            if out_features % n_groups:
                raise ValueError(f"{out_features} output features do not divide into {n_groups} groups")
            self.in_features, self.out_features, self.n_groups = in_features, out_features, n_groups
            self.compute_dtype = compute_dtype
            self.weight: Any = None
            self.input_permutation = None
            self.output_permutation = None

        def forward(self, x: torch.Tensor) -> torch.Tensor:
            w = self.weight
            logical = dequantize_gguf_tensor(w, int(w.quant_type), self.compute_dtype)
            grouped = logical.reshape(self.n_groups, self.out_features // self.n_groups, self.in_features)
            return torch.einsum("...gk,gnk->...gn", x.to(self.compute_dtype), grouped).to(x.dtype)

    ALL_GGUF_EXPERTS_FUNCTIONS: dict[str, Callable[..., torch.Tensor]] = {}

    @dataclass
    class _ExpertExecutionPlan:
        expert_indices: torch.Tensor      # active expert ids, int64
        offsets: Optional[torch.Tensor]   # cumulative row ends of the active experts, int32
        output_mask: Optional[torch.Tensor]
        offsets_full: Optional[torch.Tensor] = None

    class GGUFExperts(torch.nn.Module):
        """Bank of packed experts with split gate / up / down projections."""

        def __init__(self, num_experts: int, hidden_dim: int, intermediate_dim: int, gate_proj, up_proj, down_proj,
                     compute_dtype: torch.dtype = torch.bfloat16, swiglu_limit: Optional[float] = None,
                     experts_implementation: str = "eager") -> None:
            super().__init__()
            self.num_experts, self.hidden_dim, self.intermediate_dim = num_experts, hidden_dim, intermediate_dim
            self.gate_proj, self.up_proj, self.down_proj = gate_proj, up_proj, down_proj
            self.compute_dtype = compute_dtype
            self.projection_layout = "split_gate_up"
            self.has_bias, self.has_gate = False, True
            self.swiglu_limit = swiglu_limit
            self.config = SimpleNamespace(_experts_implementation=experts_implementation)

        def _prepare_expert_hidden_states(self, hidden_states: torch.Tensor) -> torch.Tensor:
            return hidden_states.reshape(-1, self.hidden_dim).to(self.compute_dtype).contiguous()

        def _prepare_expert_execution(self, routing_plan: Any, mode: str) -> _ExpertExecutionPlan:
            if mode != "grouped_mm":
                raise RuntimeError(f"unsupported expert execution mode {mode!r}")
            sizes = getattr(routing_plan, "group_sizes", None)
            offsets = getattr(routing_plan, "group_offsets", None)
            if sizes is None:   # a plan built elsewhere: histogram of the sorted ids
                sizes = torch.bincount(routing_plan.expert_indices, minlength=self.num_experts).to(torch.int32)
                offsets = torch.cumsum(sizes, 0).to(torch.int32)
            # Every expert is listed (zero-row experts produce no tile), so no host synchronisation
            # is needed to find the active set.
            idx = torch.arange(self.num_experts, device=sizes.device, dtype=torch.int64)
            return _ExpertExecutionPlan(expert_indices=idx, offsets=offsets, output_mask=None, offsets_full=offsets)

        def _apply_split_gate(self, gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
            return _SwiGLU.apply(gate, up, float(self.swiglu_limit or 0.0))

        def forward(self, hidden_states: torch.Tensor, top_k_index: torch.Tensor, top_k_weights: torch.Tensor, **kwargs: Any):
            fn = ALL_GGUF_EXPERTS_FUNCTIONS[self.config._experts_implementation]
            return fn(self, hidden_states, top_k_index, top_k_weights, **kwargs)

    class DeepseekV4GGUFExperts(GGUFExperts):
        """DeepSeek-V4 expert bank: built from a model config (``num_experts``, ``hidden_size``, ``moe_intermediate_size``,
        ``swiglu_limit``) with the three packed projections assigned afterwards, as the fork's loader does.  Its
        ``_apply_split_gate`` clamps before the activation: ``silu(min(gate, L)) * clamp(up, -L, L)``
        (``test_deepseek_v4_moe_lora.py:194-196``)."""

        def __init__(self, config: Any, device: Any = None, compute_dtype: torch.dtype = torch.bfloat16) -> None:
            del device          # payloads are assigned by the caller; nothing is allocated here
            super().__init__(int(config.num_experts), int(config.hidden_size), int(config.moe_intermediate_size), None, None, None,
                             compute_dtype=compute_dtype, swiglu_limit=float(config.swiglu_limit),
                             experts_implementation=getattr(config, "_experts_implementation", "eager"))
            self.config = config
            self.act_fn = torch.nn.functional.silu


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate, up, limit):
        gate, up = gate.contiguous(), up.contiguous()
        ctx.save_for_backward(gate, up)
        ctx.limit = limit
        return ops.swiglu_fwd(gate, up, limit)

    @staticmethod
    def backward(ctx, dz):
        gate, up = ctx.saved_tensors
        dg, du = ops.swiglu_bwd(gate, up, dz.contiguous(), ctx.limit)
        return dg, du, None


def swiglu(gate: torch.Tensor, up: torch.Tensor, limit: float = 0.0) -> torch.Tensor:
    return _SwiGLU.apply(gate, up, float(limit))
