"""A whole MoE block on packed weights: routed experts plus the always-on shared expert.

DeepSeek-style decoder layers add a dense "shared expert" (a gated MLP every token passes through) to the output of the
routed experts.  The routed half is the packed expert path of ``fast_moe_lora``; the shared half is three packed LoRA
linears (``fast_lora.py:78-120`` each: one fused base + LoRA product per direction) around the same SwiGLU kernel.  In the
reference the two halves meet in the transformers fork's decoder layer; this module gives them one entry point so that the
combination can be tested and measured as a unit.
"""
from __future__ import annotations

import math
from typing import Any, Optional

import torch

from . import autograd as ag
from .gguf_types import GGUFQuantizedTensor, swiglu


class SharedExpertLora(torch.nn.Module):
    """Gated MLP ``down(silu(gate(x)) * up(x))`` on three frozen packed weights, each with its own LoRA factors."""

    def __init__(self, gate_proj: GGUFQuantizedTensor, up_proj: GGUFQuantizedTensor, down_proj: GGUFQuantizedTensor, r: int,
                 lora_alpha: int, swiglu_limit: Optional[float] = None) -> None:
        super().__init__()
        inter, hidden = (int(v) for v in gate_proj.logical_shape)
        if tuple(up_proj.logical_shape) != (inter, hidden) or tuple(down_proj.logical_shape) != (hidden, inter):
            raise ValueError("shared expert: gate/up must be [inter, hidden] and down [hidden, inter]")
        self.hidden_dim, self.intermediate_dim = hidden, inter
        self.gate_proj, self.up_proj, self.down_proj = gate_proj, up_proj, down_proj
        self.scaling = lora_alpha / r
        self.swiglu_limit = float(swiglu_limit or 0.0)
        dev = gate_proj.device
        self.lora_A = torch.nn.ParameterDict()
        self.lora_B = torch.nn.ParameterDict()
        for name, (n_in, n_out) in (("gate", (hidden, inter)), ("up", (hidden, inter)), ("down", (inter, hidden))):
            a = torch.empty(r, n_in, device=dev, dtype=torch.bfloat16)
            torch.nn.init.kaiming_uniform_(a, a=math.sqrt(5))
            self.lora_A[name] = torch.nn.Parameter(a)
            self.lora_B[name] = torch.nn.Parameter(torch.zeros(n_out, r, device=dev, dtype=torch.bfloat16))

    def _linear(self, x: torch.Tensor, weight: GGUFQuantizedTensor, name: str) -> torch.Tensor:
        return ag.lora_qlinear(x, weight.as_subclass(torch.Tensor), int(weight.quant_type), int(weight.logical_shape[0]),
                               self.lora_A[name], self.lora_B[name], self.scaling)

    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        x = hidden_states.reshape(-1, self.hidden_dim)
        z = swiglu(self._linear(x, self.gate_proj, "gate"), self._linear(x, self.up_proj, "up"), self.swiglu_limit)
        return self._linear(z, self.down_proj, "down").reshape(hidden_states.shape)


def moe_block_forward(hidden_states: torch.Tensor, top_k_index: torch.Tensor, top_k_weights: torch.Tensor, experts: Any,
                      shared_expert: Optional[torch.nn.Module] = None) -> torch.Tensor:
    """``experts(hidden, top_k_index, top_k_weights) + shared_expert(hidden)``: ``experts`` is a packed expert bank or its
    LoRA wrapper (``FastGGUFMoeLora`` / ``DeepseekV4GGUFMoeLora``), ``shared_expert`` any module on ``[tokens, hidden]``."""
    routed = experts(hidden_states, top_k_index, top_k_weights)
    if shared_expert is None:
        return routed
    return routed + shared_expert(hidden_states)
