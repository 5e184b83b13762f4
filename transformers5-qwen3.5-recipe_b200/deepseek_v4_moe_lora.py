"""DeepSeek-V4 routed experts with per-expert LoRA on packed GGUF payloads (B200 build).

Public surface of the reference module of this name (``deepseek_v4_moe_lora.py:17-94``): ``EXPERTS_IMPLEMENTATION``,
``DeepseekV4GGUFMoeLora``, ``deepseek_v4_gguf_dequant_aiter_lora_forward`` and ``register_deepseek_v4_moe_lora``, which
``train_deepseek_v4.py:32`` imports.  The name of the implementation still says "dequant + AITER" because the registry key
is part of the drop-in contract; here the routed experts (IQ2_XXS gate / up, Q2_K down in the DeepSeek-V4-Flash
checkpoint) run on this library's packed grouped kernels exactly like the Qwen experts, with the clamped SwiGLU of the
DeepSeek expert bank (``swiglu_limit``) inside the fused expert block.
"""
from __future__ import annotations

from typing import Any

import torch

from b2g.gguf_types import ALL_GGUF_EXPERTS_FUNCTIONS, DeepseekV4GGUFExperts
from deepseek_v4_lora import DEEPSEEK_V4_TARGET_MODULES_PATTERN
from fast_moe_lora import FastGGUFMoeLora, _ExpertLoraWeights, qwen3_5_moe_gguf_mmq_aiter_lora_forward

EXPERTS_IMPLEMENTATION = "deepseek_v4_gguf_dequant_aiter_lora"
_LORA_WEIGHTS_KWARG = "_deepseek_v4_gguf_lora_weights"


def _require_deepseek_experts(module: Any, who: str) -> None:
    if not isinstance(module, DeepseekV4GGUFExperts):
        raise TypeError(f"{who} requires DeepseekV4GGUFExperts, got {type(module).__name__}.")


class DeepseekV4GGUFMoeLora(FastGGUFMoeLora):
    """PEFT wrapper that owns the gate|up and down factors of one DeepSeek MoE layer.  It differs from its Qwen parent
    only in what it insists on: a ``DeepseekV4GGUFExperts`` bank switched to this module's implementation key, and the
    keyword under which the factors travel to the expert forward."""

    def forward(self, hidden_states: torch.Tensor, *args: Any, **kwargs: Any) -> torch.Tensor:
        factors = self._active_lora_weights(kwargs.pop("adapter_names", None))
        bank = self.get_base_layer()
        _require_deepseek_experts(bank, "DeepSeek V4 expert LoRA")
        chosen = bank.config._experts_implementation
        if chosen != EXPERTS_IMPLEMENTATION:
            raise RuntimeError(f"DeepSeek V4 expert LoRA requires experts_implementation={EXPERTS_IMPLEMENTATION!r}, got {chosen!r}.")
        return self.base_layer(hidden_states, *args, **{**kwargs, _LORA_WEIGHTS_KWARG: factors})


def deepseek_v4_gguf_dequant_aiter_lora_forward(self: Any, hidden_states: torch.Tensor, top_k_index: torch.Tensor,
                                                top_k_weights: torch.Tensor,
                                                _deepseek_v4_gguf_lora_weights: _ExpertLoraWeights | None = None) -> torch.Tensor:
    """Expert forward registered under ``EXPERTS_IMPLEMENTATION``: the shared packed expert path on a DeepSeek bank."""
    _require_deepseek_experts(self, EXPERTS_IMPLEMENTATION)
    return qwen3_5_moe_gguf_mmq_aiter_lora_forward(self, hidden_states, top_k_index, top_k_weights,
                                                   _qwen3_5_moe_gguf_lora_weights=_deepseek_v4_gguf_lora_weights)


def register_deepseek_v4_moe_lora(lora_config: Any, model: torch.nn.Module) -> Any:
    """Register the DeepSeek expert backend (process-wide registry) and its config-local PEFT wrapper.

    ``target_modules`` is either the one exact DeepSeek pattern (a regex string, which already names ``experts``) or a
    collection, to which ``experts`` is added."""
    hook = getattr(lora_config, "_register_custom_module", None)
    if hook is None:
        raise RuntimeError("This PEFT version has no LoraConfig._register_custom_module API.")
    if getattr(lora_config, "target_parameters", None):
        raise ValueError("DeepSeek GGUF experts target complete modules, not parameters.")
    wanted = lora_config.target_modules
    if isinstance(wanted, str):
        if wanted != DEEPSEEK_V4_TARGET_MODULES_PATTERN:
            raise ValueError("DeepSeek V4 LoRA uses one exact indexer-excluding target pattern.")
    else:
        lora_config.__dict__["target_modules"] = set(wanted or ()) | {"experts"}
    ALL_GGUF_EXPERTS_FUNCTIONS[EXPERTS_IMPLEMENTATION] = deepseek_v4_gguf_dequant_aiter_lora_forward
    model.set_experts_implementation(EXPERTS_IMPLEMENTATION)
    hook({DeepseekV4GGUFExperts: DeepseekV4GGUFMoeLora})
    return lora_config
