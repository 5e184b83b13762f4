"""DeepSeek-V4 glue of the packed-weight path: wrapper aliases and the frozen eight-group projection.

Mirrors the parts of the reference's ``deepseek_v4_lora.py`` that sit on the quantized matrix-product path:

* ``DeepseekV4LoraLinear`` / ``DeepseekV4GGUFLoraLinear`` (``deepseek_v4_lora.py:51-56``): DeepSeek-owned names for the
  fused LoRA linears of ``fast_lora``; grouped ``o_a_proj`` adapters are refused (``:59-64``).
* ``register_deepseek_v4_lora`` (``:67-88``): installs those wrappers through PEFT's custom-module hook and insists on
  the exact target pattern.
* ``configure_deepseek_v4_grouped_mmq`` (``:128-162``) with its forward (``:91-125``): the frozen ``GGUFGroupedLinear``
  ``[..., 8, 4096] -> [..., 8, 1024]`` Q8_0 projection runs as one native fixed-group product on the packed payload
  (``b2g.autograd.fixed_grouped_mmq`` in place of ``torch_ggml_ops.fixed_grouped_mmq``), failing closed when a module
  does not match the contract.

* ``normalize_peft_path`` / ``audit_deepseek_v4_injection`` (``:165-287``): the check, run once before training, that the
  adapters landed exactly where the DeepSeek-V4-Flash contract says (383 ordinary wrappers, 43 expert wrappers, 43 frozen
  grouped projections, the rank-proportional parameter count, bf16 CUDA adapter tensors only, no packed payload trainable).
"""
from __future__ import annotations

import re
from types import MethodType
from typing import Any

import torch

from b2g import autograd as _ag
from b2g.gguf_types import GGUFGroupedLinear, GGUFLinear, GGUFQuantizedTensor
from fast_lora import FastGGUFLoraLinear, FastLoraLinear

ORDINARY_TARGET_MODULES = frozenset({"q_a_proj", "q_b_proj", "kv_proj", "o_b_proj", "gate_proj", "up_proj", "down_proj"})
DEEPSEEK_V4_TARGET_MODULES_PATTERN = (
    r"^(?!.*\.self_attn\.compressor\.indexer\.)(?:.*\.)?"
    r"(?:q_a_proj|q_b_proj|kv_proj|o_b_proj|gate_proj|up_proj|down_proj|experts)$"
)

EXPECTED_ORDINARY_WRAPPERS = 383
EXPECTED_EXPERT_WRAPPERS = 43
EXPECTED_RANK4_PARAMETERS = 645_609_472

# no adapter may sit on (or train) any of these
_FORBIDDEN_TRAINABLE_PATHS = (".o_a_proj.", ".mlp.gate.", ".attn_hc.", ".ffn_hc.", ".hc_head.", ".input_layernorm.",
                              ".post_attention_layernorm.", ".q_a_norm.", ".q_b_norm.", ".kv_norm.", ".sinks", ".position_bias",
                              ".self_attn.compressor.indexer.", "embed_tokens", "lm_head")
_ADAPTER_PARAMETER = re.compile(r"\.lora_[AB](?:_down)?\.")

FIXED_GROUPS, FIXED_IN_FEATURES, FIXED_GROUP_OUT_FEATURES, FIXED_QUANT_TYPE = 8, 4096, 1024, 8


class DeepseekV4LoraLinear(FastLoraLinear):
    """DeepSeek-owned wrapper for ordinary floating linear modules."""


class DeepseekV4GGUFLoraLinear(FastGGUFLoraLinear):
    """DeepSeek-owned wrapper with capability-based packed base dispatch."""


class _RejectedDeepseekV4GroupedLora(DeepseekV4GGUFLoraLinear):
    def __init__(self, *args: Any, **kwargs: Any) -> None:
        del args, kwargs
        raise RuntimeError("DeepSeek V4 grouped o_a_proj LoRA is unsupported; keep GGUFGroupedLinear frozen.")


def register_deepseek_v4_lora(lora_config):
    """Register the DeepSeek wrappers on a LoraConfig without touching the installed PEFT."""
    register = getattr(lora_config, "_register_custom_module", None)
    if register is None:
        raise RuntimeError("This PEFT version has no LoraConfig._register_custom_module API.")
    if lora_config.target_modules != DEEPSEEK_V4_TARGET_MODULES_PATTERN:
        raise ValueError("DeepSeek V4 target_modules must use the exact indexer-excluding pattern "
                         f"{DEEPSEEK_V4_TARGET_MODULES_PATTERN!r}.")
    register({GGUFGroupedLinear: _RejectedDeepseekV4GroupedLora, GGUFLinear: DeepseekV4GGUFLoraLinear,
              torch.nn.Linear: DeepseekV4LoraLinear})
    return lora_config


def _packed_groups_of(module) -> torch.Tensor:
    """The module's flattened ``[groups * N, row bytes]`` parameter viewed as ``[groups, N, row bytes]``."""
    per_group = module.out_features // module.n_groups
    raw = module.weight.as_subclass(torch.Tensor)
    if raw.ndim != 2 or raw.shape[0] != module.n_groups * per_group:
        raise RuntimeError("DeepSeek fixed grouped MMQ expects a flattened grouped payload with "
                           f"{module.n_groups * per_group} rows, got {tuple(raw.shape)}.")
    return raw.reshape(module.n_groups, per_group, -1)


def _deepseek_v4_fixed_grouped_mmq_forward(self, input: torch.Tensor) -> torch.Tensor:
    """Forward of a frozen grouped projection on its packed payload: every group multiplies its own column block of the
    input, one native product for all of them, no logical weight and no per-group copies."""
    if self.compute_dtype != torch.bfloat16:
        raise RuntimeError("DeepSeek fixed grouped MMQ requires BF16 compute_dtype.")
    if not (self.input_permutation is None and self.output_permutation is None):
        raise RuntimeError("DeepSeek fixed grouped MMQ does not support layout permutations.")
    x = input.to(self.compute_dtype)
    if x.storage_offset() != 0 or not x.is_contiguous():
        x = x.contiguous()
    y = _ag.fixed_grouped_mmq(x, _packed_groups_of(self), int(self.weight.quant_type))
    return y.to(input.dtype)


def _matches_fixed_contract(module) -> bool:
    return (int(module.weight.quant_type) == FIXED_QUANT_TYPE and module.n_groups == FIXED_GROUPS
            and module.in_features == FIXED_IN_FEATURES and module.out_features == FIXED_GROUPS * FIXED_GROUP_OUT_FEATURES)


def configure_deepseek_v4_grouped_mmq(model: torch.nn.Module) -> dict[str, Any]:
    """Install the native fixed-group path on every ``GGUFGroupedLinear`` of one model instance.  The modules stay
    ordinary frozen modules (no adapter); a module outside the eight-group Q8_0 4096 -> 1024 contract is an error, not a
    silent fallback to the logical product."""
    unwrap = getattr(model, "get_base_model", None)
    root = unwrap() if callable(unwrap) else model
    enabled: list[str] = []
    for path, module in root.named_modules():
        if isinstance(module, GGUFGroupedLinear):
            if not isinstance(module.weight, GGUFQuantizedTensor):
                raise TypeError(f"DeepSeek grouped projection {path!r} is not GGUF-quantized.")
            if not _matches_fixed_contract(module):
                raise RuntimeError("DeepSeek grouped projection does not match the fixed eight-group "
                                   f"Q8_0 4096->1024 contract: {path!r}.")
            if not getattr(module, "_deepseek_v4_grouped_mmq_enabled", False):
                module.forward = MethodType(_deepseek_v4_fixed_grouped_mmq_forward, module)
                module._deepseek_v4_grouped_mmq_enabled = True
            enabled.append(path)
    return {"enabled": len(enabled), "paths": sorted(enabled)}


def normalize_peft_path(path: str) -> str:
    """Module path as it was before PEFT wrapped the model: PEFT's ``base_model.model.`` and a leading ``model.`` are
    dropped, then decoder-layer paths get the one ``model.`` prefix the adapter contract uses."""
    for prefix in ("base_model.model.", "model."):
        if path.startswith(prefix):
            path = path[len(prefix):]
    if path.startswith("model.layers."):
        return path
    return f"model.{path}" if path.startswith("layers.") else path


def audit_deepseek_v4_injection(model: torch.nn.Module, *, expert_wrapper_type: type[torch.nn.Module], rank: int) -> dict[str, Any]:
    """Validate the complete adapter surface of a wrapped DeepSeek-V4-Flash model before training; raises one
    ``RuntimeError`` listing every violated rule, otherwise returns the census."""
    ordinary_types = (DeepseekV4LoraLinear, DeepseekV4GGUFLoraLinear)
    ordinary, expert, grouped, grouped_trainable = [], [], [], []
    for path, module in model.named_modules():
        if isinstance(module, expert_wrapper_type):
            expert.append(normalize_peft_path(path))
        elif isinstance(module, ordinary_types):
            ordinary.append(normalize_peft_path(path))
        if isinstance(module, GGUFGroupedLinear):
            grouped.append(normalize_peft_path(path))
            if module.weight.requires_grad:
                grouped_trainable.append(path)
    named = list(model.named_parameters())
    trainable = [(n, p) for n, p in named if p.requires_grad]
    n_trainable = sum(p.numel() for _, p in trainable)
    n_expected = EXPECTED_RANK4_PARAMETERS * rank // 4

    problems: list[str] = []
    for found, expected, what in ((len(ordinary), EXPECTED_ORDINARY_WRAPPERS, f"{EXPECTED_ORDINARY_WRAPPERS} ordinary wrappers"),
                                  (len(expert), EXPECTED_EXPERT_WRAPPERS, f"{EXPECTED_EXPERT_WRAPPERS} expert wrappers"),
                                  (len(grouped), EXPECTED_EXPERT_WRAPPERS, "43 frozen grouped o_a_proj modules"),
                                  (n_trainable, n_expected, f"{n_expected} rank-{rank} adapter parameters")):
        if found != expected:
            problems.append(f"expected {what}, found {found}")
    checks = (
        ("non-adapter trainable tensors", [n for n, _ in trainable if _ADAPTER_PARAMETER.search(n) is None]),
        ("forbidden trainable paths", [n for n, _ in trainable if any(frag in n for frag in _FORBIDDEN_TRAINABLE_PATHS)]),
        ("non-BF16 adapter tensors", [n for n, p in trainable if p.dtype != torch.bfloat16]),
        ("adapter tensors outside cuda:0", [n for n, p in trainable if p.device.type != "cuda"]),
        ("trainable grouped o_a_proj weights", grouped_trainable),
        ("trainable packed payloads", [n for n, p in named if isinstance(p, GGUFQuantizedTensor) and p.requires_grad]),
    )
    problems += [f"{what}: {names[:8]}" for what, names in checks if names]
    if problems:
        raise RuntimeError("DeepSeek V4 adapter injection audit failed: " + "; ".join(problems))
    return {
        "ordinary_wrappers": len(ordinary),
        "expert_wrappers": len(expert),
        "wrapped_modules": len(ordinary) + len(expert),
        "trainable_tensors": len(trainable),
        "trainable_parameters": n_trainable,
        "trainable_bytes": sum(p.numel() * p.element_size() for _, p in trainable),
        "adapter_dtypes": sorted({str(p.dtype) for _, p in trainable}),
        "ordinary_target_paths": sorted(ordinary),
        "expert_target_paths": sorted(expert),
        "grouped_output_paths": sorted(grouped),
        "packed_parameters": sum(isinstance(p, GGUFQuantizedTensor) for p in model.parameters()),
    }
