"""Router top-k selection for the fixed Qwen / DeepSeek MoE shapes (B200 build).

Public surface of the reference module of this name: ``router_topk_indices``,
``configure_fast_moe_ranking``, the geometry check and the launch helper.  Selection is one warp
per token over the 256 expert scores with packed (score, 256 - id) keys, so equal scores resolve to
the smaller expert id; normalisation of the selected scores stays ordinary autograd.
"""
from __future__ import annotations

from types import MethodType
from typing import Any, cast

import torch
import torch.nn.functional as F

from b2g import ops

try:
    from transformers.models.qwen3_5_moe.modeling_qwen3_5_moe import Qwen3_5MoeTopKRouter
except Exception:  # transformers without this model family
    class Qwen3_5MoeTopKRouter(torch.nn.Module):  # type: ignore[no-redef]
        pass
try:
    from transformers.models.deepseek_v4.modeling_deepseek_v4 import DeepseekV4HashRouter, DeepseekV4TopKRouter
except Exception:  # stock transformers has no DeepSeek-V4 yet
    class DeepseekV4TopKRouter(torch.nn.Module):  # type: ignore[no-redef]
        pass

    class DeepseekV4HashRouter(torch.nn.Module):  # type: ignore[no-redef]
        pass

_NUM_EXPERTS = 256
_SEQUENCE_LENGTH = 2048
_MAX_TOKENS = 32 * _SEQUENCE_LENGTH   # the reference stops at 16 x 2048; raised for the 65,536-token EP baseline point
_QWEN_HIDDEN_SIZE, _QWEN_TOP_K = 2048, 8
_DEEPSEEK_HIDDEN_SIZE, _DEEPSEEK_TOP_K = 4096, 6


def _is_supported_router_geometry(num_tokens: int, num_experts: int, top_k: int) -> bool:
    return 0 < num_tokens <= _MAX_TOKENS and num_experts == _NUM_EXPERTS and top_k in {_QWEN_TOP_K, _DEEPSEEK_TOP_K}


def _router_topk_launch(num_tokens: int) -> tuple[int, int, int]:
    """(rows per block, experts per lane pass, warps): 8 token rows per 256-thread block, 32 experts per
    coalesced load, one warp per row at every token count."""
    del num_tokens
    return 8, 32, 8


def router_topk_indices(logits: torch.Tensor, top_k: int, *, correction_bias: torch.Tensor | None = None,
                        score_function: str = "identity") -> torch.Tensor:
    """int64 [tokens, top_k] expert ids, best first; ties go to the smaller expert id."""
    if logits.ndim != 2:
        raise ValueError(f"Router logits must be [tokens,experts], got {logits.shape}.")
    if score_function not in {"identity", "sqrtsoftplus"}:
        raise ValueError(f"Unsupported router score function: {score_function!r}.")
    num_tokens, num_experts = logits.shape
    if not _is_supported_router_geometry(num_tokens, num_experts, top_k):
        raise RuntimeError(f"Optimized router selection supports only 256-expert top-8/top-6 workloads with at most "
                           f"{_MAX_TOKENS:,} tokens.")
    if logits.device.type != "cuda" or logits.dtype not in {torch.bfloat16, torch.float32}:
        raise RuntimeError("Optimized router selection requires CUDA BF16 or FP32 logits.")
    sqrt_softplus = score_function == "sqrtsoftplus"
    if correction_bias is not None:
        if not sqrt_softplus:
            raise ValueError("Router correction bias is supported only with sqrt-softplus scoring.")
        if correction_bias.shape != (num_experts,):
            raise ValueError(f"Router correction bias must have shape {(num_experts,)}, got {correction_bias.shape}.")
        if correction_bias.device != logits.device:
            raise ValueError("Router correction bias must be on the logits device.")
    return ops.router_topk(logits.contiguous(), top_k, correction_bias, sqrt_softplus)


def _qwen_router_forward(self: Any, hidden_states: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    flat = hidden_states.reshape(-1, self.hidden_dim)
    router_logits = F.linear(flat, self.weight)
    router_indices = router_topk_indices(router_logits, self.top_k)
    selected = router_logits.gather(1, router_indices)
    router_scores = torch.softmax(selected, dtype=torch.float32, dim=-1).to(router_logits.dtype)
    return router_logits, router_scores, router_indices


def _deepseek_topk_router_forward(self: Any, hidden_states: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    self = cast(Any, self)
    flat = hidden_states.reshape(-1, self.hidden_dim)
    logits = F.linear(flat.float(), self.weight.float())
    indices = router_topk_indices(logits, self.top_k, correction_bias=self.e_score_correction_bias, score_function="sqrtsoftplus")
    scores = self.score_fn(logits.gather(1, indices))
    weights = scores / (scores.sum(dim=-1, keepdim=True) + 1e-20)
    return logits, weights * self.routed_scaling_factor, indices


def _deepseek_hash_router_forward(self: Any, hidden_states: torch.Tensor, input_ids: torch.Tensor):
    self = cast(Any, self)
    flat = hidden_states.reshape(-1, self.hidden_dim)
    logits = F.linear(flat.float(), self.weight.float())
    indices = self.tid2eid[input_ids.reshape(-1)].long()
    scores = self.score_fn(logits.gather(1, indices))
    weights = scores / (scores.sum(dim=-1, keepdim=True) + 1e-20)
    return logits, weights * self.routed_scaling_factor, indices


def _check(module: Any, name: str, hidden: int, top_k: int, label: str, extra_ok: bool = True) -> None:
    if module.hidden_dim != hidden or module.num_experts != _NUM_EXPERTS or module.top_k != top_k or not extra_ok:
        raise RuntimeError(f"{label} router {name!r} does not match {hidden}/{_NUM_EXPERTS}/top-{top_k}.")


def configure_fast_moe_ranking(model: torch.nn.Module) -> dict[str, Any]:
    """Patch every router of a Qwen3.5-MoE or DeepSeek-V4 model with the fixed-shape selection."""
    get_base = getattr(model, "get_base_model", None)
    base = get_base() if callable(get_base) else model
    cfg = getattr(base, "config", None)
    model_type, scoring = getattr(cfg, "model_type", None), getattr(cfg, "scoring_func", None)
    paths: dict[str, list[str]] = {"qwen": [], "deepseek_topk": [], "deepseek_hash": []}
    for name, module in base.named_modules():
        if isinstance(module, Qwen3_5MoeTopKRouter):
            _check(module, name, _QWEN_HIDDEN_SIZE, _QWEN_TOP_K, "Qwen")
            module.forward = MethodType(_qwen_router_forward, module)
            paths["qwen"].append(name)
        elif isinstance(module, DeepseekV4TopKRouter):
            _check(module, name, _DEEPSEEK_HIDDEN_SIZE, _DEEPSEEK_TOP_K, "DeepSeek", scoring == "sqrtsoftplus")
            module.forward = MethodType(_deepseek_topk_router_forward, module)
            paths["deepseek_topk"].append(name)
        elif isinstance(module, DeepseekV4HashRouter):
            _check(module, name, _DEEPSEEK_HIDDEN_SIZE, _DEEPSEEK_TOP_K, "DeepSeek hash", scoring == "sqrtsoftplus")
            module.forward = MethodType(_deepseek_hash_router_forward, module)
            paths["deepseek_hash"].append(name)
    if model_type in {"qwen3_5_moe", "qwen3_5_moe_text"} and len(paths["qwen"]) != 40:
        raise RuntimeError(f"expected 40 Qwen routers, found {len(paths['qwen'])}")
    if model_type == "deepseek_v4" and (len(paths["deepseek_topk"]) != 40 or len(paths["deepseek_hash"]) != 3):
        raise RuntimeError(f"expected 40 learned and 3 hash DeepSeek routers, found {len(paths['deepseek_topk'])} and "
                           f"{len(paths['deepseek_hash'])}")
    return {"qwen": len(paths["qwen"]), "deepseek_topk": len(paths["deepseek_topk"]), "deepseek_hash": len(paths["deepseek_hash"]),
            "paths": {k: sorted(v) for k, v in paths.items()}}
