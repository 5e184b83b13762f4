"""Packed LM-head chunked cross-entropy: the loss of a causal LM whose head stays in its GGUF block layout.

Mirrors the packed-loss half of the reference's ``deepseek_v4_liger_loss.py`` (``:66-318``; the Qwen twin is
``gguf_liger_loss.py:38-262``): per chunk of hidden-state rows the packed product ``mmq`` makes bf16 logits, a
cross-entropy kernel turns them into their cotangents in place, and ``mmq_grad_input`` multiplies those back through the
packed head, so that neither a logical LM-head matrix nor the logits of the whole sequence ever exist.  The input
gradient is finished in the forward and only scaled in the backward.

Differences from the reference: the cross-entropy kernel is this library's (``b2g_cross_entropy_inplace``) instead of
Liger's Triton kernel; the count of non-ignored targets stays on the device (no ``.item()``); chunks are row views of the
hidden states (the packed product accepts an offset view, so the per-chunk clone is gone).  Every native type of this
library is accepted as the head's type here (the reference validates Q8_0 here and Q6_K in the Qwen twin, `gguf_liger_loss`).
``apply_deepseek_v4_liger_loss`` (``:395-416``) patches one ``DeepseekV4ForCausalLM`` instance so that its forward
(``_deepseek_v4_liger_forward``, ``:321-392``) computes the training loss through the packed path, and
``deepseek_v4_liger_causal_lm_loss`` (``:35-63``) is the comparison loss that materialises the head.  The model class comes
from the transformers fork; without the fork the installer recognises the model by its class name and structure.
"""
from __future__ import annotations

from types import MethodType
from typing import Any, Optional

import torch
from torch import nn

from b2g import ops as _ops
from b2g.gguf_types import GGUFLinear, GGUFQuantizedTensor, dequantize_gguf_tensor

try:  # the transformers fork carries the DeepSeek-V4 model
    from transformers.models.deepseek_v4.modeling_deepseek_v4 import DeepseekV4ForCausalLM, load_balancing_loss_func  # type: ignore
except Exception:
    DeepseekV4ForCausalLM = None   # recognised by name below

    def load_balancing_loss_func(gate_logits, num_experts=None, top_k=2, attention_mask=None):
        """Switch-Transformer auxiliary loss: experts x (fraction of routed slots) . (mean router probability), summed."""
        if gate_logits is None or not isinstance(gate_logits, (tuple, list)):
            return 0
        device = gate_logits[0].device
        logits = torch.cat([layer.to(device) for layer in gate_logits], dim=0)
        probs = torch.softmax(logits, dim=-1)
        chosen = torch.nn.functional.one_hot(torch.topk(probs, top_k, dim=-1).indices, num_experts).float()
        if attention_mask is None:
            slots, mean_prob = chosen.mean(dim=0), probs.mean(dim=0)
        else:
            batch, seq = attention_mask.shape
            layers = logits.shape[0] // (batch * seq)
            keep = attention_mask[None, :, :, None].expand(layers, batch, seq, 1).reshape(-1, 1).to(device).float()
            slots = (chosen * keep[:, None, :]).sum(dim=0) / keep.sum().clamp(min=1)
            mean_prob = (probs * keep).sum(dim=0) / keep.sum().clamp(min=1)
        return (slots * mean_prob[None, :]).sum() * num_experts

# Rows per chunk.  The reference uses 512 (256 for Qwen) to bound the logits workspace on a memory-poor APU.  Here the input
# gradient of a chunk is a product with a 129280-step reduction and only (rows / 512) x (hidden / 256) output tiles, so 512
# rows would keep 16 of the 74 CTA pairs busy; 2048 rows fill them, and the 530 MB of bf16 logits are small on a 180 GB part.
_PACKED_LM_HEAD_CHUNK_SIZE = 2048


def _packed_q8_linear_cross_entropy_forward(input: torch.Tensor, packed_weight: torch.Tensor, target: torch.Tensor, quant_type: int,
                                            out_features: int, chunk_size: int, ignore_index: int, lse_square_scale: float,
                                            label_smoothing: float, reduction: str, softcap: Optional[float],
                                            return_token_accuracy: bool = False, return_predicted_tokens: bool = False):
    """Chunked packed product, in-place cross-entropy and packed input gradient.
    Returns (loss, token_accuracy | None, predicted_tokens | None, grad_input)."""
    if input.ndim != 2:
        raise ValueError(f"Packed LM-head loss expects two-dimensional hidden states, got {input.shape}.")
    if input.dtype != torch.bfloat16:
        raise TypeError(f"Packed LM-head loss requires BF16 hidden states, got {input.dtype}.")
    if target.ndim != 1 or target.shape[0] != input.shape[0]:
        raise ValueError("Packed LM-head targets must be one-dimensional and match the hidden-state row count.")
    if target.dtype != torch.long:
        raise TypeError(f"Packed LM-head targets require torch.long, got {target.dtype}.")
    if reduction not in {"mean", "sum"}:
        raise ValueError(f"Packed LM-head loss supports only mean or sum reduction, got {reduction!r}.")
    if chunk_size <= 0:
        raise ValueError(f"Packed LM-head chunk_size must be positive, got {chunk_size}.")
    if lse_square_scale != 0.0 or label_smoothing != 0.0 or softcap is not None:
        raise RuntimeError("Packed LM-head loss supports neither LSE square scaling, label smoothing nor logit softcapping.")

    rows, hidden_size = input.shape
    input = input.contiguous()
    target = target.contiguous()
    count = (target != ignore_index).sum().reshape(1)                     # stays on the device
    grad_input = torch.empty_like(input)
    loss_rows = torch.empty(rows, dtype=torch.float32, device=input.device)
    correct = torch.empty(rows, dtype=torch.float32, device=input.device) if return_token_accuracy else None
    predicted = torch.empty(rows, dtype=torch.int64, device=input.device) if return_predicted_tokens else None
    payload = packed_weight.reshape(-1)
    for start in range(0, rows, chunk_size):
        end = min(start + chunk_size, rows)
        logits = torch.ops.b2g.mmq(input[start:end], payload, int(quant_type), int(out_features))
        _ops.cross_entropy_inplace(logits, target[start:end], loss_rows[start:end], count, reduction == "mean", ignore_index,
                                   None if predicted is None else predicted[start:end], None if correct is None else correct[start:end])
        grad_input[start:end] = torch.ops.b2g.mmq_grad_input(logits, payload, int(quant_type), int(hidden_size))
    loss = loss_rows.sum()
    accuracy = None if correct is None else correct.sum() / count.clamp(min=1).to(torch.float32)[0]
    return loss, accuracy, predicted, grad_input


class _PackedQ8LigerLinearCrossEntropyFunction(torch.autograd.Function):
    """Fused loss over a frozen packed LM head; the input gradient is computed in the forward."""

    @staticmethod
    def forward(ctx, input, packed_weight, target, quant_type, out_features, chunk_size, ignore_index, lse_square_scale,
                label_smoothing, reduction, softcap, return_token_accuracy=False, return_predicted_tokens=False):
        loss, accuracy, predicted, grad_input = _packed_q8_linear_cross_entropy_forward(
            input, packed_weight, target, quant_type, out_features, chunk_size, ignore_index, lse_square_scale, label_smoothing,
            reduction, softcap, return_token_accuracy, return_predicted_tokens)
        ctx.save_for_backward(grad_input.detach())
        extras = tuple(t for t in (accuracy, predicted) if t is not None)
        if extras:
            ctx.mark_non_differentiable(*extras)
        return loss, accuracy, predicted

    @staticmethod
    def backward(ctx, grad_output, grad_accuracy, grad_predicted):
        del grad_accuracy, grad_predicted
        if torch.is_grad_enabled():
            raise RuntimeError("Packed GGUF LM-head loss does not support higher-order gradients")
        (grad_input,) = ctx.saved_tensors
        return (grad_input * grad_output.to(grad_input.dtype),) + (None,) * 12


def _packed_q8_liger_for_causal_lm_loss(hidden_states: torch.Tensor, lm_head, labels: torch.Tensor, hidden_size: int,
                                        num_items_in_batch=None, ignore_index: int = -100, shift_labels: Optional[torch.Tensor] = None,
                                        final_logit_softcapping: Optional[float] = None, **kwargs: Any) -> torch.Tensor:
    """Causal-LM loss on a packed head: labels are shifted by one unless ``shift_labels`` is given; ``num_items_in_batch``
    switches to sum reduction divided by that count (gradient accumulation), as in the reference."""
    refused = (("return_z_loss", kwargs.get("return_z_loss", False)), ("use_token_scaling", kwargs.get("use_token_scaling", False)),
               ("ce_weight", kwargs.get("ce_weight") is not None), ("bias", kwargs.get("bias") is not None),
               ("label_smoothing", float(kwargs.get("label_smoothing", 0.0)) != 0.0),
               ("lse_square_scale", float(kwargs.get("lse_square_scale", 0.0)) != 0.0),
               ("final_logit_softcapping", final_logit_softcapping is not None))
    for name, on in refused:
        if on:
            raise RuntimeError(f"Packed DeepSeek Q8_0 LM-head loss does not support {name}.")
    if kwargs.get("accum_dtype") not in {None, torch.float32}:
        raise RuntimeError("Packed DeepSeek Q8_0 LM-head loss supports only FP32 internal accumulation.")
    if not isinstance(lm_head.weight, GGUFQuantizedTensor):
        raise TypeError("Packed DeepSeek LM-head loss requires a GGUFQuantizedTensor.")
    if lm_head.input_permutation is not None or lm_head.output_permutation is not None:
        raise RuntimeError("Packed DeepSeek Q8_0 LM-head loss does not support layout permutations.")
    if lm_head.compute_dtype != torch.bfloat16:
        raise RuntimeError("Packed DeepSeek Q8_0 LM-head loss requires BF16 compute_dtype.")
    if lm_head.in_features != hidden_size or hidden_states.shape[-1] != hidden_size:
        raise RuntimeError("Packed DeepSeek Q8_0 LM-head loss hidden size does not match the LM head.")
    quant_type = int(lm_head.weight.quant_type)
    if quant_type not in _ops.NATIVE_QUANT_TYPES:
        raise RuntimeError("Packed DeepSeek LM-head loss is validated only for Q8_0 weights (the other native types of this library are accepted too).")
    if lm_head.weight.requires_grad:
        raise RuntimeError("Packed DeepSeek LM-head weights must remain frozen.")

    if shift_labels is None:
        shift_labels = nn.functional.pad(labels, (0, 1), value=ignore_index)[..., 1:].contiguous()
    flat_hidden = hidden_states.reshape(-1, hidden_size)
    flat_labels = shift_labels.reshape(-1).to(flat_hidden.device)
    reduction = "sum" if num_items_in_batch is not None else "mean"
    loss, _, _ = _PackedQ8LigerLinearCrossEntropyFunction.apply(
        flat_hidden, lm_head.weight.as_subclass(torch.Tensor), flat_labels, quant_type, lm_head.out_features,
        _PACKED_LM_HEAD_CHUNK_SIZE, ignore_index, 0.0, 0.0, reduction, None)
    return loss / num_items_in_batch if num_items_in_batch is not None else loss


def deepseek_v4_packed_liger_causal_lm_loss(hidden_states: torch.Tensor, lm_head, labels: torch.Tensor, *, hidden_size: int,
                                            loss_kwargs: Optional[dict[str, Any]] = None) -> torch.Tensor:
    """Public scoped packed loss used by an optimized model forward."""
    return _packed_q8_liger_for_causal_lm_loss(hidden_states, lm_head, labels, hidden_size=hidden_size, **(loss_kwargs or {}))


def _logical_head(lm_head, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
    materialize = getattr(lm_head, "materialize_logical_weight", None)
    if callable(materialize):
        return materialize(dtype=dtype, device=device)
    w = lm_head.weight
    return dequantize_gguf_tensor(w, int(w.quant_type), dtype, device).reshape(lm_head.out_features, lm_head.in_features)


def deepseek_v4_liger_causal_lm_loss(hidden_states: torch.Tensor, lm_head, labels: torch.Tensor, *, hidden_size: int,
                                     loss_kwargs: Optional[dict[str, Any]] = None) -> torch.Tensor:
    """Comparison loss that MATERIALISES the frozen head (dequantised to the hidden states' dtype) and takes the shifted
    causal-LM cross-entropy of full logits, 1024 rows at a time.  For correctness audits of the packed loss only: it holds a
    vocabulary-sized logical matrix, which the training path never does."""
    if lm_head.weight.requires_grad:
        raise RuntimeError("DeepSeek V4 reference loss requires a frozen LM head.")
    kw = dict(loss_kwargs or {})
    ignore_index = int(kw.get("ignore_index", -100))
    shift = kw.get("shift_labels")
    if shift is None:
        shift = nn.functional.pad(labels, (0, 1), value=ignore_index)[..., 1:]
    rows = hidden_states.reshape(-1, hidden_size)
    shift = shift.reshape(-1).to(rows.device)
    head = _logical_head(lm_head, hidden_states.dtype, hidden_states.device)
    total = rows.new_zeros((), dtype=torch.float32)
    for start in range(0, rows.shape[0], 1024):
        logits = nn.functional.linear(rows[start:start + 1024], head).float()
        total = total + nn.functional.cross_entropy(logits, shift[start:start + 1024], ignore_index=ignore_index, reduction="sum")
    items = kw.get("num_items_in_batch")
    return total / (items if items is not None else (shift != ignore_index).sum().clamp(min=1))


def _deepseek_v4_liger_forward(self, input_ids=None, attention_mask=None, position_ids=None, past_key_values=None, inputs_embeds=None,
                               labels=None, use_cache=None, output_router_logits=None, logits_to_keep: Any = 0, **kwargs: Any):
    """``DeepseekV4ForCausalLM.forward`` with the training loss taken on the packed head: with labels the logits are never
    formed (``logits`` is None in the output); without labels the head runs on the kept positions as usual.  The router
    auxiliary loss is added as in the stock forward."""
    from transformers.modeling_outputs import MoeCausalLMOutputWithPast

    if output_router_logits is None:
        output_router_logits = self.config.output_router_logits
    body = self.model(input_ids=input_ids, attention_mask=attention_mask, position_ids=position_ids, past_key_values=past_key_values,
                      inputs_embeds=inputs_embeds, use_cache=use_cache, output_router_logits=output_router_logits, **kwargs)
    hidden = body.last_hidden_state
    loss = logits = aux_loss = None
    if labels is not None:
        loss = deepseek_v4_packed_liger_causal_lm_loss(hidden, self.lm_head, labels, hidden_size=self.config.hidden_size, loss_kwargs=kwargs)
    else:
        keep = slice(-logits_to_keep, None) if isinstance(logits_to_keep, int) else logits_to_keep
        logits = self.lm_head(hidden[:, keep, :])
    if output_router_logits:
        aux_loss = load_balancing_loss_func(body.router_logits, self.num_experts, self.num_experts_per_tok, attention_mask)
        if labels is not None:
            if loss is None:
                raise RuntimeError("router auxiliary loss requires a primary loss")
            loss = loss + self.router_aux_loss_coef * aux_loss.to(loss.device)
    return MoeCausalLMOutputWithPast(loss=loss, aux_loss=aux_loss, logits=logits, past_key_values=body.past_key_values,
                                     hidden_states=body.hidden_states, attentions=body.attentions, router_logits=body.router_logits)


def _is_deepseek_v4_causal_lm(module: Any) -> bool:
    if DeepseekV4ForCausalLM is not None:
        return isinstance(module, DeepseekV4ForCausalLM)
    return any(c.__name__ == "DeepseekV4ForCausalLM" for c in type(module).__mro__)


def apply_deepseek_v4_liger_loss(model: torch.nn.Module):
    """Patch ONE model instance (PEFT-wrapped or not) with the packed-head loss forward; idempotent.  Returns the patched
    base model."""
    unwrap = getattr(model, "get_base_model", None)
    base = unwrap() if callable(unwrap) else model
    if not _is_deepseek_v4_causal_lm(base):
        raise TypeError(f"DeepSeek V4 Liger loss requires DeepseekV4ForCausalLM, got {type(base).__name__}.")
    if not isinstance(base.lm_head, GGUFLinear):
        raise TypeError(f"DeepSeek V4 GGUF loss requires GGUFLinear lm_head, got {type(base.lm_head).__name__}.")
    if not getattr(base, "_deepseek_v4_liger_loss_enabled", False):
        base.forward = MethodType(_deepseek_v4_liger_forward, base)
        base.__dict__["_deepseek_v4_liger_loss_enabled"] = True
    return base
