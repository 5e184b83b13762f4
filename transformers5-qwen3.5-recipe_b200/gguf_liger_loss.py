"""Packed LM-head chunked cross-entropy for Qwen3.5-MoE: the Q6_K head (248320 x 2048) stays in its GGUF block layout.

Mirrors the packed-loss half of the reference's ``gguf_liger_loss.py`` (``:38-355``).  The chunk loop, the autograd
function and the cross-entropy kernel are the ones of ``deepseek_v4_liger_loss`` (the two reference files carry the same
loop twice); this module adds the Qwen entry point with its own contract -- Q6_K weights, hidden size 2048 -- and the
optional token accuracy / predicted tokens (``:275-276,334-354``), and the model-forward replacement with its installer
(``gguf_liger_lce_forward`` ``:359-512``, ``apply_gguf_liger_fused_linear_cross_entropy`` ``:515-532``), which
``train_qwen3.5_35b.py:29`` imports.
"""
from __future__ import annotations

from dataclasses import dataclass
from types import MethodType
from typing import Any, Optional

import torch
from torch import nn

from b2g.gguf_types import GGUFLinear, GGUFQuantizedTensor
from deepseek_v4_liger_loss import (_PACKED_LM_HEAD_CHUNK_SIZE, _PackedQ8LigerLinearCrossEntropyFunction,  # noqa: F401
                                    _packed_q8_linear_cross_entropy_forward)

_QWEN_HEAD_QUANT_TYPE, _QWEN_HIDDEN_SIZE = 14, 2048


def _packed_q8_liger_for_causal_lm_loss(hidden_states: torch.Tensor, lm_head, labels: torch.Tensor, hidden_size: int,
                                        num_items_in_batch=None, ignore_index: int = -100, shift_labels: Optional[torch.Tensor] = None,
                                        final_logit_softcapping: Optional[float] = None, return_token_accuracy: bool = False,
                                        return_predicted_tokens: bool = False, **kwargs: Any):
    """Loss (or ``(loss, None, token_accuracy, predicted_tokens)`` when either extra is requested) of a causal LM whose
    head is a frozen packed Q6_K ``GGUFLinear``."""
    refusals = ((kwargs.get("return_z_loss", False), "z-loss output"), (kwargs.get("use_token_scaling", False), "token scaling"),
                (kwargs.get("ce_weight") is not None, "class weights"), (kwargs.get("bias") is not None, "a fused bias"),
                (float(kwargs.get("label_smoothing", 0.0)) != 0.0, "label smoothing"),
                (float(kwargs.get("lse_square_scale", 0.0)) != 0.0, "LSE square scaling"),
                (final_logit_softcapping is not None, "logit softcapping"))
    for on, what in refusals:
        if on:
            raise RuntimeError(f"Packed GGUF LM-head loss does not support {what}.")
    if kwargs.get("accum_dtype") not in {None, torch.float32}:
        raise RuntimeError("Packed GGUF LM-head loss supports only FP32 internal accumulation.")
    if not isinstance(lm_head.weight, GGUFQuantizedTensor):
        raise TypeError("Packed GGUF LM-head loss requires a GGUFQuantizedTensor weight.")
    if lm_head.input_permutation is not None or lm_head.output_permutation is not None:
        raise RuntimeError("Packed GGUF LM-head loss does not support layout permutations.")
    if lm_head.compute_dtype != torch.bfloat16:
        raise RuntimeError("Packed GGUF LM-head loss requires BF16 compute_dtype.")
    if lm_head.in_features != hidden_size or hidden_size != _QWEN_HIDDEN_SIZE:
        raise RuntimeError("Packed GGUF LM-head loss is validated only for hidden size 2048.")
    quant_type = int(lm_head.weight.quant_type)
    if quant_type != _QWEN_HEAD_QUANT_TYPE:
        raise RuntimeError("Packed GGUF LM-head loss is validated only for Q6_K weights.")
    if lm_head.weight.requires_grad:
        raise RuntimeError("Packed GGUF LM-head weights must remain frozen.")

    if shift_labels is None:
        shift_labels = nn.functional.pad(labels, (0, 1), value=ignore_index)[..., 1:].contiguous()
    flat_hidden = hidden_states.reshape(-1, hidden_size)
    flat_labels = shift_labels.reshape(-1).to(flat_hidden.device)
    reduction = "sum" if num_items_in_batch is not None else "mean"
    loss, accuracy, predicted = _PackedQ8LigerLinearCrossEntropyFunction.apply(
        flat_hidden, lm_head.weight.as_subclass(torch.Tensor), flat_labels, quant_type, lm_head.out_features,
        _PACKED_LM_HEAD_CHUNK_SIZE, ignore_index, 0.0, 0.0, reduction, None, return_token_accuracy, return_predicted_tokens)
    if num_items_in_batch is not None:
        loss = loss / num_items_in_batch
    if return_token_accuracy or return_predicted_tokens:
        return loss, None, accuracy, predicted
    return loss


def _model_types():
    """(Qwen3_5MoeForCausalLM, load_balancing_loss_func, output class): imported on first use, transformers is heavy."""
    from transformers.modeling_outputs import MoeCausalLMOutputWithPast
    from transformers.models.qwen3_5_moe.modeling_qwen3_5_moe import Qwen3_5MoeForCausalLM, load_balancing_loss_func

    try:
        from liger_kernel.transformers.model.output_classes import LigerMoeCausalLMOutputWithPast as Out  # type: ignore
    except Exception:
        @dataclass
        class Out(MoeCausalLMOutputWithPast):  # type: ignore[no-redef]
            """The stock MoE causal-LM output plus the two optional by-products of the fused loss."""
            token_accuracy: Optional[torch.Tensor] = None
            predicted_tokens: Optional[torch.Tensor] = None
    return Qwen3_5MoeForCausalLM, load_balancing_loss_func, Out


def gguf_liger_lce_forward(self, input_ids=None, attention_mask=None, position_ids=None, past_key_values=None, inputs_embeds=None,
                           labels=None, use_cache=None, output_attentions=None, output_hidden_states=None, output_router_logits=None,
                           mm_token_type_ids=None, cache_position=None, logits_to_keep: Any = 0, skip_logits: Optional[bool] = None,
                           return_dict: Optional[bool] = None, **kwargs: Any):
    """Qwen3.5-MoE causal-LM forward whose training loss runs on the packed LM head, chunk by chunk, without full logits.

    In training with labels (or ``shift_labels``) the logits are skipped and the loss comes from
    ``_packed_q8_liger_for_causal_lm_loss``; asking for logits together with labels in training is refused, as is
    ``logits_to_keep != 0`` on the fused path.  Otherwise the head and the stock loss function run as usual."""
    _, aux_loss_fn, Out = _model_types()
    cfg = self.config
    output_attentions = cfg.output_attentions if output_attentions is None else output_attentions
    output_router_logits = cfg.output_router_logits if output_router_logits is None else output_router_logits
    output_hidden_states = cfg.output_hidden_states if output_hidden_states is None else output_hidden_states
    return_dict = cfg.use_return_dict if return_dict is None else return_dict

    body = self.model(input_ids=input_ids, attention_mask=attention_mask, position_ids=position_ids, past_key_values=past_key_values,
                      inputs_embeds=inputs_embeds, use_cache=use_cache, output_attentions=output_attentions,
                      output_hidden_states=output_hidden_states, output_router_logits=output_router_logits,
                      mm_token_type_ids=mm_token_type_ids, cache_position=cache_position, **kwargs)
    hidden = body.last_hidden_state
    if hidden is None:
        raise RuntimeError("Qwen model did not return hidden states")
    keep = slice(-logits_to_keep, None) if isinstance(logits_to_keep, int) else logits_to_keep
    kept = hidden[:, keep, :]
    shift_labels = kwargs.pop("shift_labels", None)
    supervised = labels is not None or shift_labels is not None
    if skip_logits is None:
        skip_logits = bool(self.training and supervised)
    if skip_logits and not (isinstance(logits_to_keep, int) and logits_to_keep == 0):
        raise RuntimeError("Packed GGUF LM-head loss requires logits_to_keep=0 during training.")
    if skip_logits and not supervised:
        raise RuntimeError("Packed GGUF LM-head loss requires labels or shift_labels.")
    if self.training and supervised and not skip_logits:
        raise RuntimeError("Packed GGUF training with labels requires the no-full-logits fused loss.")

    loss = logits = token_accuracy = predicted_tokens = None
    if skip_logits:
        if not isinstance(self.lm_head, GGUFLinear):
            raise TypeError(f"GGUF-aware Liger loss requires a GGUFLinear LM head, got {type(self.lm_head).__name__}.")
        if self.lm_head.bias is not None:
            raise RuntimeError("GGUF-aware Liger loss currently requires a bias-free LM head.")
        result = _packed_q8_liger_for_causal_lm_loss(hidden_states=kept, lm_head=self.lm_head, labels=labels, shift_labels=shift_labels,
                                                     hidden_size=cfg.hidden_size, **kwargs)
        if isinstance(result, tuple):
            loss, _, token_accuracy, predicted_tokens = result
        else:
            loss = result
    else:
        logits = self.lm_head(kept)
        if supervised:
            loss = self.loss_function(logits=logits, labels=labels, shift_labels=shift_labels, vocab_size=self.vocab_size, **kwargs)

    aux_loss = None
    if output_router_logits:
        aux_loss = aux_loss_fn(body.router_logits, self.num_experts, self.num_experts_per_tok, attention_mask)
        if labels is not None:
            if loss is None:
                raise RuntimeError("router auxiliary loss requires a primary loss")
            loss = loss + self.router_aux_loss_coef * aux_loss.to(loss.device)

    if not return_dict:
        parts = [v for v in (loss, aux_loss) if v is not None] + [logits] + list(body[1:])
        parts += [v for v in (token_accuracy, predicted_tokens) if v is not None]
        return tuple(parts)
    return Out(loss=loss, aux_loss=aux_loss, logits=logits, past_key_values=body.past_key_values, hidden_states=body.hidden_states,
               attentions=body.attentions, router_logits=body.router_logits, token_accuracy=token_accuracy,
               predicted_tokens=predicted_tokens)


def apply_gguf_liger_fused_linear_cross_entropy(model: torch.nn.Module):
    """Patch ONE loaded Qwen3.5-MoE text model (PEFT-wrapped or not) with ``gguf_liger_lce_forward``; returns the patched model."""
    model_cls, _, _ = _model_types()
    unwrap = getattr(model, "get_base_model", None)
    target = unwrap() if callable(unwrap) else model
    if not isinstance(target, model_cls):
        raise TypeError(f"GGUF-aware Liger loss requires Qwen3_5MoeForCausalLM after unwrapping PEFT, got {type(target).__name__}.")
    if not isinstance(target.lm_head, GGUFLinear):
        raise TypeError(f"GGUF-aware Liger loss requires GGUFLinear, got {type(target.lm_head).__name__}.")
    target.forward = MethodType(gguf_liger_lce_forward, target)
    return target
