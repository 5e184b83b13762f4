"""Packed LM-head chunked cross-entropy for Qwen3.5-MoE: the Q6_K head (248320 x 2048) stays in its GGUF block layout.

Mirrors the packed-loss half of the reference's ``gguf_liger_loss.py`` (``:38-355``).  The chunk loop, the autograd
function and the cross-entropy kernel are the ones of ``deepseek_v4_liger_loss`` (the two reference files carry the same
loop twice); this module adds the Qwen entry point with its own contract -- Q6_K weights, hidden size 2048 -- and the
optional token accuracy / predicted tokens (``:275-276,334-354``).  The model-forward replacement of the reference
(``gguf_liger_lce_forward`` and its installer) is trainer glue and not part of this path.
"""
from __future__ import annotations

from typing import Any, Optional

import torch
from torch import nn

from b2g.gguf_types import GGUFQuantizedTensor
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
