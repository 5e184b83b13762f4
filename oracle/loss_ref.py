"""CPU oracle of the packed LM-head chunked cross-entropy (test infrastructure only; never imported by the product).

Restates what the reference computes per chunk (``gguf_liger_loss.py:107-178``, ``deepseek_v4_liger_loss.py:115-165``):
logits = bf16(hidden . W^T), cross-entropy of the fp32 view of those bf16 logits with the batch-wide count of non-ignored
targets as the mean's denominator, cotangent (softmax - onehot) / count rounded to bf16, input gradient = cotangent . W.
The chunking itself does not change any number (rows are independent), so the oracle evaluates all rows at once.
"""
from __future__ import annotations

import torch


def packed_linear_cross_entropy(hidden: torch.Tensor, weight: torch.Tensor, target: torch.Tensor, ignore_index: int = -100,
                                reduction: str = "mean") -> dict[str, torch.Tensor]:
    """hidden [T, H] bf16, weight [V, H] (dequantised, bf16 or fp32), target [T] int64 ->
    loss (fp32 scalar), grad_input [T, H] fp32, predicted [T] int64 (-1 where ignored), accuracy (scalar)."""
    w = weight.float()
    logits = (hidden.float() @ w.t()).bfloat16().float()
    live = target != ignore_index
    n = int(live.sum())
    per_row = torch.nn.functional.cross_entropy(logits, target, ignore_index=ignore_index, reduction="none")
    scale = 1.0 / max(n, 1) if reduction == "mean" else 1.0
    loss = per_row.sum() * scale
    prob = torch.softmax(logits, dim=-1)
    onehot = torch.zeros_like(prob)
    rows = torch.nonzero(live).reshape(-1)
    onehot[rows, target[rows]] = 1.0
    cot = ((prob - onehot) * scale * live[:, None]).bfloat16().float()
    pred = torch.where(live, logits.argmax(dim=-1), torch.full_like(target, -1))
    acc = ((pred == target) & live).sum().float() / max(n, 1)
    return {"loss": loss, "grad_input": cot @ w, "predicted": pred, "accuracy": acc, "logits": logits}
