"""CPU oracle for the grouped-MoE part of the path (TEST INFRASTRUCTURE ONLY).

Only ``tests/``, the smoke entry and the benchmark's CPU legs may import this file.

Each function restates, in plain PyTorch on the CPU, what one piece of the reference
computes; the citations name the reference lines (and the reference test lines that use
the same independent expression as their own oracle).  The reference stores no known
answers for these; index work is compared bit-exactly, floating point within the
tolerances written in the tests.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


# ---------------------------------------------------------------------------------------
# Router top-k  (fast_moe_ranking.py:109-196; ties go to the smaller expert id, :206-210)
# ---------------------------------------------------------------------------------------
def router_scores(logits: torch.Tensor, bias: torch.Tensor | None, score_function: str) -> torch.Tensor:
    if score_function == "identity":
        return logits
    x = logits.float()
    softplus = torch.clamp(x, min=0.0) + torch.log(1.0 + torch.exp(-x.abs()))  # :98-100
    s = torch.sqrt(softplus)
    if bias is not None:
        s = s + bias.float()
    return s


def router_topk(logits: torch.Tensor, top_k: int, bias: torch.Tensor | None = None,
                score_function: str = "identity") -> torch.Tensor:
    """int64 [T, top_k], best first; equal scores resolved toward the smaller index."""
    s = router_scores(logits, bias, score_function)
    # A stable descending sort keeps equal scores in ascending index order.
    order = torch.sort(s.float(), dim=1, descending=True, stable=True).indices
    return order[:, :top_k].contiguous()


def qwen_router_weights(logits: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
    """softmax over the selected logits in fp32, cast back (fast_moe_ranking.py:280-283)."""
    return torch.softmax(logits.gather(1, indices), dtype=torch.float32, dim=-1).to(logits.dtype)


# ---------------------------------------------------------------------------------------
# Routing plan  (fast_moe_routing.py:379-428; test_fast_moe_routing.py:51-66)
# ---------------------------------------------------------------------------------------
def route_plan(top_k_index: torch.Tensor, num_experts: int = 256) -> dict[str, torch.Tensor]:
    flat = top_k_index.reshape(-1).to(torch.int64)
    expert_sorted, perm = torch.sort(flat, stable=True)     # CUDA radix sort is stable; CPU needs the flag
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(flat.numel(), dtype=torch.int64)
    sizes = torch.bincount(flat, minlength=num_experts).to(torch.int32)
    offsets = torch.cumsum(sizes, 0).to(torch.int32)         # cumulative ends, as fast_moe_lora.py:652-660 expects
    return dict(expert_indices=expert_sorted, permutation=perm, inverse_permutation=inv,
                group_sizes=sizes, offsets=offsets)


def route_gather(hidden: torch.Tensor, perm: torch.Tensor, top_k: int) -> torch.Tensor:
    return hidden[perm // top_k]                              # test_fast_moe_routing.py:147-148


def route_gather_bwd(grad_sel: torch.Tensor, inv: torch.Tensor, num_tokens: int, top_k: int) -> torch.Tensor:
    """Sum the k routed rows of a token in ascending sorted position, rounding to bf16
    after every add (fast_moe_routing.py:126-159)."""
    pos = torch.sort(inv.view(num_tokens, top_k), dim=1).values
    acc = torch.zeros(num_tokens, grad_sel.shape[1], dtype=torch.float32)
    for j in range(top_k):
        acc = (acc + grad_sel[pos[:, j]].float()).to(torch.bfloat16).float()
    return acc.to(torch.bfloat16)


def route_combine(out: torch.Tensor, weights: torch.Tensor, inv: torch.Tensor) -> torch.Tensor:
    """out[t] = sum_j expert_out[inv[t*k+j]] * bf16(w[t,j]), fp32 accumulate, one bf16 store
    (fast_moe_routing.py:162-194)."""
    t, k = weights.shape
    acc = torch.zeros(t, out.shape[1], dtype=torch.float32)
    w = weights.to(torch.bfloat16).float()
    pos = inv.view(t, k)
    for j in range(k):
        acc = acc + out[pos[:, j]].float() * w[:, j:j + 1]
    return acc.to(torch.bfloat16)


def route_combine_bwd(out: torch.Tensor, weights: torch.Tensor, perm: torch.Tensor,
                      grad_final: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """(dExpertOut bf16 [R,H], dWeights [T,k] in the weights' dtype) (fast_moe_routing.py:197-226)."""
    t, k = weights.shape
    tok = perm // k
    w = weights.reshape(-1)[perm].to(torch.bfloat16).float()
    g = grad_final[tok].float()
    d_out = (g * w[:, None]).to(torch.bfloat16)
    d_w_sorted = (g * out.float()).sum(dim=1)
    d_w = torch.empty(t * k, dtype=torch.float32)
    d_w[perm] = d_w_sorted
    return d_out, d_w.view(t, k).to(weights.dtype)


# ---------------------------------------------------------------------------------------
# Grouped products  (fast_moe_lora.py:175-396; test_fast_moe_lora.py:106-130)
# ---------------------------------------------------------------------------------------
def _segments(offsets: torch.Tensor):
    begin = 0
    for g, end in enumerate(offsets.tolist()):
        yield g, begin, int(end)
        begin = int(end)


def grouped_linear(x: torch.Tensor, w: torch.Tensor, expert_indices: torch.Tensor,
                   offsets: torch.Tensor) -> torch.Tensor:
    """rows [off[g-1], off[g]) times deq(W[expert_indices[g]])^T, fp32 accumulate, bf16 out."""
    out = torch.zeros(x.shape[0], w.shape[1], dtype=torch.bfloat16)
    for g, b, e in _segments(offsets):
        if e > b:
            out[b:e] = (x[b:e].float() @ w[int(expert_indices[g])].float().t()).to(torch.bfloat16)
    return out


def grouped_grad_input(g_out: torch.Tensor, w: torch.Tensor, expert_indices: torch.Tensor,
                       offsets: torch.Tensor, g_out2: torch.Tensor | None = None,
                       w2: torch.Tensor | None = None) -> torch.Tensor:
    """dX = dY.deq(W) per segment; with a second pair both terms share one fp32 accumulator
    and round once (test_fast_moe_lora.py:106-130)."""
    out = torch.zeros(g_out.shape[0], w.shape[2], dtype=torch.bfloat16)
    for g, b, e in _segments(offsets):
        if e > b:
            ex = int(expert_indices[g])
            acc = g_out[b:e].float() @ w[ex].float()
            if g_out2 is not None:
                acc = acc + g_out2[b:e].float() @ w2[ex].float()
            out[b:e] = acc.to(torch.bfloat16)
    return out


def grouped_mm(lhs: torch.Tensor, rhs: torch.Tensor, group_sizes: torch.Tensor) -> torch.Tensor:
    """[M,K] x [E,K,N] over contiguous row groups, zero-size groups allowed
    (the AITER gmm contract, fast_moe_lora.py:90-123)."""
    out = torch.zeros(lhs.shape[0], rhs.shape[2], dtype=lhs.dtype)
    b = 0
    for e, n in enumerate(group_sizes.tolist()):
        if n:
            out[b:b + n] = (lhs[b:b + n].float() @ rhs[e].float()).to(lhs.dtype)
        b += n
    return out


def grouped_mm_autograd(lhs: torch.Tensor, rhs: torch.Tensor, group_sizes: torch.Tensor) -> torch.Tensor:
    """Differentiable form of ``grouped_mm`` (per-group matmul in the operands' dtype)."""
    parts = []
    b = 0
    for e, n in enumerate(group_sizes.tolist()):
        if n:
            parts.append(lhs[b:b + n] @ rhs[e])
        b += n
    if not parts:
        return lhs.new_zeros(0, rhs.shape[2])
    return torch.cat(parts, 0)


def swiglu(gate: torch.Tensor, up: torch.Tensor, limit: float | None = None) -> torch.Tensor:
    """silu(gate)*up; with ``limit`` the DeepSeek clamp of test_deepseek_v4_moe_lora.py:194-196."""
    if limit is not None:
        gate = gate.clamp(max=limit)
        up = up.clamp(min=-limit, max=limit)
    return F.silu(gate) * up


def moe_layer(hidden: torch.Tensor, top_k_index: torch.Tensor, top_k_weights: torch.Tensor,
              w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor,
              lora: dict[str, torch.Tensor] | None, scaling: float,
              grad_out: torch.Tensor | None = None, compute_dtype: torch.dtype = torch.bfloat16,
              swiglu_limit: float | None = None) -> dict[str, torch.Tensor]:
    """The whole expert forward of fast_moe_lora.py:685-770 on dequantised weights, with
    autograd for the backward.  ``w_*`` are logical [E, out, in] weights; ``lora`` holds
    gate_up_a [E,r,H], gate_up_b [E,2I,r], down_a [E,r,I], down_b [E,H,r]."""
    t, k = top_k_index.shape
    plan = route_plan(top_k_index, w_gate.shape[0])
    perm, sizes = plan["permutation"], plan["group_sizes"]
    need = grad_out is not None
    h = hidden.detach().to(compute_dtype).clone().requires_grad_(need)
    wts = top_k_weights.detach().clone().float().requires_grad_(need)
    params = {}
    if lora is not None:
        params = {n: v.detach().to(compute_dtype).clone().requires_grad_(need) for n, v in lora.items()}
    sel = h[perm // k]
    cd = compute_dtype
    gate = grouped_mm_autograd(sel, w_gate.to(cd).transpose(1, 2), sizes)
    up = grouped_mm_autograd(sel, w_up.to(cd).transpose(1, 2), sizes)
    if lora is not None:
        xa = grouped_mm_autograd(sel, params["gate_up_a"].transpose(1, 2), sizes)
        delta = grouped_mm_autograd(xa, params["gate_up_b"].transpose(1, 2), sizes)
        dg, du = delta.chunk(2, dim=-1)
        gate = torch.add(gate, dg, alpha=scaling)
        up = torch.add(up, du, alpha=scaling)
    inter = swiglu(gate, up, swiglu_limit)
    out = grouped_mm_autograd(inter, w_down.to(cd).transpose(1, 2), sizes)
    if lora is not None:
        za = grouped_mm_autograd(inter, params["down_a"].transpose(1, 2), sizes)
        out = torch.add(out, grouped_mm_autograd(za, params["down_b"].transpose(1, 2), sizes), alpha=scaling)
    w_sorted = wts.reshape(-1)[perm].to(torch.bfloat16).to(out.dtype)
    final = (out * w_sorted[:, None])[plan["inverse_permutation"]].view(t, k, -1).float().sum(1).to(cd)
    res = {"out": final.detach(), "gate": gate.detach(), "up": up.detach(), "inter": inter.detach(),
           "expert_out": out.detach(), "plan": plan}
    if need:
        final.backward(grad_out.to(cd))
        res["d_hidden"] = h.grad
        res["d_weights"] = wts.grad
        for n, v in params.items():
            res["d_" + n] = v.grad if v.grad is not None else torch.zeros_like(v)
    return res


def expert_slice(rows: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor,
                 lora: dict[str, torch.Tensor] | None, scaling: float, grad_out_rows: torch.Tensor | None = None,
                 swiglu_limit: float | None = None, compute_dtype: torch.dtype = torch.float32) -> dict[str, torch.Tensor]:
    """ONE expert of ``moe_layer`` on exactly the rows routed to it: gate|up -> LoRA -> SwiGLU (clamped when
    ``swiglu_limit`` is given) -> down -> LoRA, and with ``grad_out_rows`` (the cotangent of the expert's output rows)
    the backward: the rows' input gradient and the expert's four factor gradients.  Weights are this expert's logical
    [out, in] matrices, ``lora`` its own factors gate_up_a [r,H], gate_up_b [2I,r], down_a [r,I], down_b [H,r].
    A full-size layer is checked expert by expert with this (fast_moe_lora.py:720-763 restricted to one segment)."""
    need = grad_out_rows is not None
    cd = compute_dtype
    x = rows.detach().to(cd).clone().requires_grad_(need)
    p = {} if lora is None else {n: v.detach().to(cd).clone().requires_grad_(need) for n, v in lora.items()}
    gate = x @ w_gate.to(cd).t()
    up = x @ w_up.to(cd).t()
    if lora is not None:
        delta = (x @ p["gate_up_a"].t()) @ p["gate_up_b"].t()
        dg, du = delta.chunk(2, dim=-1)
        gate = torch.add(gate, dg, alpha=scaling)
        up = torch.add(up, du, alpha=scaling)
    inter = swiglu(gate, up, swiglu_limit)
    out = inter @ w_down.to(cd).t()
    if lora is not None:
        out = torch.add(out, (inter @ p["down_a"].t()) @ p["down_b"].t(), alpha=scaling)
    res = {"out": out.detach(), "gate": gate.detach(), "up": up.detach(), "inter": inter.detach()}
    if need:
        out.backward(grad_out_rows.to(cd))
        res["d_rows"] = x.grad
        for n, v in p.items():
            res["d_" + n] = v.grad
    return res
