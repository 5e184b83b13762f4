"""CPU oracle for the dense quantized LoRA linear (TEST INFRASTRUCTURE ONLY).

Only ``tests/``, the smoke entry and the benchmark's CPU legs may import this file; the
product never does.

Restates the dequantize-then-matmul expressions the reference's own test uses as its
oracle (``test_fast_lora.py:110-128``): ``F.linear(x, deq(W))``, ``x @ A^T`` and
``addmm(base, xA, B^T, beta=1, alpha=s)`` (``fast_lora.py:34-65``), with autograd for
dX, dA and dB.  The reference stores no known answers for these products, so the GEMM
parity bar is the stated tolerance (rel-L2 <= 1e-2) against this file: "parity unpinned"
at the byte level, pinned only for the dequantised weights (``oracle/gguf_oracle.py``).
"""
from __future__ import annotations

import numpy as np
import torch

from . import gguf_oracle as go


def dequant_bf16(payload_u8: torch.Tensor | np.ndarray, qtype: int) -> torch.Tensor:
    """Packed uint8 [..., row_bytes] -> logical bf16 weight [..., K] on the CPU."""
    arr = payload_u8.cpu().numpy() if isinstance(payload_u8, torch.Tensor) else payload_u8
    return torch.from_numpy(go.dequantize(arr, qtype)).to(torch.bfloat16)


def lora_linear_fwd_bwd(
    x: torch.Tensor,            # bf16 [M, K]
    w_bf16: torch.Tensor,       # bf16 [N, K] (already dequantised)
    lora_a: torch.Tensor,       # bf16 [r, K]
    lora_b: torch.Tensor,       # bf16 [N, r]
    scaling: float,
    dy: torch.Tensor | None,    # bf16 [M, N]
    compute_dtype: torch.dtype = torch.bfloat16,
) -> dict[str, torch.Tensor]:
    """Y, and with ``dy`` also dX, dA, dB, by the reference test's expressions.

    ``compute_dtype=torch.float32`` gives the high-precision variant used to decide which
    of two bf16 implementations is closer to the exact product.
    """
    xr = x.detach().to(compute_dtype).clone().requires_grad_(dy is not None)
    ar = lora_a.detach().to(compute_dtype).clone().requires_grad_(dy is not None)
    br = lora_b.detach().to(compute_dtype).clone().requires_grad_(dy is not None)
    w = w_bf16.to(compute_dtype)
    base = torch.nn.functional.linear(xr, w)
    xa = torch.matmul(xr, ar.transpose(0, 1))
    y = torch.addmm(base, xa, br.transpose(0, 1), beta=1, alpha=scaling)
    out = {"y": y.detach(), "xa": xa.detach()}
    if dy is not None:
        y.backward(dy.to(compute_dtype))
        out.update(dx=xr.grad, da=ar.grad, db=br.grad)
    return out


def rel_l2(actual: torch.Tensor, expected: torch.Tensor) -> float:
    a = actual.detach().double().cpu()
    e = expected.detach().double().cpu()
    den = float(e.norm())
    return float((a - e).norm()) / (den if den > 0 else 1.0)


def fixed_grouped(x: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
    """Oracle of the fixed-group projection: ``x [..., G, K]``, dequantised ``weights [G, N, K]`` -> ``[..., G, N]`` in
    fp32, each group an independent ``F.linear`` on its slice -- the expression the reference's own check builds from
    per-group ``mmq`` calls (``test_deepseek_v4_lora.py:128-141``)."""
    groups = weights.shape[0]
    cols = [torch.nn.functional.linear(x[..., g, :].float(), weights[g].float()) for g in range(groups)]
    return torch.stack(cols, dim=-2)


def fixed_grouped_grad_input(dy: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
    """Input gradient of ``fixed_grouped``: ``dy [..., G, N]`` -> ``[..., G, K]``."""
    groups = weights.shape[0]
    cols = [dy[..., g, :].float() @ weights[g].float() for g in range(groups)]
    return torch.stack(cols, dim=-2)


def shared_expert_fwd_bwd(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor,
                          lora: dict[str, tuple[torch.Tensor, torch.Tensor]], scaling: float, dy: torch.Tensor | None,
                          swiglu_limit: float | None = None, compute_dtype: torch.dtype = torch.float32) -> dict[str, torch.Tensor]:
    """A dense gated MLP of three LoRA linears, ``down(silu(gate(x)) * up(x))`` (clamped as the DeepSeek experts are when
    ``swiglu_limit`` is given), each linear the expression of ``lora_linear_fwd_bwd``; ``lora[name] = (A [r,in], B [out,r])``
    for name in gate, up, down.  Returns y and, with ``dy``, dx and d_<name>_a / d_<name>_b."""
    need = dy is not None
    cd = compute_dtype
    xr = x.detach().to(cd).clone().requires_grad_(need)
    p = {n: (a.detach().to(cd).clone().requires_grad_(need), b.detach().to(cd).clone().requires_grad_(need)) for n, (a, b) in lora.items()}

    def lin(inp, w, name):
        a, b = p[name]
        return torch.addmm(torch.nn.functional.linear(inp, w.to(cd)), inp @ a.t(), b.t(), beta=1, alpha=scaling)

    gate, up = lin(xr, w_gate, "gate"), lin(xr, w_up, "up")
    if swiglu_limit is not None:
        gate, up = gate.clamp(max=swiglu_limit), up.clamp(min=-swiglu_limit, max=swiglu_limit)
    y = lin(torch.nn.functional.silu(gate) * up, w_down, "down")
    out = {"y": y.detach()}
    if need:
        y.backward(dy.to(cd))
        out["dx"] = xr.grad
        for n, (a, b) in p.items():
            out[f"d_{n}_a"], out[f"d_{n}_b"] = a.grad, b.grad
    return out
