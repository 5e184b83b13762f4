"""Autograd layer over ``b2g.ops``: the operators the reference's modules call.

Dense path
    ``mmq`` / ``mmq_grad_input``    the two operators of the third-party torch_ggml_ops package that
                                    ``fast_lora.py:155`` and ``gguf_liger_loss.py:109,172`` call,
                                    registered as ``torch.ops.b2g.*`` with fake kernels and autograd
    ``lora_qlinear``                base product and LoRA residual of ``fast_lora.py:78-120`` in one
                                    pass: Y = X.deq(W)^T + s.(X.A^T).B^T, backward dX, dA, dB
Grouped path
    ``grouped_mmq`` / ``grouped_mmq_pair`` and their ``*_grad_input`` (``fast_moe_lora.py:221-262,339-375``)
    ``grouped_lora_experts``        the expert block of ``fast_moe_lora.py:720-763`` (pair product, LoRA,
                                    SwiGLU, down product, LoRA) with a hand-written backward

Packed payloads are frozen: none of these ever produces a gradient for them.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import ops

_LIB = torch.library.Library("b2g", "DEF")
_LIB.define("mmq(Tensor x, Tensor payload, int quant_type, int out_features) -> Tensor")
_LIB.define("mmq_grad_input(Tensor grad_output, Tensor payload, int quant_type, int in_features) -> Tensor")
_LIB.define("fixed_grouped_mmq(Tensor x, Tensor packed_groups, int quant_type) -> Tensor")
_LIB.define("fixed_grouped_mmq_grad_input(Tensor grad_output, Tensor packed_groups, int quant_type) -> Tensor")
_LIB.define("grouped_mmq(Tensor x, Tensor payload, Tensor expert_indices, Tensor expert_offsets, int quant_type, "
            "int out_features) -> Tensor")
_LIB.define("grouped_mmq_grad_input(Tensor grad_output, Tensor payload, Tensor expert_indices, Tensor expert_offsets, "
            "int quant_type, int in_features) -> Tensor")
_LIB.define("grouped_mmq_pair(Tensor x, Tensor payload0, Tensor payload1, Tensor expert_indices, Tensor expert_offsets, "
            "int quant_type, int out_features) -> (Tensor, Tensor)")
_LIB.define("grouped_mmq_pair_grad_input(Tensor grad0, Tensor grad1, Tensor payload0, Tensor payload1, Tensor expert_indices, "
            "Tensor expert_offsets, int quant_type, int in_features) -> Tensor")


def _flat2d(x: torch.Tensor) -> torch.Tensor:
    if x.dtype != torch.bfloat16:
        raise TypeError(f"packed GGUF products need bf16 activations, got {x.dtype}")
    if not x.is_contiguous():
        raise RuntimeError("packed GGUF products need a contiguous activation (no hidden copy is made)")
    return x.reshape(-1, x.shape[-1])


def _payload_experts(payload: torch.Tensor, qtype: int, n: int, k: int) -> int:
    per = n * ops.payload_row_bytes(qtype, k)
    if payload.numel() % per:
        raise ValueError(f"payload of {payload.numel()} bytes is not a whole number of [{n} x {k}] experts")
    return payload.numel() // per


# ---- dense -----------------------------------------------------------------------------------
def _mmq_cuda(x, payload, quant_type, out_features):
    y = ops.qlinear_fwd(_flat2d(x), payload.reshape(-1), quant_type, out_features)
    return y.reshape(*x.shape[:-1], out_features)


def _mmq_grad_input_cuda(grad_output, payload, quant_type, in_features):
    dx = ops.qlinear_dgrad(_flat2d(grad_output), payload.reshape(-1), quant_type, in_features)
    return dx.reshape(*grad_output.shape[:-1], in_features)


def _mmq_fake(x, payload, quant_type, out_features):
    return x.new_empty(*x.shape[:-1], out_features)


def _mmq_grad_input_fake(grad_output, payload, quant_type, in_features):
    return grad_output.new_empty(*grad_output.shape[:-1], in_features)


_LIB.impl("mmq", _mmq_cuda, "CUDA")
_LIB.impl("mmq_grad_input", _mmq_grad_input_cuda, "CUDA")
_LIB.impl("mmq", _mmq_fake, "Meta")
_LIB.impl("mmq_grad_input", _mmq_grad_input_fake, "Meta")


def _mmq_setup(ctx, inputs, output):
    x, payload, quant_type, out_features = inputs
    ctx.save_for_backward(payload)
    ctx.quant_type, ctx.in_features = quant_type, x.shape[-1]


def _mmq_backward(ctx, grad):
    (payload,) = ctx.saved_tensors
    dx = torch.ops.b2g.mmq_grad_input(grad.contiguous(), payload, ctx.quant_type, ctx.in_features)
    return dx, None, None, None


def _no_double_backward(ctx, *grads):
    raise RuntimeError("higher-order gradients through packed GGUF products are not supported")


torch.library.register_autograd("b2g::mmq", _mmq_backward, setup_context=_mmq_setup)
torch.library.register_autograd("b2g::mmq_grad_input", _no_double_backward)


def mmq(x: torch.Tensor, payload: torch.Tensor, quant_type: int, out_features: int) -> torch.Tensor:
    """``Y[..., N] = X[..., K] . deq(W)^T`` on a packed payload; autograd gives ``dX`` only."""
    return torch.ops.b2g.mmq(x, payload, int(quant_type), int(out_features))


def mmq_grad_input(grad_output: torch.Tensor, payload: torch.Tensor, quant_type: int, in_features: int) -> torch.Tensor:
    return torch.ops.b2g.mmq_grad_input(grad_output, payload, int(quant_type), int(in_features))


# ---- fixed groups (DeepSeek's frozen eight-group o_a_proj) ------------------------------------------
def _fixed_k(packed_groups, quant_type):
    blk, nbytes = ops._BLOCK[int(quant_type)]
    return packed_groups.shape[-1] // nbytes * blk


_LIB.impl("fixed_grouped_mmq", lambda x, pg, q: ops.fixed_grouped_fwd(x, pg, q), "CUDA")
_LIB.impl("fixed_grouped_mmq_grad_input", lambda g, pg, q: ops.fixed_grouped_dgrad(g, pg, q), "CUDA")
_LIB.impl("fixed_grouped_mmq", lambda x, pg, q: x.new_empty(*x.shape[:-1], pg.shape[1]), "Meta")
_LIB.impl("fixed_grouped_mmq_grad_input", lambda g, pg, q: g.new_empty(*g.shape[:-1], _fixed_k(pg, q)), "Meta")


def _fixed_setup(ctx, inputs, output):
    _, packed_groups, quant_type = inputs
    ctx.save_for_backward(packed_groups)
    ctx.quant_type = quant_type


def _fixed_backward(ctx, grad):
    (packed_groups,) = ctx.saved_tensors
    return torch.ops.b2g.fixed_grouped_mmq_grad_input(grad.contiguous(), packed_groups, ctx.quant_type), None, None


torch.library.register_autograd("b2g::fixed_grouped_mmq", _fixed_backward, setup_context=_fixed_setup)
torch.library.register_autograd("b2g::fixed_grouped_mmq_grad_input", _no_double_backward)


def fixed_grouped_mmq(x: torch.Tensor, packed_groups: torch.Tensor, quant_type: int = 8) -> torch.Tensor:
    """``Y[..., g, :] = X[..., g, :] . deq(W_g)^T`` for a payload ``[G, N, row bytes]``: the operator behind DeepSeek's
    frozen grouped projection (``torch_ggml_ops.fixed_grouped_mmq(input, packed_groups)``, ``deepseek_v4_lora.py:123``,
    which fixes Q8_0; the type is a third, optional argument here).  Autograd gives the input gradient only."""
    return torch.ops.b2g.fixed_grouped_mmq(x, packed_groups, int(quant_type))


class _LoraQLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, payload, quant_type, out_features, lora_a, lora_b, scaling, bias):
        x2 = _flat2d(x)
        r = lora_a.shape[0]
        a = lora_a.to(torch.bfloat16).contiguous()
        b = lora_b.to(torch.bfloat16).contiguous()
        xa, xas = ops.lora_down(x2, a, False, scaling, r)
        y = ops.qlinear_fwd(x2, payload.reshape(-1), quant_type, out_features,
                            None if bias is None else bias.to(torch.bfloat16).contiguous(), xas, ops.pad_rank_cols(b))
        ctx.save_for_backward(x2, payload, a, b, xa)
        ctx.meta = (int(quant_type), float(scaling), r, x.shape, lora_a.dtype, lora_b.dtype)
        return y.reshape(*x.shape[:-1], out_features)

    @staticmethod
    def backward(ctx, grad):
        x2, payload, a, b, xa = ctx.saved_tensors
        quant_type, scaling, r, xshape, a_dtype, b_dtype = ctx.meta
        dy = grad.contiguous().reshape(-1, grad.shape[-1])
        need_x, need_a, need_b = ctx.needs_input_grad[0], ctx.needs_input_grad[4], ctx.needs_input_grad[5]
        dyb = dybs = None
        if need_x or need_a:
            n = dy.shape[1]
            if n % 8:
                pad = (n + 7) // 8 * 8
                dy_p = dy.new_zeros(dy.shape[0], pad)
                dy_p[:, :n] = dy
                b_p = b.new_zeros(r, pad)
                b_p[:, :n] = b.t()
                dyb, dybs = ops.lora_down(dy_p, b_p, False, scaling, r)
            else:
                # B is tiny: transposing it once lets the projection stream it with the [r, C] layout
                dyb, dybs = ops.lora_down(dy, b.t().contiguous(), False, scaling, r)
        dx = da = db = None
        if need_x:
            dx = ops.qlinear_dgrad(dy, payload.reshape(-1), quant_type, x2.shape[1], dybs, ops.pad_rank_rows(a)).reshape(xshape)
        if need_a:
            da = ops.lora_wgrad(dyb, x2, scaling, r, False).to(a_dtype)
        if need_b:
            n = dy.shape[1]
            if n % 8:
                pad = (n + 7) // 8 * 8
                dy_p = dy.new_zeros(dy.shape[0], pad)
                dy_p[:, :n] = dy
                db = ops.lora_wgrad(xa, dy_p, scaling, r, True)[:n].to(b_dtype)
            else:
                db = ops.lora_wgrad(xa, dy, scaling, r, True).to(b_dtype)
        return dx, None, None, None, da, db, None, None


def lora_qlinear(x: torch.Tensor, payload: torch.Tensor, quant_type: int, out_features: int, lora_a: torch.Tensor,
                 lora_b: torch.Tensor, scaling: float, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Y = X.deq(W)^T (+bias) + scaling.(X.A^T).B^T with A [r,K], B [N,r]; one base pass each way."""
    if lora_a.shape[0] > ops.LORA_PAD:
        raise ValueError(f"the fused LoRA path supports rank <= {ops.LORA_PAD}, got {lora_a.shape[0]}")
    return _LoraQLinear.apply(x, payload, int(quant_type), int(out_features), lora_a, lora_b, float(scaling), bias)


# ---- grouped ---------------------------------------------------------------------------------
def _grouped_args(x, expert_indices, expert_offsets):
    if x.dtype != torch.bfloat16 or not x.is_contiguous() or x.ndim != 2:
        raise RuntimeError("grouped GGUF products need a contiguous bf16 [rows, features] activation")
    if expert_indices.dtype != torch.int64 or expert_offsets.dtype != torch.int32:
        raise TypeError("expert_indices must be int64 and expert_offsets int32")
    return ops.grouped_schedule(expert_indices.contiguous(), expert_offsets.contiguous(), x.shape[0])


def _grouped_mmq_cuda(x, payload, expert_indices, expert_offsets, quant_type, out_features):
    tiles = _grouped_args(x, expert_indices, expert_offsets)
    e = _payload_experts(payload, quant_type, out_features, x.shape[1])
    return ops.grouped_fwd(x, payload.reshape(-1), None, quant_type, out_features, e, tiles)


def _grouped_mmq_grad_input_cuda(g, payload, expert_indices, expert_offsets, quant_type, in_features):
    tiles = _grouped_args(g, expert_indices, expert_offsets)
    e = _payload_experts(payload, quant_type, g.shape[1], in_features)
    return ops.grouped_dgrad(g, None, payload.reshape(-1), None, quant_type, in_features, e, tiles)


def _grouped_mmq_pair_cuda(x, p0, p1, expert_indices, expert_offsets, quant_type, out_features):
    tiles = _grouped_args(x, expert_indices, expert_offsets)
    e = _payload_experts(p0, quant_type, out_features, x.shape[1])
    return ops.grouped_fwd(x, p0.reshape(-1), p1.reshape(-1), quant_type, out_features, e, tiles)


def _grouped_mmq_pair_grad_input_cuda(g0, g1, p0, p1, expert_indices, expert_offsets, quant_type, in_features):
    tiles = _grouped_args(g0, expert_indices, expert_offsets)
    e = _payload_experts(p0, quant_type, g0.shape[1], in_features)
    return ops.grouped_dgrad(g0, g1.contiguous(), p0.reshape(-1), p1.reshape(-1), quant_type, in_features, e, tiles)


_LIB.impl("grouped_mmq", _grouped_mmq_cuda, "CUDA")
_LIB.impl("grouped_mmq_grad_input", _grouped_mmq_grad_input_cuda, "CUDA")
_LIB.impl("grouped_mmq_pair", _grouped_mmq_pair_cuda, "CUDA")
_LIB.impl("grouped_mmq_pair_grad_input", _grouped_mmq_pair_grad_input_cuda, "CUDA")
_LIB.impl("grouped_mmq", lambda x, p, i, o, q, n: x.new_empty(x.shape[0], n), "Meta")
_LIB.impl("grouped_mmq_grad_input", lambda g, p, i, o, q, k: g.new_empty(g.shape[0], k), "Meta")
_LIB.impl("grouped_mmq_pair", lambda x, p0, p1, i, o, q, n: (x.new_empty(x.shape[0], n), x.new_empty(x.shape[0], n)), "Meta")
_LIB.impl("grouped_mmq_pair_grad_input", lambda g0, g1, p0, p1, i, o, q, k: g0.new_empty(g0.shape[0], k), "Meta")


def _gmmq_setup(ctx, inputs, output):
    x, payload, idx, off, quant_type, out_features = inputs
    ctx.save_for_backward(payload, idx, off)
    ctx.quant_type, ctx.in_features = quant_type, x.shape[1]


def _gmmq_backward(ctx, grad):
    payload, idx, off = ctx.saved_tensors
    dx = torch.ops.b2g.grouped_mmq_grad_input(grad.contiguous(), payload, idx, off, ctx.quant_type, ctx.in_features)
    return dx, None, None, None, None, None


def _gpair_setup(ctx, inputs, output):
    x, p0, p1, idx, off, quant_type, out_features = inputs
    ctx.save_for_backward(p0, p1, idx, off)
    ctx.quant_type, ctx.in_features = quant_type, x.shape[1]


def _gpair_backward(ctx, g0, g1):
    p0, p1, idx, off = ctx.saved_tensors
    if g0 is not None and g1 is not None:
        dx = torch.ops.b2g.grouped_mmq_pair_grad_input(g0.contiguous(), g1.contiguous(), p0, p1, idx, off, ctx.quant_type,
                                                      ctx.in_features)
    elif g0 is not None:
        dx = torch.ops.b2g.grouped_mmq_grad_input(g0.contiguous(), p0, idx, off, ctx.quant_type, ctx.in_features)
    elif g1 is not None:
        dx = torch.ops.b2g.grouped_mmq_grad_input(g1.contiguous(), p1, idx, off, ctx.quant_type, ctx.in_features)
    else:
        dx = None
    return dx, None, None, None, None, None, None


torch.library.register_autograd("b2g::grouped_mmq", _gmmq_backward, setup_context=_gmmq_setup)
torch.library.register_autograd("b2g::grouped_mmq_pair", _gpair_backward, setup_context=_gpair_setup)
torch.library.register_autograd("b2g::grouped_mmq_grad_input", _no_double_backward)
torch.library.register_autograd("b2g::grouped_mmq_pair_grad_input", _no_double_backward)


def grouped_mmq(x, payload, expert_indices, expert_offsets, quant_type, out_features):
    return torch.ops.b2g.grouped_mmq(x, payload, expert_indices, expert_offsets, int(quant_type), int(out_features))


def grouped_mmq_pair(x, payload0, payload1, expert_indices, expert_offsets, quant_type, out_features):
    return torch.ops.b2g.grouped_mmq_pair(x, payload0, payload1, expert_indices, expert_offsets, int(quant_type), int(out_features))


def expert_block_forward(sel, gate_p, up_p, down_p, quant_gu, quant_down, inter_dim, expert_indices, expert_offsets, offsets_full,
                         gu_a, gu_b, down_a, down_b, scaling, swiglu_limit):
    """Pair product + LoRA, SwiGLU, down product + LoRA over sorted expert segments: ``(out, saved)``.

    ``saved`` is what :func:`expert_block_backward` needs (selected rows, gate, up, the two rank projections and, with
    adapters, the SwiGLU output), so nothing of size [rows, hidden] is kept twice.  Plain functions, so that a caller that
    schedules its own backward (the expert-parallel layer) can use them outside an autograd node."""
    rows, hidden = sel.shape
    tiles = ops.grouped_schedule(expert_indices, expert_offsets, rows)
    e = _payload_experts(gate_p, quant_gu, inter_dim, hidden)
    has_lora = gu_a is not None
    xa = xas = za = zas = None
    r = 0
    if has_lora:
        r = gu_a.shape[1]
        xa, xas = ops.grouped_lora_down(sel, None, gu_a.contiguous(), False, scaling, r, tiles, zero=False)
        gate, up = ops.grouped_fwd(sel, gate_p.reshape(-1), up_p.reshape(-1), quant_gu, inter_dim, e, tiles, xas,
                                   ops.pad_rank_cols(gu_b))
    else:
        gate, up = ops.grouped_fwd(sel, gate_p.reshape(-1), up_p.reshape(-1), quant_gu, inter_dim, e, tiles)
    # the last cumulative end = rows that hold data; an expert-parallel receive buffer is larger than that
    live = offsets_full[-1:] if offsets_full is not None and offsets_full.numel() else None
    z = ops.swiglu_fwd(gate, up, swiglu_limit, None, live)
    if has_lora:
        za, zas = ops.grouped_lora_down(z, None, down_a.contiguous(), False, scaling, r, tiles, zero=False)
        out = ops.grouped_fwd(z, down_p.reshape(-1), None, quant_down, hidden, e, tiles, zas, ops.pad_rank_cols(down_b))
    else:
        out = ops.grouped_fwd(z, down_p.reshape(-1), None, quant_down, hidden, e, tiles)
    # z is kept for the down-projection factor gradient (rows x inter_dim bf16: small next to 180 GB, and cheaper than a
    # second pass over gate and up in the backward); without adapters nothing in the backward reads it
    tensors = (sel, gate_p, up_p, down_p, tiles, offsets_full, gate, up, xa, za, gu_a, gu_b, down_a, down_b, z if has_lora else None)
    meta = (int(quant_gu), int(quant_down), int(inter_dim), e, r, float(scaling), float(swiglu_limit), has_lora)
    return out, (tensors, meta)


def expert_block_backward(saved, d_out):
    """``(d_sel, d_gate_up_a, d_gate_up_b, d_down_a, d_down_b)`` from what :func:`expert_block_forward` saved."""
    (sel, gate_p, up_p, down_p, tiles, offsets_full, gate, up, xa, za, gu_a, gu_b, down_a, down_b, z), meta = saved
    quant_gu, quant_down, inter_dim, e, r, scaling, limit, has_lora = meta
    hidden = sel.shape[1]
    d_out = d_out.contiguous()
    d_gu_a = d_gu_b = d_down_a = d_down_b = None
    if has_lora:
        # down projection: dZ = dOut.deq(Wd) + s.(dOut.Bd).Ad ; dAd = s.(dOut.Bd)^T.Z ; dBd = s.dOut^T.(Z.Ad^T)
        dob, dobs = ops.grouped_lora_down(d_out, None, down_b.transpose(1, 2).contiguous(), False, scaling, r, tiles, zero=False)
        dz = ops.grouped_dgrad(d_out, None, down_p.reshape(-1), None, quant_down, inter_dim, e, tiles, dobs,
                               ops.pad_rank_rows(down_a))
        d_down_a = torch.empty_like(down_a)
        ops.grouped_lora_wgrad(dob, z, scaling, r, offsets_full, d_down_a, False)
        d_down_b = torch.empty_like(down_b)
        ops.grouped_lora_wgrad(za, d_out, scaling, r, offsets_full, d_down_b, True)
    else:
        dz = ops.grouped_dgrad(d_out, None, down_p.reshape(-1), None, quant_down, inter_dim, e, tiles)
    live = offsets_full[-1:] if offsets_full is not None and offsets_full.numel() else None
    d_gate, d_up = ops.swiglu_bwd(gate, up, dz, limit, None, live)
    if has_lora:
        # gate|up: dX = dG.deq(Wg) + dU.deq(Wu) + s.([dG|dU].Bgu).Agu
        dgb, dgbs = ops.grouped_lora_down(d_gate, d_up, gu_b.transpose(1, 2).contiguous(), False, scaling, r, tiles, zero=False)
        d_sel = ops.grouped_dgrad(d_gate, d_up, gate_p.reshape(-1), up_p.reshape(-1), quant_gu, hidden, e, tiles, dgbs,
                                  ops.pad_rank_rows(gu_a))
        d_gu_a = torch.empty_like(gu_a)
        ops.grouped_lora_wgrad(dgb, sel, scaling, r, offsets_full, d_gu_a, False)
        d_gu_b = torch.empty_like(gu_b)
        ops.grouped_lora_wgrad(xa, d_gate, scaling, r, offsets_full, d_gu_b, True, 0)
        ops.grouped_lora_wgrad(xa, d_up, scaling, r, offsets_full, d_gu_b, True, inter_dim)
    else:
        d_sel = ops.grouped_dgrad(d_gate, d_up, gate_p.reshape(-1), up_p.reshape(-1), quant_gu, hidden, e, tiles)
    return d_sel, d_gu_a, d_gu_b, d_down_a, d_down_b


class _GroupedLoraExperts(torch.autograd.Function):
    """The expert block (:func:`expert_block_forward` / :func:`expert_block_backward`) as one autograd node."""

    @staticmethod
    def forward(ctx, sel, gate_p, up_p, down_p, quant_gu, quant_down, inter_dim, expert_indices, expert_offsets, offsets_full,
                gu_a, gu_b, down_a, down_b, scaling, swiglu_limit):
        out, (tensors, meta) = expert_block_forward(sel, gate_p, up_p, down_p, quant_gu, quant_down, inter_dim, expert_indices,
                                                    expert_offsets, offsets_full, gu_a, gu_b, down_a, down_b, scaling, swiglu_limit)
        ctx.save_for_backward(*tensors)
        ctx.meta = meta
        return out

    @staticmethod
    def backward(ctx, d_out):
        d_sel, d_gu_a, d_gu_b, d_down_a, d_down_b = expert_block_backward((ctx.saved_tensors, ctx.meta), d_out)
        return (d_sel, None, None, None, None, None, None, None, None, None, d_gu_a, d_gu_b, d_down_a, d_down_b, None, None)


def grouped_lora_experts(sel, gate_payload, up_payload, down_payload, quant_gate_up, quant_down, inter_dim, expert_indices,
                         expert_offsets, offsets_full, gate_up_a=None, gate_up_b=None, down_a=None, down_b=None,
                         scaling: float = 1.0, swiglu_limit: float = 0.0) -> torch.Tensor:
    """Expert outputs [rows, hidden] for rows already sorted by expert.

    ``expert_indices`` / ``expert_offsets`` list the active experts and their cumulative row ends;
    ``offsets_full`` is the cumulative-end array over all experts (for the factor gradients).
    LoRA factors: gate_up_a [E,r,H], gate_up_b [E,2I,r], down_a [E,r,I], down_b [E,H,r].
    """
    return _GroupedLoraExperts.apply(sel, gate_payload, up_payload, down_payload, quant_gate_up, quant_down, inter_dim,
                                     expert_indices, expert_offsets, offsets_full, gate_up_a, gate_up_b, down_a, down_b,
                                     scaling, swiglu_limit)
