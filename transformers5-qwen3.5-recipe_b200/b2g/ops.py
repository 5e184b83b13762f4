"""Tensor-level wrappers over the libb2g C ABI.

Every function here takes CUDA tensors, allocates the outputs with torch (the library
itself allocates nothing), launches on the current torch stream and returns without
synchronising.  Arguments are validated fail-closed: wrong device, dtype or layout raises
instead of copying behind the caller's back.
"""
from __future__ import annotations

import ctypes as C
import weakref
from typing import Optional

import torch

from . import _lib

Q8_0, Q2_K, Q3_K, Q4_K, Q5_K, Q6_K, IQ2_XXS, IQ2_S = 8, 10, 11, 12, 13, 14, 16, 22
NATIVE_QUANT_TYPES = frozenset({Q8_0, Q2_K, Q3_K, Q4_K, Q5_K, Q6_K, IQ2_XXS, IQ2_S})
_BLOCK = {Q8_0: (32, 34), Q2_K: (256, 84), Q3_K: (256, 110), Q4_K: (256, 144), Q5_K: (256, 176), Q6_K: (256, 210), IQ2_XXS: (256, 66), IQ2_S: (256, 82)}
LORA_PAD = 16


def payload_row_bytes(qtype: int, k: int) -> int:
    blk, nbytes = _BLOCK[int(qtype)]
    if k % blk:
        raise ValueError(f"K={k} is not a multiple of the {blk}-value block of GGML type {qtype}")
    return k // blk * nbytes


def _p(t: Optional[torch.Tensor]):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream(t: torch.Tensor):
    return C.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _need(t: torch.Tensor, dtype: torch.dtype, what: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{what} must be a CUDA tensor (this package has no CPU path)")
    if t.dtype != dtype:
        raise TypeError(f"{what} must be {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise RuntimeError(f"{what} must be contiguous")


class _DeviceCtx:
    """Make the tensor's device current for the duration of a launch."""

    def __init__(self, t: torch.Tensor):
        self.guard = torch.cuda.device(t.device)

    def __enter__(self):
        self.guard.__enter__()

    def __exit__(self, *exc):
        return self.guard.__exit__(*exc)


# --------------------------------------------------------------------------------------
# per-device state: status word (set by a kernel whose bounded wait ran out), IQ2_XXS table
# --------------------------------------------------------------------------------------
_status: dict[int, torch.Tensor] = {}
_grid_done: set[int] = set()


def status_word(device: torch.device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _status:
        _status[idx] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
    return _status[idx]


def check_status(device: Optional[torch.device] = None) -> None:
    """Synchronise and raise if any kernel on the device reported a problem through the status word: a bounded wait that
    ran out (sites 1xx-4xx), a receive buffer too small for an expert-parallel exchange (901), a label outside the
    vocabulary in the cross-entropy kernel (902), an expert id outside the expert count in the routing plan (903), expert
    offsets beyond the rows of a grouped product (904)."""
    devs = [device.index if device is not None and device.index is not None else torch.cuda.current_device()] \
        if device is not None else list(_status)
    for idx in devs:
        if idx in _status:
            code = int(_status[idx].item())
            if code:
                _status[idx].zero_()
                what = {901: "an expert-parallel receive buffer was too small (rows beyond it were dropped)",
                        902: "a cross-entropy target was outside the vocabulary",
                        903: "an expert id was outside the expert count (its route was dropped)",
                        904: "expert offsets reached beyond the rows of a grouped product (they were clamped)"}.get(
                    code, "a libb2g kernel gave up a bounded wait")
                raise _lib.B2GError(f"{what} on cuda:{idx} (status {code})")


def ensure_iq2xxs_grid(device: torch.device) -> None:
    """Upload the IQ2_XXS magnitude table, read from the installed gguf package, once per device."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx in _grid_done:
        return
    import numpy as np
    from gguf import quants as gq

    gq.IQ2_XXS.init_grid()
    grid = np.ascontiguousarray(np.asarray(gq.IQ2_XXS.grid, dtype=np.float32).reshape(256, 8).astype(np.uint8))
    with torch.cuda.device(idx):
        _lib.call("b2g_set_iq2xxs_grid", C.c_void_p(grid.ctypes.data))
    _grid_done.add(idx)


_grid_s_done: set[int] = set()


def ensure_iq2s_grid(device: torch.device) -> None:
    """The same for IQ2_S and its 1024-row table."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx in _grid_s_done:
        return
    import numpy as np
    from gguf import quants as gq

    gq.IQ2_S.init_grid()
    grid = np.ascontiguousarray(np.asarray(gq.IQ2_S.grid, dtype=np.float32).reshape(1024, 8).astype(np.uint8))
    with torch.cuda.device(idx):
        _lib.call("b2g_set_iq2s_grid", C.c_void_p(grid.ctypes.data))
    _grid_s_done.add(idx)


def _check_payload(payload: torch.Tensor, qtype: int, rows: int, k: int, what: str) -> None:
    _need(payload, torch.uint8, what)
    if int(qtype) not in NATIVE_QUANT_TYPES:
        raise ValueError(f"GGML type {qtype} is not supported natively (supported: 8 Q8_0, 10 Q2_K, 11 Q3_K, 12 Q4_K, 13 Q5_K, 14 Q6_K, 16 IQ2_XXS, 22 IQ2_S)")
    want = rows * payload_row_bytes(qtype, k)
    if payload.numel() != want:
        raise ValueError(f"{what} holds {payload.numel()} bytes, expected {want} for {rows} x {k} of type {qtype}")
    if payload.storage_offset() != 0 and payload.data_ptr() % 16:
        raise RuntimeError(f"{what} must be 16-byte aligned")
    if int(qtype) == IQ2_XXS:
        ensure_iq2xxs_grid(payload.device)
    if int(qtype) == IQ2_S:
        ensure_iq2s_grid(payload.device)


PADDED_ROWS = 0x100     # B2G_PADDED_ROWS: flag on the type id, "payload rows are padded to a multiple of 16 bytes"


# Padded copies of frozen payloads whose rows are not 16-byte multiples, made ONCE per payload and kept for as long as the
# payload itself lives: key = (storage address, byte count, tensor version), value = (weak reference to the payload's
# storage owner, padded copy).  A frozen weight is padded on its first product and never again.
_padded: dict[tuple[int, int, int], tuple[weakref.ref, torch.Tensor]] = {}


def pad_payload_rows(payload: torch.Tensor, qtype: int, rows: int, k: int) -> torch.Tensor:
    """``payload`` copied into rows padded to the next multiple of 16 bytes (what ``B2G_PADDED_ROWS`` announces)."""
    pitch = payload_row_bytes(qtype, k)
    padded = (pitch + 15) // 16 * 16
    out = torch.zeros(rows, padded, dtype=torch.uint8, device=payload.device)
    out[:, :pitch] = payload.reshape(rows, pitch)
    return out.reshape(-1)


def _tma_payload(payload: torch.Tensor, qtype: int, rows: int, k: int):
    """The payload as the matrix-product kernels take it, and the type argument to pass with it.

    TMA needs row pitches that are multiples of 16 bytes.  Q4_K, Q5_K and Q8_0 rows always are; the other formats' rows
    only for some widths (a 512-wide IQ2_XXS row is 132 bytes).  Such a payload is copied into padded rows the first time
    a product sees it; the copy is cached beside the (frozen) payload and reused by every later forward and backward, so
    no call after the first moves or allocates packed bytes.  A payload that was modified in place (its version counter
    moved) is padded again."""
    pitch = payload_row_bytes(qtype, k)
    if pitch % 16 == 0:
        return payload, int(qtype)
    key = (payload.data_ptr(), payload.numel(), payload._version)
    hit = _padded.get(key)
    if hit is not None and hit[0]() is not None:
        return hit[1], int(qtype) | PADDED_ROWS
    for stale in [kk for kk, (ref, _) in _padded.items() if ref() is None]:
        del _padded[stale]
    out = pad_payload_rows(payload, qtype, rows, k)
    _padded[key] = (weakref.ref(payload.untyped_storage()), out)
    return out, int(qtype) | PADDED_ROWS


# --------------------------------------------------------------------------------------
# dequantise
# --------------------------------------------------------------------------------------
def dequantize(payload: torch.Tensor, qtype: int, logical_shape: tuple[int, ...]) -> torch.Tensor:
    """Packed uint8 payload -> logical bf16 tensor of ``logical_shape`` (last dim = K)."""
    k = int(logical_shape[-1])
    rows = 1
    for d in logical_shape[:-1]:
        rows *= int(d)
    _check_payload(payload, qtype, rows, k, "payload")
    out = torch.empty(logical_shape, dtype=torch.bfloat16, device=payload.device)
    with _DeviceCtx(payload):
        _lib.call("b2g_dequant", int(qtype), _p(payload), rows, k, _p(out), _stream(payload))
    return out


# --------------------------------------------------------------------------------------
# LoRA rank-side helpers
# --------------------------------------------------------------------------------------
def pad_rank_cols(b: torch.Tensor) -> torch.Tensor:
    """[..., N, r] -> [..., N, 16] (zero padded); a no-op view when r == 16."""
    if b.shape[-1] == LORA_PAD:
        return b.contiguous()
    out = b.new_zeros(*b.shape[:-1], LORA_PAD)
    out[..., : b.shape[-1]] = b
    return out


def pad_rank_rows(a: torch.Tensor) -> torch.Tensor:
    """[..., r, K] -> [..., 16, K] (zero padded); a no-op view when r == 16."""
    if a.shape[-2] == LORA_PAD:
        return a.contiguous()
    out = a.new_zeros(*a.shape[:-2], LORA_PAD, a.shape[-1])
    out[..., : a.shape[-2], :] = a
    return out


def lora_down(x: torch.Tensor, w: torch.Tensor, w_is_cr: bool, scale: float, r: int,
              plain: bool = True, scaled: bool = True) -> tuple[Optional[torch.Tensor], Optional[torch.Tensor]]:
    """P = X . W^T onto the LoRA rank.  Returns ([M,16] bf16(P), [M,16] bf16(scale*P))."""
    _need(x, torch.bfloat16, "x")
    _need(w, torch.bfloat16, "w")
    m, c = x.shape
    if tuple(w.shape) != ((c, r) if w_is_cr else (r, c)):
        raise ValueError(f"weight shape {tuple(w.shape)} does not match C={c}, r={r}, w_is_cr={w_is_cr}")
    o_plain = torch.empty(m, LORA_PAD, dtype=torch.bfloat16, device=x.device) if plain else None
    o_scaled = torch.empty(m, LORA_PAD, dtype=torch.bfloat16, device=x.device) if scaled else None
    with _DeviceCtx(x):
        _lib.call("b2g_lora_down", _p(x), _p(w), int(w_is_cr), float(scale), _p(o_plain), _p(o_scaled), m, c, int(r), _stream(x))
    return o_plain, o_scaled


def lora_wgrad(s16: torch.Tensor, t: torch.Tensor, scale: float, r: int, transpose_out: bool) -> torch.Tensor:
    """scale * S[:, :r]^T . T as [r, C] or, transposed, [C, r]."""
    _need(s16, torch.bfloat16, "s")
    _need(t, torch.bfloat16, "t")
    m, c = t.shape
    if tuple(s16.shape) != (m, LORA_PAD):
        raise ValueError(f"s must be [{m}, 16], got {tuple(s16.shape)}")
    out = torch.empty((c, r) if transpose_out else (r, c), dtype=torch.bfloat16, device=t.device)
    if m == 0:
        return out.zero_()
    nbytes = _lib.query("b2g_lora_wgrad_workspace_bytes", m, c)
    ws = torch.empty(nbytes // 4, dtype=torch.float32, device=t.device)
    with _DeviceCtx(t):
        _lib.call("b2g_lora_wgrad", _p(s16), _p(t), float(scale), _p(out), int(transpose_out), _p(ws), nbytes, m, c, int(r), _stream(t))
    return out


# --------------------------------------------------------------------------------------
# dense quantized linear
# --------------------------------------------------------------------------------------
def qlinear_fwd(x: torch.Tensor, payload: torch.Tensor, qtype: int, n: int, bias: Optional[torch.Tensor] = None,
                xas: Optional[torch.Tensor] = None, lora_b16: Optional[torch.Tensor] = None) -> torch.Tensor:
    _need(x, torch.bfloat16, "x")
    m, k = x.shape
    _check_payload(payload, qtype, n, k, "payload")
    if bias is not None:
        _need(bias, torch.bfloat16, "bias")
    if xas is not None:
        _need(xas, torch.bfloat16, "xas")
        _need(lora_b16, torch.bfloat16, "lora_b16")
        if tuple(xas.shape) != (m, LORA_PAD) or tuple(lora_b16.shape) != (n, LORA_PAD):
            raise ValueError("LoRA operands must be [M,16] and [N,16]")
    y = torch.empty(m, n, dtype=torch.bfloat16, device=x.device)
    payload, qarg = _tma_payload(payload, qtype, n, k)
    with _DeviceCtx(x):
        _lib.call("b2g_qlinear_fwd", qarg, _p(x), _p(payload), _p(bias), _p(xas), _p(lora_b16), _p(y), m, n, k,
                  _p(status_word(x.device)), _stream(x))
    return y


def cross_entropy_inplace(logits: torch.Tensor, target: torch.Tensor, loss: torch.Tensor, count: Optional[torch.Tensor], mean: bool,
                          ignore_index: int = -100, predicted: Optional[torch.Tensor] = None,
                          correct: Optional[torch.Tensor] = None) -> None:
    """Cross-entropy of bf16 ``logits [rows, V]`` against ``target [rows]``: ``loss [rows]`` (fp32) is written and the logits
    are overwritten by their cotangent (softmax - onehot) / count (mean) or (softmax - onehot) (sum).  ``count`` is a
    one-element int64 device tensor holding the number of non-ignored targets of the whole batch."""
    _need(logits, torch.bfloat16, "logits")
    _need(target, torch.int64, "target")
    _need(loss, torch.float32, "loss")
    rows, v = logits.shape
    if logits.stride(1) != 1 or target.shape != (rows,) or loss.shape != (rows,) or not target.is_contiguous() or not loss.is_contiguous():
        raise ValueError("cross_entropy_inplace: logits [rows, V] with unit column stride, target and loss [rows], contiguous")
    if mean:
        _need(count, torch.int64, "count")
    for name, t, dt in (("predicted", predicted, torch.int64), ("correct", correct, torch.float32)):
        if t is not None:
            _need(t, dt, name)
            if t.shape != (rows,) or not t.is_contiguous():
                raise ValueError(f"cross_entropy_inplace: {name} must be a contiguous [rows] tensor")
    with _DeviceCtx(logits):
        _lib.call("b2g_cross_entropy_inplace", _p(logits), logits.stride(0), _p(target), _p(loss), _p(predicted), _p(correct), rows, v,
                  int(ignore_index), _p(count) if mean else None, int(bool(mean)), _p(status_word(logits.device)), _stream(logits))


def _fixed_group_geometry(a: torch.Tensor, payload: torch.Tensor, qtype: int, forward: bool):
    """Shapes of the fixed-group product: activations [..., G, width] (contiguous), payload [G, N, row bytes]."""
    _need(a, torch.bfloat16, "activation")
    _need(payload, torch.uint8, "packed_groups")
    if a.dim() < 2 or payload.dim() != 3:
        raise ValueError("fixed groups need activations [..., G, width] and a payload [G, N, row bytes]")
    if not a.is_contiguous():
        raise RuntimeError("fixed-group products need a contiguous activation (no hidden copy is made)")
    groups, n, row_bytes = payload.shape
    if a.shape[-2] != groups:
        raise ValueError(f"activation has {a.shape[-2]} groups, the payload {groups}")
    block_values, block_bytes = _BLOCK[int(qtype)] if int(qtype) in NATIVE_QUANT_TYPES else (0, 0)
    if not block_values:
        raise ValueError(f"GGML type {qtype} is not supported natively (supported: 8 Q8_0, 10 Q2_K, 11 Q3_K, 12 Q4_K, 13 Q5_K, 14 Q6_K, 16 IQ2_XXS, 22 IQ2_S)")
    if row_bytes % block_bytes:
        raise ValueError(f"payload rows of {row_bytes} bytes are not whole blocks of type {qtype}")
    k = row_bytes // block_bytes * block_values
    width = a.shape[-1]
    if width != (k if forward else n):
        raise ValueError(f"activation width {width} does not match the payload ({k if forward else n} expected)")
    _check_payload(payload, qtype, groups * n, k, "packed_groups")
    m = a.numel() // (groups * width)
    return m, groups, n, k


def fixed_grouped_fwd(x: torch.Tensor, packed_groups: torch.Tensor, qtype: int) -> torch.Tensor:
    """Y[..., g, :] = X[..., g, :] . deq(W_g)^T for every group, in place on column blocks (no per-group copies)."""
    m, groups, n, k = _fixed_group_geometry(x, packed_groups, qtype, True)
    y = torch.empty(*x.shape[:-1], n, dtype=torch.bfloat16, device=x.device)
    packed_groups, qarg = _tma_payload(packed_groups, qtype, groups * n, k)
    with _DeviceCtx(x):
        _lib.call("b2g_fixed_grouped_fwd", qarg, _p(x), _p(packed_groups), _p(y), m, groups, n, k, _p(status_word(x.device)), _stream(x))
    return y


def fixed_grouped_dgrad(dy: torch.Tensor, packed_groups: torch.Tensor, qtype: int) -> torch.Tensor:
    """dX[..., g, :] = dY[..., g, :] . deq(W_g) for every group."""
    m, groups, n, k = _fixed_group_geometry(dy, packed_groups, qtype, False)
    dx = torch.empty(*dy.shape[:-1], k, dtype=torch.bfloat16, device=dy.device)
    packed_groups, qarg = _tma_payload(packed_groups, qtype, groups * n, k)
    with _DeviceCtx(dy):
        _lib.call("b2g_fixed_grouped_dgrad", qarg, _p(dy), _p(packed_groups), _p(dx), m, groups, n, k, _p(status_word(dy.device)),
                  _stream(dy))
    return dx


def qlinear_dgrad(dy: torch.Tensor, payload: torch.Tensor, qtype: int, k: int,
                  dybs: Optional[torch.Tensor] = None, lora_a16: Optional[torch.Tensor] = None) -> torch.Tensor:
    _need(dy, torch.bfloat16, "dy")
    m, n = dy.shape
    _check_payload(payload, qtype, n, k, "payload")
    if n % 8:
        # TMA needs a 16-byte row pitch; rows of odd width are zero-padded (the extra columns meet
        # zero-filled weight rows, so the product is unchanged).
        n_pad = (n + 7) // 8 * 8
        dyp = dy.new_zeros(m, n_pad)
        dyp[:, :n] = dy
        pitch = payload_row_bytes(qtype, k)
        pp = payload.new_zeros(n_pad * pitch)
        pp[: n * pitch] = payload.reshape(-1)
        return qlinear_dgrad(dyp, pp, qtype, k, dybs, lora_a16)
    if dybs is not None:
        _need(dybs, torch.bfloat16, "dybs")
        _need(lora_a16, torch.bfloat16, "lora_a16")
        if tuple(dybs.shape) != (m, LORA_PAD) or tuple(lora_a16.shape) != (LORA_PAD, k):
            raise ValueError("LoRA operands must be [M,16] and [16,K]")
    dx = torch.empty(m, k, dtype=torch.bfloat16, device=dy.device)
    payload, qarg = _tma_payload(payload, qtype, n, k)
    with _DeviceCtx(dy):
        _lib.call("b2g_qlinear_dgrad", qarg, _p(dy), _p(payload), _p(dybs), _p(lora_a16), _p(dx), m, n, k,
                  _p(status_word(dy.device)), _stream(dy))
    return dx


# --------------------------------------------------------------------------------------
# router / routing
# --------------------------------------------------------------------------------------
def router_topk(logits: torch.Tensor, top_k: int, bias: Optional[torch.Tensor], sqrt_softplus: bool) -> torch.Tensor:
    if logits.dtype not in (torch.bfloat16, torch.float32):
        raise RuntimeError("router logits must be bf16 or fp32")
    _need(logits, logits.dtype, "logits")
    t, e = logits.shape
    if bias is not None:
        bias = bias.to(device=logits.device, dtype=torch.float32).contiguous()
    out = torch.empty(t, top_k, dtype=torch.int64, device=logits.device)
    with _DeviceCtx(logits):
        _lib.call("b2g_router_topk", _p(logits), int(logits.dtype == torch.float32), _p(bias), int(sqrt_softplus), _p(out),
                  t, e, int(top_k), _stream(logits))
    return out


def route_plan(top_k_index: torch.Tensor, num_experts: int = 256):
    """Stable sort of the flat expert ids: (sorted_expert, perm, inv_perm, group_sizes, offsets)."""
    if top_k_index.dtype not in (torch.int32, torch.int64):
        raise RuntimeError("expert indices must be int32 or int64")
    _need(top_k_index, top_k_index.dtype, "top_k_index")
    t, k = top_k_index.shape
    r = t * k
    dev = top_k_index.device
    # zero-filled: a route whose expert id is out of range is dropped by the kernel (status 903), and its slots must still
    # hold indices that the permute kernels can follow without leaving their tensors
    triple = torch.zeros(3, r, dtype=torch.int64, device=dev)
    sorted_e, perm, inv = triple[0], triple[1], triple[2]
    sizes = torch.empty(num_experts, dtype=torch.int32, device=dev)
    offsets = torch.empty(num_experts, dtype=torch.int32, device=dev)
    nbytes = _lib.query("b2g_route_plan_workspace_bytes", r, num_experts)
    ws = torch.empty((nbytes + 3) // 4, dtype=torch.int32, device=dev)
    with _DeviceCtx(top_k_index):
        _lib.call("b2g_route_plan", _p(top_k_index), int(top_k_index.dtype == torch.int64), t, k, num_experts, _p(sorted_e),
                  _p(perm), _p(inv), _p(sizes), _p(offsets), _p(ws), nbytes, _p(status_word(dev)), _stream(top_k_index))
    return sorted_e, perm, inv, sizes, offsets


def route_gather(hidden: torch.Tensor, perm: torch.Tensor, top_k: int) -> torch.Tensor:
    _need(hidden, torch.bfloat16, "hidden")
    _need(perm, torch.int64, "perm")
    t, h = hidden.shape
    out = torch.empty(perm.numel(), h, dtype=torch.bfloat16, device=hidden.device)
    with _DeviceCtx(hidden):
        _lib.call("b2g_route_gather", _p(hidden), _p(perm), _p(out), t, int(top_k), h, _stream(hidden))
    return out


def route_gather_bwd(grad_sel: torch.Tensor, inv: torch.Tensor, num_tokens: int, top_k: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _need(grad_sel, torch.bfloat16, "grad_selected")
    _need(inv, torch.int64, "inverse_permutation")
    h = grad_sel.shape[1]
    if out is None:
        out = torch.empty(num_tokens, h, dtype=torch.bfloat16, device=grad_sel.device)
    else:
        _need(out, torch.bfloat16, "out")
    with _DeviceCtx(grad_sel):
        _lib.call("b2g_route_gather_bwd", _p(grad_sel), _p(inv), _p(out), num_tokens, int(top_k), h, _stream(grad_sel))
    return out


def _wdtype(w: torch.Tensor) -> int:
    if w.dtype not in (torch.bfloat16, torch.float32):
        raise RuntimeError("routing weights must be bf16 or fp32")
    return int(w.dtype == torch.float32)


def route_combine(expert_out: torch.Tensor, weights: torch.Tensor, inv: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _need(expert_out, torch.bfloat16, "expert_out")
    _need(weights, weights.dtype, "routing_weights")
    _need(inv, torch.int64, "inverse_permutation")
    t, k = weights.shape
    h = expert_out.shape[1]
    if out is None:
        out = torch.empty(t, h, dtype=torch.bfloat16, device=expert_out.device)
    else:
        _need(out, torch.bfloat16, "out")
    with _DeviceCtx(expert_out):
        _lib.call("b2g_route_combine", _p(expert_out), _p(weights), _wdtype(weights), _p(inv), _p(out), t, k, h, _stream(expert_out))
    return out


def route_combine_bwd(expert_out: torch.Tensor, weights: torch.Tensor, perm: torch.Tensor, grad_final: torch.Tensor):
    _need(expert_out, torch.bfloat16, "expert_out")
    _need(grad_final, torch.bfloat16, "grad_final")
    _need(weights, weights.dtype, "routing_weights")
    _need(perm, torch.int64, "permutation")
    t, k = weights.shape
    h = expert_out.shape[1]
    d_out = torch.empty_like(expert_out)
    d_w = torch.empty_like(weights)
    with _DeviceCtx(expert_out):
        _lib.call("b2g_route_combine_bwd", _p(expert_out), _p(weights), _wdtype(weights), _p(perm), _p(grad_final), _p(d_out),
                  _p(d_w), t, k, h, _stream(expert_out))
    return d_out, d_w


def swiglu_fwd(gate: torch.Tensor, up: torch.Tensor, limit: float = 0.0, row_begin: Optional[torch.Tensor] = None,
               row_end: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``silu(gate) * up`` (clamped when ``limit > 0``).  ``row_begin`` / ``row_end``: one-element int32 device tensors; only the
    rows in between are computed (the rest of ``out`` is left untouched)."""
    _need(gate, torch.bfloat16, "gate")
    _need(up, torch.bfloat16, "up")
    z = torch.empty_like(gate) if out is None else out
    with _DeviceCtx(gate):
        _lib.call("b2g_swiglu_fwd", _p(gate), _p(up), _p(z), gate.numel(), float(limit), _p(row_begin), _p(row_end), gate.shape[-1], _stream(gate))
    return z


def swiglu_bwd(gate: torch.Tensor, up: torch.Tensor, dz: torch.Tensor, limit: float = 0.0, row_begin: Optional[torch.Tensor] = None,
               row_end: Optional[torch.Tensor] = None, out: Optional[tuple[torch.Tensor, torch.Tensor]] = None):
    _need(dz, torch.bfloat16, "dz")
    dg, du = (torch.empty_like(gate), torch.empty_like(up)) if out is None else out
    with _DeviceCtx(gate):
        _lib.call("b2g_swiglu_bwd", _p(gate), _p(up), _p(dz), _p(dg), _p(du), gate.numel(), float(limit), _p(row_begin), _p(row_end),
                  gate.shape[-1], _stream(gate))
    return dg, du


# --------------------------------------------------------------------------------------
# grouped (MoE) path
# --------------------------------------------------------------------------------------
def grouped_schedule(expert_indices: torch.Tensor, offsets: torch.Tensor, total_rows: int, first_row: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Tile table (int32 scratch) for the active experts ``expert_indices`` with cumulative ends ``offsets``; ``first_row`` (a
    one-element int32 device tensor) is where the first listed expert's rows begin when that is not row 0."""
    _need(expert_indices, torch.int64, "expert_indices")
    _need(offsets, torch.int32, "expert_offsets")
    g = expert_indices.numel()
    if offsets.numel() != g:
        raise ValueError("expert_indices and expert_offsets must have the same length")
    nbytes = _lib.query("b2g_grouped_tiles_bytes", total_rows, g)
    tiles = torch.empty(nbytes // 4, dtype=torch.int32, device=offsets.device)
    with _DeviceCtx(offsets):
        _lib.call("b2g_grouped_schedule", _p(expert_indices), _p(offsets), _p(first_row), g, total_rows, _p(tiles),
                  _p(status_word(offsets.device)), _stream(offsets))
    return tiles


def grouped_fwd(x: torch.Tensor, payload0: torch.Tensor, payload1: Optional[torch.Tensor], qtype: int, n: int, num_experts: int,
                tiles: torch.Tensor, xas: Optional[torch.Tensor] = None, lora_b16: Optional[torch.Tensor] = None,
                out0: Optional[torch.Tensor] = None, out1: Optional[torch.Tensor] = None):
    """Grouped Y = X . deq(W_e)^T for one payload, or (Y0, Y1) for two.  ``lora_b16`` is [E, rows, 16]
    with rows = n (single) or 2n (pair: first n rows for Y0, next n for Y1)."""
    _need(x, torch.bfloat16, "x")
    r, k = x.shape
    _check_payload(payload0, qtype, num_experts * n, k, "payload")
    if payload1 is not None:
        _check_payload(payload1, qtype, num_experts * n, k, "second payload")
    lora_rows = 0
    if xas is not None:
        _need(xas, torch.bfloat16, "xas")
        _need(lora_b16, torch.bfloat16, "lora_b16")
        lora_rows = lora_b16.shape[1]
        if tuple(xas.shape) != (r, LORA_PAD) or lora_b16.shape[0] != num_experts or lora_b16.shape[2] != LORA_PAD \
                or lora_rows != n * (2 if payload1 is not None else 1):
            raise ValueError("bad LoRA operand shapes for the grouped forward")
    y0 = torch.empty(r, n, dtype=torch.bfloat16, device=x.device) if out0 is None else out0
    y1 = (torch.empty(r, n, dtype=torch.bfloat16, device=x.device) if out1 is None else out1) if payload1 is not None else None
    for t in (y0, y1):
        if t is not None and (t.dtype != torch.bfloat16 or tuple(t.shape) != (r, n) or not t.is_contiguous()):
            raise ValueError("grouped_fwd: an output buffer must be a contiguous bf16 [rows, n] tensor")
    payload0, qarg = _tma_payload(payload0, qtype, num_experts * n, k)
    if payload1 is not None:
        payload1, _ = _tma_payload(payload1, qtype, num_experts * n, k)
    with _DeviceCtx(x):
        _lib.call("b2g_grouped_fwd", qarg, _p(x), _p(payload0), _p(payload1), _p(tiles), _p(xas), _p(lora_b16), lora_rows,
                  _p(y0), _p(y1), r, n, k, int(num_experts), _p(status_word(x.device)), _stream(x))
    return (y0, y1) if payload1 is not None else y0


def grouped_dgrad(dy0: torch.Tensor, dy1: Optional[torch.Tensor], payload0: torch.Tensor, payload1: Optional[torch.Tensor],
                  qtype: int, k: int, num_experts: int, tiles: torch.Tensor, dybs: Optional[torch.Tensor] = None,
                  lora_a16: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _need(dy0, torch.bfloat16, "dy")
    r, n = dy0.shape
    _check_payload(payload0, qtype, num_experts * n, k, "payload")
    if payload1 is not None:
        _need(dy1, torch.bfloat16, "second dy")
        _check_payload(payload1, qtype, num_experts * n, k, "second payload")
    if dybs is not None:
        _need(dybs, torch.bfloat16, "dybs")
        _need(lora_a16, torch.bfloat16, "lora_a16")
        if tuple(dybs.shape) != (r, LORA_PAD) or tuple(lora_a16.shape) != (num_experts, LORA_PAD, k):
            raise ValueError("bad LoRA operand shapes for the grouped input gradient")
    dx = torch.empty(r, k, dtype=torch.bfloat16, device=dy0.device) if out is None else out
    if dx.dtype != torch.bfloat16 or tuple(dx.shape) != (r, k) or not dx.is_contiguous():
        raise ValueError("grouped_dgrad: the output buffer must be a contiguous bf16 [rows, k] tensor")
    payload0, qarg = _tma_payload(payload0, qtype, num_experts * n, k)
    if payload1 is not None:
        payload1, _ = _tma_payload(payload1, qtype, num_experts * n, k)
    with _DeviceCtx(dy0):
        _lib.call("b2g_grouped_dgrad", qarg, _p(dy0), _p(dy1), _p(payload0), _p(payload1), _p(tiles), _p(dybs), _p(lora_a16),
                  _p(dx), r, n, k, int(num_experts), _p(status_word(dy0.device)), _stream(dy0))
    return dx


def grouped_lora_down(x: torch.Tensor, x1: Optional[torch.Tensor], w: torch.Tensor, w_is_cr: bool, scale: float, r: int,
                      tiles: torch.Tensor, plain: bool = True, scaled: bool = True, zero: bool = True,
                      out: Optional[tuple[Optional[torch.Tensor], Optional[torch.Tensor]]] = None):
    """Per-expert projection onto the rank.  ``w`` is [E, r, C] or (w_is_cr) [E, C(or 2C), r].
    The kernel writes only rows that belong to a tile of the table, so the outputs start zeroed unless the caller says that
    nobody reads the other rows (``zero=False``: the fused expert block, whose consumers walk the same table)."""
    _need(x, torch.bfloat16, "x")
    _need(w, torch.bfloat16, "w")
    rows, c = x.shape
    e = w.shape[0]
    make = torch.zeros if zero else torch.empty
    if out is not None:
        o_plain, o_scaled = out
    else:
        o_plain = make(rows, LORA_PAD, dtype=torch.bfloat16, device=x.device) if plain else None
        o_scaled = make(rows, LORA_PAD, dtype=torch.bfloat16, device=x.device) if scaled else None
    with _DeviceCtx(x):
        _lib.call("b2g_grouped_lora_down", _p(x), _p(x1), _p(w), int(w_is_cr), float(scale), _p(tiles), _p(o_plain), _p(o_scaled),
                  rows, c, int(r), int(e), _stream(x))
    return o_plain, o_scaled


def grouped_lora_wgrad(s16: torch.Tensor, t: torch.Tensor, scale: float, r: int, offsets_full: torch.Tensor, out: torch.Tensor,
                       transpose_out: bool, out_col_offset: int = 0, first_row: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Per-expert factor gradient into ``out`` ([E, r, Ctot] or, transposed, [E, Ctot, r])."""
    _need(s16, torch.bfloat16, "s")
    _need(t, torch.bfloat16, "t")
    _need(offsets_full, torch.int32, "offsets")
    _need(out, torch.bfloat16, "out")
    rows, c = t.shape
    e = offsets_full.numel()
    ctot = out.shape[1] if transpose_out else out.shape[2]
    with _DeviceCtx(t):
        _lib.call("b2g_grouped_lora_wgrad", _p(s16), _p(t), float(scale), _p(offsets_full), _p(first_row), _p(out), int(transpose_out), rows, c,
                  int(r), int(e), int(out_col_offset), int(ctot), _stream(t))
    return out


def grouped_lora_up(p: torch.Tensor, w: torch.Tensor, w_is_nr: bool, offsets_full: torch.Tensor) -> torch.Tensor:
    """Y[rows_e, N] = P[rows_e, :r] . W[e]^T; ``p`` is [R, >=r] (row stride taken from the tensor),
    ``w`` is [E, N, r] (w_is_nr) or [E, r, N]."""
    _need(w, torch.bfloat16, "w")
    _need(offsets_full, torch.int32, "offsets")
    if p.dtype != torch.bfloat16 or not p.is_cuda or p.stride(1) != 1:
        raise RuntimeError("p must be a CUDA bf16 matrix with unit column stride")
    e = w.shape[0]
    n, r = (w.shape[1], w.shape[2]) if w_is_nr else (w.shape[2], w.shape[1])
    y = torch.empty(p.shape[0], n, dtype=torch.bfloat16, device=p.device)
    with _DeviceCtx(p):
        _lib.call("b2g_grouped_lora_up", _p(p), p.stride(0), _p(w), int(w_is_nr), _p(offsets_full), _p(y), p.shape[0], n, int(r),
                  int(e), _stream(p))
    return y
