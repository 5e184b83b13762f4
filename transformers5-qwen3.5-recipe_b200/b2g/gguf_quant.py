"""GGUF block encoders in PyTorch (run on the GPU or the CPU), for building packed weights.

The reference repository loads packed payloads from GGUF files and never encodes; these
encoders exist so that synthetic weights of a benchmark configuration (W ~ N(0, 0.02)) can be
brought into the on-disk block layout that the kernels consume.  Layouts follow the public
GGUF format: Q8_0 = fp16 d + 32 int8; Q4_K = fp16 d, fp16 dmin, 12 bytes of 6-bit
(scale, min) pairs, 128 nibble bytes; IQ2_XXS = fp16 d + 8 x (4 grid indices, u32 of
4 x 7-bit sign indices + 4-bit sub-scale).
"""
from __future__ import annotations

import torch


def _round_half_away(x: torch.Tensor) -> torch.Tensor:
    return torch.sign(x) * torch.floor(x.abs() + 0.5)


def _f16_bytes(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.float16).contiguous().view(torch.uint8)


def quantize_q8_0(w: torch.Tensor) -> torch.Tensor:
    """float [..., K] -> uint8 [..., K/32*34]; d = absmax/127, q = round(x/d)."""
    *lead, k = w.shape
    x = w.float().reshape(-1, 32)
    d = x.abs().amax(dim=1, keepdim=True) / 127.0
    inv = torch.where(d == 0, torch.zeros_like(d), 1.0 / d)
    q = _round_half_away(x * inv).to(torch.int8)
    out = torch.empty(x.shape[0], 34, dtype=torch.uint8, device=w.device)
    out[:, :2] = _f16_bytes(d).reshape(-1, 2)
    out[:, 2:] = q.view(torch.uint8)
    return out.reshape(*lead, k // 32 * 34)


def quantize_q4_k(w: torch.Tensor) -> torch.Tensor:
    """float [..., K] -> uint8 [..., K/256*144]; affine 4-bit per 32 values, 6-bit scales/mins per 256."""
    *lead, k = w.shape
    x = w.float().reshape(-1, 8, 32)
    n = x.shape[0]
    lo = x.amin(dim=2).clamp(max=0)
    hi = torch.maximum(x.amax(dim=2), lo)
    scale = (hi - lo) / 15.0
    off = -lo
    d = (scale.amax(dim=1, keepdim=True) / 63.0).to(torch.float16)
    dmin = (off.amax(dim=1, keepdim=True) / 63.0).to(torch.float16)
    d32, dmin32 = d.float(), dmin.float()
    sc = torch.where(d32 > 0, _round_half_away(scale / d32.clamp(min=1e-30)), torch.zeros_like(scale)).clamp(0, 63).to(torch.uint8)
    mn = torch.where(dmin32 > 0, _round_half_away(off / dmin32.clamp(min=1e-30)), torch.zeros_like(off)).clamp(0, 63).to(torch.uint8)
    dsc = (d32 * sc.float()).unsqueeze(2)
    dm = (dmin32 * mn.float()).unsqueeze(2)
    q = torch.where(dsc > 0, _round_half_away((x + dm) / dsc.clamp(min=1e-30)), torch.zeros_like(x)).clamp(0, 15).to(torch.uint8)
    out = torch.empty(n, 144, dtype=torch.uint8, device=w.device)
    out[:, 0:2] = _f16_bytes(d).reshape(n, 2)
    out[:, 2:4] = _f16_bytes(dmin).reshape(n, 2)
    out[:, 4:8] = (sc[:, 0:4] & 63) | ((sc[:, 4:8] >> 4) << 6)
    out[:, 8:12] = (mn[:, 0:4] & 63) | ((mn[:, 4:8] >> 4) << 6)
    out[:, 12:16] = (sc[:, 4:8] & 15) | ((mn[:, 4:8] & 15) << 4)
    qp = q.reshape(n, 4, 2, 32)
    out[:, 16:144] = (qp[:, :, 0, :] | (qp[:, :, 1, :] << 4)).reshape(n, 128)
    return out.reshape(*lead, k // 256 * 144)


def random_payload(qtype: int, shape: tuple[int, ...], seed: int, std: float = 0.02, device="cpu") -> torch.Tensor:
    """Uniformly random valid blocks whose decode has a spread near ``std`` (any type on the path).

    For IQ2_XXS this stands in for an encoder: every index/sign/sub-scale field is uniform and the
    fp16 block scale sets the magnitude.
    """
    blk, nbytes = {8: (32, 34), 10: (256, 84), 11: (256, 110), 12: (256, 144), 13: (256, 176), 14: (256, 210), 16: (256, 66), 22: (256, 82)}[int(qtype)]
    *lead, k = shape
    n = 1
    for v in lead:
        n *= int(v)
    n *= k // blk
    g = torch.Generator(device=device).manual_seed(seed)
    b = torch.randint(0, 256, (n, nbytes), dtype=torch.uint8, generator=g, device=device)
    jitter = torch.rand(n, 1, generator=g, device=device) * 0.6 + 0.7
    if qtype == 8:
        b[:, 0:2] = _f16_bytes(std / 73.9 * jitter)
    elif qtype == 12:
        b[:, 0:2] = _f16_bytes(std / 190.0 * jitter)
        b[:, 2:4] = _f16_bytes(std / 25.0 * jitter)
    elif qtype == 10:
        b[:, 80:82] = _f16_bytes(std / 11.0 * jitter)
        b[:, 82:84] = _f16_bytes(std / 6.5 * jitter)
    elif qtype == 11:
        b[:, 108:110] = _f16_bytes(std / (18.5 * 2.3) * jitter)
    elif qtype == 13:
        b[:, 0:2] = _f16_bytes(std / 390.0 * jitter)
        b[:, 2:4] = _f16_bytes(std / 25.0 * jitter)
    elif qtype == 14:
        b[:, 208:210] = _f16_bytes(std / (74.0 * 18.5) * jitter)
    else:
        b[:, 0:2] = _f16_bytes(std * 4.0 / (85.0 * 600.0) ** 0.5 * jitter)
    return b.reshape(*lead, k // blk * nbytes)
