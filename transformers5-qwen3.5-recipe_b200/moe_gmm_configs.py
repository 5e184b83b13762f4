"""Tile configurations of the rank-side grouped products (B200 build).

The reference keeps exact-key tables of Triton tile shapes tuned for one AMD part and rejects any
shape that was not measured.  The B200 kernels have one fixed tiling each, so this module keeps the
import surface (``gmm_config``, ``ptgmm_config``) and the fail-closed behaviour: a shape the
rank-side kernels cannot take is rejected here, before anything launches.
"""
from __future__ import annotations

_CONFIG_KEYS = ("BLOCK_SIZE_M", "BLOCK_SIZE_K", "BLOCK_SIZE_N", "GROUP_SIZE", "GRID_DIM", "num_warps", "num_stages")
_MAX_RANK = 16


def _config(values: tuple[int, ...]) -> dict[str, int]:
    return dict(zip(_CONFIG_KEYS, values, strict=True))


def gmm_config(m: int, k: int, n: int, transposed_rhs: bool) -> dict[str, int]:
    """Grouped [M,K] x [E,K,N]: one side must be the LoRA rank (<= 16)."""
    del transposed_rhs
    if m < 0 or k <= 0 or n <= 0:
        raise ValueError(f"Invalid grouped-MM shape M={m}, K={k}, N={n}.")
    if n <= _MAX_RANK:      # projection onto the rank: 64-row CTAs, 128-column cp.async stages, 4 warps
        if k % 8:
            raise ValueError(f"No B200 rank-projection kernel for K={k}: K must be a multiple of 8.")
        return _config((64, 128, 16, 1, 592, 4, 3))
    if k <= _MAX_RANK:      # projection from the rank: one row per block, 128 threads
        return _config((1, 16, 128, 1, 2368, 4, 1))
    raise ValueError(f"No B200 grouped-MM kernel for M={m}, K={k}, N={n}: neither side is a LoRA rank (<= {_MAX_RANK}); "
                     "base-weight products run on packed payloads instead.")


def ptgmm_config(m: int, k: int, n: int) -> dict[str, int]:
    """Grouped lhs^T x rhs -> [E,K,N] factor gradient: one side must be the LoRA rank."""
    if m < 0 or k <= 0 or n <= 0:
        raise ValueError(f"Invalid grouped factor-gradient shape M={m}, K={k}, N={n}.")
    if min(k, n) > _MAX_RANK:
        raise ValueError(f"No B200 factor-gradient kernel for M={m}, K={k}, N={n}: neither side is a LoRA rank (<= {_MAX_RANK}).")
    if max(k, n) % 8:
        raise ValueError(f"No B200 factor-gradient kernel for K={k}, N={n}: the wide side must be a multiple of 8.")
    return _config((64, 16, 128, 1, 4096, 4, 3))
