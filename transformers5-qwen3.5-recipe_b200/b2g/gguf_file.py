"""GGUF file -> packed device payloads: the step before the hot path.

The reference reads its checkpoints through the transformers fork; its own tests take single tensors straight from
``gguf.GGUFReader`` and wrap the bytes as ``GGUFQuantizedTensor(payload, quant_type, logical_shape)``
(``test_fast_moe_lora.py:78-103``, ``test_fast_lora.py:37-60``).  This module does the same for whole files: the payload
bytes go to the device exactly as they lie in the file (the kernels consume the on-disk block layout), nothing is
dequantised, and tensors of a type this library cannot multiply natively are reported instead of silently converted.
"""
from __future__ import annotations

from pathlib import Path
from typing import Iterator, Optional, Union

import numpy as np
import torch

from . import ops
from .gguf_types import GGUFQuantizedTensor

_FLOAT_TYPES = {0: torch.float32, 1: torch.float16, 30: torch.bfloat16}   # GGML ids F32, F16, BF16


def _reader(source):
    import gguf

    return source if isinstance(source, gguf.GGUFReader) else gguf.GGUFReader(str(Path(source)))


def logical_shape(tensor) -> tuple[int, ...]:
    """GGUF stores dimensions fastest-first; the logical (row-major) shape is the reverse."""
    return tuple(int(v) for v in reversed(tensor.shape))


def tensor_names(source) -> list[str]:
    return [t.name for t in _reader(source).tensors]


def load_tensor(source, name: str, device: Union[str, torch.device] = "cuda", *, leading: Optional[int] = None,
                rows: Optional[int] = None):
    """One tensor of a GGUF file on ``device``.

    Quantized tensors of a native type come back as ``GGUFQuantizedTensor`` (uint8 ``[..., rows, row bytes]``) with
    ``quant_type`` and ``logical_shape``; float tensors as ordinary tensors.  ``leading`` / ``rows`` keep only the first
    experts / output rows, as the reference's tests do to bound their fixtures.  Any other type raises."""
    reader = _reader(source)
    tensor = next((t for t in reader.tensors if t.name == name), None)
    if tensor is None:
        raise KeyError(f"{name!r} is not in the GGUF file")
    qt = int(tensor.tensor_type)
    shape = logical_shape(tensor)
    data = np.asarray(tensor.data)
    if qt in _FLOAT_TYPES:
        arr = data.view(np.uint16) if qt == 30 else data
        out = torch.from_numpy(np.array(arr, copy=True)).reshape(shape)
        out = out.view(torch.bfloat16) if qt == 30 else out
        return out.to(device)
    if qt not in ops.NATIVE_QUANT_TYPES:
        raise ValueError(f"{name!r} has GGML type {qt}, which this library cannot multiply natively "
                         f"(native: {sorted(ops.NATIVE_QUANT_TYPES)})")
    k = shape[-1]
    payload = data.reshape(*shape[:-1], ops.payload_row_bytes(qt, k))
    if leading is not None:
        if payload.ndim < 3:
            raise ValueError("`leading` needs a tensor with a leading (expert) dimension")
        payload = payload[:leading]
    if rows is not None:
        payload = payload[..., :rows, :]
    kept = tuple(payload.shape[:-1]) + (k,)
    dev_payload = torch.from_numpy(np.array(payload, dtype=np.uint8, copy=True, order="C")).to(device)
    return GGUFQuantizedTensor(dev_payload, quant_type=qt, logical_shape=kept)


def iter_tensors(source, device: Union[str, torch.device] = "cuda", *, skip_unsupported: bool = False) -> Iterator[tuple[str, torch.Tensor]]:
    """(name, tensor) for every tensor of the file, in file order."""
    reader = _reader(source)
    for t in reader.tensors:
        try:
            yield t.name, load_tensor(reader, t.name, device)
        except ValueError:
            if not skip_unsupported:
                raise


def type_census(source) -> dict[int, int]:
    """How many tensors of each GGML type the file holds (what a caller checks before choosing the native path)."""
    census: dict[int, int] = {}
    for t in _reader(source).tensors:
        census[int(t.tensor_type)] = census.get(int(t.tensor_type), 0) + 1
    return census
