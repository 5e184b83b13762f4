"""Fast LoRA wrappers for ordinary and packed-GGUF linear layers (B200 build).

Same public surface as the reference module of this name (``register_fast_lora``,
``FastLoraLinear``, ``FastGGUFLoraLinear``, ``supports_native_mmq``, ``_fused_lora_add``), so the
training scripts import it unchanged.  What differs is below the surface:

* the packed base product is ``b2g.mmq`` (tcgen05 kernel on the packed payload, bf16 activations,
  no activation quantisation) with ``b2g.mmq_grad_input`` as its registered backward;
* when an ordinary single-adapter LoRA sits on a packed layer, base product and LoRA residual run
  as ONE fused operator each way (``b2g.autograd.lora_qlinear``): the low-rank update is an extra
  K=16 MMA step into the same TMEM accumulator, so no full-size intermediate exists at all.

PEFT is optional at import time: with PEFT installed the wrappers subclass its ``Linear`` exactly
like the reference; without it a small stand-in base with the same attributes is used so that the
module (and its tests) work on a machine that has no PEFT.
"""
from __future__ import annotations

from typing import Any

import torch

from b2g import autograd as _ag
from b2g.autograd import mmq
from b2g.gguf_types import GGUFLinear, GGUFQuantizedTensor
from b2g.ops import LORA_PAD, NATIVE_QUANT_TYPES

try:
    from peft import LoraConfig
    from peft.tuners.lora.layer import VARIANT_KWARG_KEYS
    from peft.tuners.lora.layer import Linear as PeftLinear

    HAVE_PEFT = True
except Exception:  # PEFT absent: minimal base with the attributes the forward uses
    HAVE_PEFT = False
    VARIANT_KWARG_KEYS: list[str] = []

    class LoraConfig:  # type: ignore[no-redef]
        def __init__(self, r: int = 8, lora_alpha: int = 8, target_modules: Any = None, lora_dropout: float = 0.0,
                     bias: str = "none", use_rslora: bool = False, **kwargs: Any) -> None:
            self.r, self.lora_alpha, self.target_modules = r, lora_alpha, target_modules
            self.lora_dropout, self.bias, self.use_rslora = lora_dropout, bias, use_rslora
            self.lora_bias = False
            self.use_dora = False
            self.alora_invocation_tokens = None
            self.init_lora_weights = kwargs.pop("init_lora_weights", True)
            self.inference_mode = False
            self.target_parameters = None
            self._custom_modules: dict[type, type] = {}
            self.__dict__.update(kwargs)

        def _register_custom_module(self, mapping: dict[type, type]) -> None:
            self._custom_modules.update(mapping)

    class PeftLinear(torch.nn.Module):  # type: ignore[no-redef]
        """Single-adapter LoRA linear holding what PEFT's ``Linear`` exposes to the fast forward."""

        def __init__(self, base_layer: torch.nn.Module, adapter_name: str = "default", r: int = 8, lora_alpha: int = 8,
                     lora_dropout: float = 0.0, use_rslora: bool = False, dtype: torch.dtype = torch.bfloat16, **kwargs: Any):
            super().__init__()
            self.base_layer = base_layer
            in_f, out_f = base_layer.in_features, base_layer.out_features
            dev = next((p.device for p in base_layer.parameters()), None)
            w = getattr(base_layer, "weight", None)
            if dev is None and isinstance(w, torch.Tensor):
                dev = w.device
            self.lora_A = torch.nn.ModuleDict({adapter_name: torch.nn.Linear(in_f, r, bias=False, device=dev, dtype=dtype)})
            self.lora_B = torch.nn.ModuleDict({adapter_name: torch.nn.Linear(r, out_f, bias=False, device=dev, dtype=dtype)})
            torch.nn.init.zeros_(self.lora_B[adapter_name].weight)
            self.lora_dropout = torch.nn.ModuleDict(
                {adapter_name: torch.nn.Dropout(lora_dropout) if lora_dropout > 0 else torch.nn.Identity()})
            self.scaling = {adapter_name: lora_alpha / (r ** 0.5 if use_rslora else r)}
            self.lora_variant: dict[str, Any] = {}
            self.active_adapters = [adapter_name]
            self.disable_adapters = False
            self.merged = False

        def _check_forward_args(self, x: torch.Tensor, *args: Any, **kwargs: Any) -> None:
            return None

        def _cast_input_dtype(self, x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
            return x if x.dtype == dtype else x.to(dtype)

        def forward(self, x: torch.Tensor, *args: Any, **kwargs: Any) -> torch.Tensor:
            out = self.base_layer(x, *args, **kwargs)
            if self.disable_adapters:
                return out
            for name in self.active_adapters:
                a, b = self.lora_A[name], self.lora_B[name]
                out = out + b(a(self.lora_dropout[name](x.to(a.weight.dtype)))).to(out.dtype) * self.scaling[name]
            return out


# GGML type ids with a native packed kernel in this build (the reference's wheel lists
# {8, 10, 11, 12, 13, 14, 16, 22}; the others stay on the generic dequantise-then-matmul route).
_NATIVE_MMQ_QUANT_TYPES = frozenset(NATIVE_QUANT_TYPES)


def supports_native_mmq(weight: Any) -> bool:
    return int(weight.quant_type) in _NATIVE_MMQ_QUANT_TYPES


def _fused_lora_add(result: torch.Tensor, x: torch.Tensor, lora_A: torch.nn.Linear, lora_B: torch.nn.Linear,
                    dropout: torch.nn.Module, scaling: float) -> torch.Tensor:
    """``result + scaling * lora_B(lora_A(dropout(x)))`` with the residual folded into the second
    product (``addmm``), so only one full-size tensor is written."""
    dt = result.dtype
    hidden = torch.matmul(dropout(x).to(dt), lora_A.weight.to(dt).t())
    shape = result.shape
    out = torch.addmm(result.reshape(-1, shape[-1]), hidden.reshape(-1, hidden.shape[-1]), lora_B.weight.to(dt).t(),
                      beta=1, alpha=scaling).reshape(shape)
    if lora_B.bias is not None:
        out = torch.add(out, lora_B.bias.to(dt), alpha=scaling)
    return out


def _dropout_is_noop(dropout: torch.nn.Module) -> bool:
    return isinstance(dropout, torch.nn.Identity) or (isinstance(dropout, torch.nn.Dropout) and dropout.p == 0.0)


class _FastLoraForwardMixin:
    """Fused path for plain single-adapter LoRA; every other PEFT mode goes to PEFT's own forward."""

    _cast_input_only_without_autocast = False

    def _base_layer_forward(self: Any, x: torch.Tensor, *args: Any, **kwargs: Any) -> torch.Tensor:
        return self.base_layer(x, *args, **kwargs)

    def _fully_fused_forward(self: Any, x: torch.Tensor, lora_A: Any, lora_B: Any, scaling: float) -> torch.Tensor | None:
        return None  # only packed layers have a one-kernel form

    def forward(self: Any, x: torch.Tensor, *args: Any, **kwargs: Any) -> torch.Tensor:
        adapter_names = kwargs.get("adapter_names")
        active = self.active_adapters
        if self.disable_adapters or self.merged or adapter_names is not None or len(active) != 1:
            return super().forward(x, *args, **kwargs)
        name = active[0]
        if name not in self.lora_A or name in self.lora_variant:
            return super().forward(x, *args, **kwargs)

        self._check_forward_args(x, *args, **kwargs)
        base_kwargs = {k: v for k, v in kwargs.items() if k != "adapter_names" and k not in VARIANT_KWARG_KEYS}
        lora_A, lora_B = self.lora_A[name], self.lora_B[name]
        dropout, scaling = self.lora_dropout[name], self.scaling[name]
        noop = _dropout_is_noop(dropout)

        if noop and not args and not base_kwargs:
            fused = self._fully_fused_forward(x, lora_A, lora_B, scaling)
            if fused is not None:
                return fused

        result = self._base_layer_forward(x, *args, **base_kwargs)
        # With a no-op dropout x feeds the LoRA branch in the base-result dtype directly (no
        # bf16 -> adapter dtype -> bf16 round trip).
        if not noop and (not self._cast_input_only_without_autocast or not torch.is_autocast_enabled()):
            x = self._cast_input_dtype(x, lora_A.weight.dtype)
        return _fused_lora_add(result, x, lora_A, lora_B, dropout, scaling)


class FastLoraLinear(_FastLoraForwardMixin, PeftLinear):
    """Drop-in PEFT LoRA wrapper for ordinary floating-point linear modules."""


class FastGGUFLoraLinear(FastLoraLinear):
    """LoRA wrapper for frozen packed ``GGUFLinear`` modules: native packed kernels both ways."""

    def _native(self) -> bool:
        base = self.base_layer
        return (isinstance(base.weight, GGUFQuantizedTensor) and supports_native_mmq(base.weight)
                and base.input_permutation is None and base.output_permutation is None)

    def _base_layer_forward(self, x: torch.Tensor, *args: Any, **kwargs: Any) -> torch.Tensor:
        base = self.base_layer
        if not self._native():
            return base(x, *args, **kwargs)
        if args or kwargs:
            raise TypeError("The packed GGUF MMQ linear path accepts only its input tensor.")
        if base.compute_dtype != torch.bfloat16:
            raise RuntimeError("The packed GGUF MMQ linear path requires BF16 compute_dtype.")
        payload = base.weight.as_subclass(torch.Tensor)
        result = mmq(x, payload, int(base.weight.quant_type), base.out_features)
        if base.bias is not None:
            result = result + base.bias.to(device=result.device, dtype=result.dtype)
        return result

    def _fully_fused_forward(self, x: torch.Tensor, lora_A: Any, lora_B: Any, scaling: float) -> torch.Tensor | None:
        base = self.base_layer
        if (not self._native() or base.compute_dtype != torch.bfloat16 or x.dtype != torch.bfloat16 or not x.is_cuda
                or not x.is_contiguous() or lora_B.bias is not None or lora_A.weight.shape[0] > LORA_PAD):
            return None
        payload = base.weight.as_subclass(torch.Tensor)
        return _ag.lora_qlinear(x, payload, int(base.weight.quant_type), base.out_features, lora_A.weight, lora_B.weight,
                                float(scaling), base.bias)

    def merge(self, safe_merge: bool = False, adapter_names: list[str] | None = None) -> None:
        raise RuntimeError("GGUF LoRA adapters cannot be merged into packed base weights.")

    def unmerge(self) -> None:
        raise RuntimeError("GGUF LoRA adapters cannot be unmerged because merging is unsupported.")


def register_fast_lora(lora_config: Any) -> Any:
    """Register the fast wrappers on one ``LoraConfig`` (config-local, nothing is patched globally)."""
    register = getattr(lora_config, "_register_custom_module", None)
    if register is None:
        raise RuntimeError("This PEFT version has no LoraConfig._register_custom_module API. "
                           "Cannot install fast LoRA without a global monkey patch.")
    # GGUFLinear may subclass nn.Linear: its merge-safe wrapper has to be matched first.
    register({GGUFLinear: FastGGUFLoraLinear, torch.nn.Linear: FastLoraLinear})
    return lora_config
