"""Packed-GGUF MoE experts with per-expert LoRA (B200 build).

Public surface of the reference module of this name (``register_fast_moe_lora``, ``FastGGUFMoeLora``,
``FastMoeParamWrapper``, ``EXPERTS_IMPLEMENTATION``, ``qwen3_5_moe_gguf_mmq_aiter_lora_forward``,
``aiter_grouped_mm`` and the underscore helpers its tests and ``deepseek_v4_moe_lora.py`` import).
The names that mention AITER are kept for drop-in compatibility; on B200 they run this
repository's own kernels:

* base projections: one persistent tcgen05 launch over the ragged expert segments per product
  (gate and up share one launch and one pass over the routed rows);
* rank-side products: grouped skinny kernels; in the expert forward the LoRA up-projection and the
  ``add(alpha=s)`` are folded into the base launch as one extra MMA step per tile;
* input gradients: gate and up accumulate into one fp32 TMEM accumulator and round once.
No logical base matrix, expert LoRA delta or effective weight gradient is ever materialised.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, cast

import torch

from b2g import autograd as _ag
from b2g import ops as _ops
from b2g.gguf_types import ALL_GGUF_EXPERTS_FUNCTIONS, GGUFExperts, GGUFQuantizedTensor, dequantize_gguf_tensor  # noqa: F401
from fast_lora import HAVE_PEFT, LoraConfig, supports_native_mmq
from fast_moe_routing import finalize_expert_routing, prepare_expert_routing
from moe_gmm_configs import gmm_config as _gmm_config
from moe_gmm_configs import ptgmm_config as _ptgmm_config

if HAVE_PEFT:
    from peft.tuners.lora.layer import LoraLayer
else:
    class LoraLayer:  # type: ignore[no-redef]
        """The slice of PEFT's LoraLayer that the expert wrapper uses."""

        def __init__(self, base_layer: torch.nn.Module, **kwargs: Any) -> None:
            self.base_layer = base_layer
            self.r: dict[str, int] = {}
            self.lora_alpha: dict[str, int] = {}
            self.scaling: dict[str, float] = {}
            self.use_rslora: dict[str, bool] = {}
            self.use_dora: dict[str, bool] = {}
            self.lora_bias: dict[str, bool] = {}
            self.lora_dropout = torch.nn.ModuleDict()
            self.lora_A = torch.nn.ModuleDict()
            self.lora_B = torch.nn.ModuleDict()
            self._disable_adapters = False
            self._active_adapter: Any = "default"

        def get_base_layer(self) -> torch.nn.Module:
            return self.base_layer

        @property
        def disable_adapters(self) -> bool:
            return self._disable_adapters

        @property
        def active_adapters(self) -> list[str]:
            a = self._active_adapter
            return [a] if isinstance(a, str) else list(a)

        def set_adapter(self, adapter_names: Any, inference_mode: bool = False) -> None:
            self._active_adapter = adapter_names

EXPERTS_IMPLEMENTATION = "qwen3_5_moe_gguf_mmq_aiter_lora"
_LORA_WEIGHTS_KWARG = "_qwen3_5_moe_gguf_lora_weights"
_GGUF_EXPERTS_TYPE = cast(type[Any], GGUFExperts)


# ---- rank-side grouped products (the reference's AITER gmm / ptgmm call sites) --------------------
def _rhs_storage(rhs: torch.Tensor) -> tuple[torch.Tensor, bool]:
    """(contiguous storage, is_transposed_view): rhs [E,K,N] given either plainly or as a transpose(1,2) view."""
    if rhs.is_contiguous():
        return rhs, False
    t = rhs.transpose(1, 2)
    if t.is_contiguous():
        return t, True
    raise ValueError("grouped MM rhs must be contiguous or a transpose(1, 2) view of a contiguous tensor")


def _offsets_of(group_sizes: torch.Tensor) -> torch.Tensor:
    return torch.cumsum(group_sizes, 0).to(torch.int32)


def _aiter_forward(lhs: torch.Tensor, rhs: torch.Tensor, group_sizes: torch.Tensor) -> torch.Tensor:
    """[M,K] x [E,K,N] over contiguous row groups (zero-size groups allowed); one side is a LoRA rank."""
    m, k = lhs.shape
    e, _, n = rhs.shape
    _gmm_config(m, k, n, rhs.stride(1) == 1)
    offsets = _offsets_of(group_sizes)
    store, transposed = _rhs_storage(rhs)
    if n <= _ops.LORA_PAD:
        tiles = _ops.grouped_schedule(torch.arange(e, device=lhs.device), offsets, m)
        # storage [E,N,K] (transposed view) is the [r,C] layout; plain [E,K,N] is the [C,r] layout
        plain, _ = _ops.grouped_lora_down(lhs.contiguous(), None, store, not transposed, 1.0, n, tiles, plain=True, scaled=False)
        return plain[:, :n].contiguous() if n < _ops.LORA_PAD else plain
    return _ops.grouped_lora_up(lhs, store, transposed, offsets)


def _aiter_input_grad(grad_output: torch.Tensor, rhs: torch.Tensor, group_sizes: torch.Tensor) -> torch.Tensor:
    return _aiter_forward(grad_output, rhs.transpose(1, 2), group_sizes)


def _aiter_weight_grad(lhs: torch.Tensor, grad_output: torch.Tensor, group_sizes: torch.Tensor) -> torch.Tensor:
    """Per-expert lhs_e^T . grad_e -> [E, K, N] (inactive experts exactly zero)."""
    m, k = lhs.shape
    n = grad_output.shape[1]
    _ptgmm_config(m, k, n)
    e = group_sizes.numel()
    offsets = _offsets_of(group_sizes)
    out = torch.empty(e, k, n, dtype=lhs.dtype, device=lhs.device)
    if k <= _ops.LORA_PAD:      # rank on the left: [E, r, N]
        s16 = lhs if k == _ops.LORA_PAD else _ops.pad_rank_cols(lhs)
        _ops.grouped_lora_wgrad(s16.contiguous(), grad_output.contiguous(), 1.0, k, offsets, out, False)
    else:                       # rank on the right: [E, K, r] = (grad^T . lhs)^T
        s16 = grad_output if n == _ops.LORA_PAD else _ops.pad_rank_cols(grad_output)
        _ops.grouped_lora_wgrad(s16.contiguous(), lhs.contiguous(), 1.0, n, offsets, out, True)
    return out


class _AiterGroupedMM(torch.autograd.Function):
    """Autograd-capable ``(M,K) @ (E,K,N)`` grouped product for the LoRA factors."""

    @staticmethod
    def forward(ctx, lhs: torch.Tensor, rhs: torch.Tensor, group_sizes: torch.Tensor) -> torch.Tensor:
        if lhs.ndim != 2 or rhs.ndim != 3 or group_sizes.ndim != 1:
            raise ValueError("AITER grouped MM expects lhs [M,K], rhs [E,K,N], and group_sizes [E].")
        if lhs.shape[1] != rhs.shape[1]:
            raise ValueError(f"Grouped-MM K mismatch: lhs has {lhs.shape[1]}, rhs has {rhs.shape[1]}.")
        if rhs.shape[0] != group_sizes.numel():
            raise ValueError(f"Grouped-MM expert mismatch: rhs has {rhs.shape[0]}, group_sizes has {group_sizes.numel()}.")
        if lhs.dtype not in (torch.float16, torch.bfloat16) or rhs.dtype != lhs.dtype:
            raise TypeError(f"AITER grouped MM requires matching FP16/BF16 inputs, got {lhs.dtype} and {rhs.dtype}.")
        if lhs.dtype != torch.bfloat16:
            raise TypeError("The B200 grouped MM kernels are BF16 only.")
        if lhs.stride() != (lhs.shape[1], 1):
            raise ValueError("AITER grouped MM lhs must be row-major.")
        if group_sizes.device != lhs.device:
            raise ValueError("AITER grouped MM group_sizes must share the lhs device.")
        if group_sizes.dtype != torch.int32 or group_sizes.stride() != (1,):
            raise ValueError("AITER grouped MM group_sizes must be contiguous int32.")
        ctx.save_for_backward(lhs, rhs, group_sizes)
        return _aiter_forward(lhs, rhs, group_sizes)

    @staticmethod
    def backward(ctx, grad_output: torch.Tensor):
        lhs, rhs, group_sizes = ctx.saved_tensors
        if grad_output.stride() != (grad_output.shape[1], 1):
            raise ValueError("AITER grouped MM output gradient must be row-major.")
        grad_lhs = _aiter_input_grad(grad_output, rhs, group_sizes) if ctx.needs_input_grad[0] else None
        grad_rhs = _aiter_weight_grad(lhs, grad_output, group_sizes) if ctx.needs_input_grad[1] else None
        return grad_lhs, grad_rhs, None


def aiter_grouped_mm(lhs: torch.Tensor, rhs: torch.Tensor, group_sizes: torch.Tensor) -> torch.Tensor:
    """Autograd-capable grouped product for the expert LoRA factors."""
    return _AiterGroupedMM.apply(lhs, rhs, group_sizes)


# ---- packed base projections ------------------------------------------------------------------------
def _require_native(weight: Any) -> None:
    if not isinstance(weight, GGUFQuantizedTensor):
        raise RuntimeError("GGUF expert weights must be packed GGUFQuantizedTensor payloads on this path.")
    if not supports_native_mmq(weight):
        raise RuntimeError(f"GGML type {int(weight.quant_type)} has no native B200 kernel (supported: 8, 10, 11, 12, 13, 14, 16, 22); "
                           "there is no dequantise-then-matmul fallback in this build.")
    if weight.requires_grad:
        raise RuntimeError("Fast GGUF expert execution requires frozen packed base weights.")


class _AiterGGUFExpertProjection:
    """One packed grouped projection (the reference's autograd class of this name, as a callable)."""

    @staticmethod
    def apply(hidden_states: torch.Tensor, weight: Any, expert_indices: torch.Tensor, expert_offsets: torch.Tensor,
              group_sizes: torch.Tensor, compute_dtype: torch.dtype) -> torch.Tensor:
        del group_sizes
        _require_native(weight)
        if compute_dtype != torch.bfloat16:
            raise RuntimeError("Grouped GGUF MMQ requires BF16 compute dtype.")
        x = hidden_states.to(compute_dtype).contiguous()
        out = _ag.grouped_mmq(x, weight.as_subclass(torch.Tensor),
                              expert_indices.to(device=x.device, dtype=torch.long).contiguous(),
                              expert_offsets.to(device=x.device, dtype=torch.int32).contiguous(),
                              int(weight.quant_type), int(weight.logical_shape[-2]))
        return out


class _AiterGGUFExpertPairProjection:
    """Gate and up in one launch forward, one shared accumulator backward."""

    @staticmethod
    def apply(hidden_states: torch.Tensor, first_weight: Any, second_weight: Any, expert_indices: torch.Tensor,
              expert_offsets: torch.Tensor, group_sizes: torch.Tensor, compute_dtype: torch.dtype):
        del group_sizes
        _require_native(first_weight)
        _require_native(second_weight)
        if compute_dtype != torch.bfloat16:
            raise RuntimeError("Grouped GGUF MMQ requires BF16 compute dtype.")
        if first_weight.quant_type != second_weight.quant_type:
            raise RuntimeError("Paired grouped GGUF MMQ requires one quantization type.")
        if first_weight.logical_shape != second_weight.logical_shape:
            raise RuntimeError("Paired grouped GGUF MMQ requires matching logical shapes.")
        x = hidden_states.to(compute_dtype).contiguous()
        return _ag.grouped_mmq_pair(x, first_weight.as_subclass(torch.Tensor), second_weight.as_subclass(torch.Tensor),
                                    expert_indices.to(device=x.device, dtype=torch.long).contiguous(),
                                    expert_offsets.to(device=x.device, dtype=torch.int32).contiguous(),
                                    int(first_weight.quant_type), int(first_weight.logical_shape[-2]))


def _base_grouped_linear(hidden_states, weight, expert_indices, expert_offsets, group_sizes, compute_dtype):
    return _AiterGGUFExpertProjection.apply(hidden_states, weight, expert_indices, expert_offsets, group_sizes, compute_dtype)


def _base_grouped_pair(hidden_states, first_weight, second_weight, expert_indices, expert_offsets, group_sizes, compute_dtype):
    same = (isinstance(first_weight, GGUFQuantizedTensor) and isinstance(second_weight, GGUFQuantizedTensor)
            and supports_native_mmq(first_weight) and supports_native_mmq(second_weight)
            and first_weight.quant_type == second_weight.quant_type and first_weight.logical_shape == second_weight.logical_shape)
    if same:
        return _AiterGGUFExpertPairProjection.apply(hidden_states, first_weight, second_weight, expert_indices, expert_offsets,
                                                    group_sizes, compute_dtype)
    return (_base_grouped_linear(hidden_states, first_weight, expert_indices, expert_offsets, group_sizes, compute_dtype),
            _base_grouped_linear(hidden_states, second_weight, expert_indices, expert_offsets, group_sizes, compute_dtype))


# ---- PEFT wrapper -----------------------------------------------------------------------------------
class _ExpertFactor(torch.nn.Module):
    """One PEFT-visible expert factor with a conventional logical weight layout."""

    def __init__(self, shape: tuple[int, ...], *, device: Any, dtype: torch.dtype):
        super().__init__()
        self.weight = torch.nn.Parameter(torch.empty(shape, device=device, dtype=dtype))


@dataclass(frozen=True)
class _ExpertLoraWeights:
    gate_up_a: torch.Tensor  # [experts, rank, hidden]
    gate_up_b: torch.Tensor  # [experts, 2 * intermediate, rank]
    down_a: torch.Tensor     # [experts, rank, intermediate]
    down_b: torch.Tensor     # [experts, hidden, rank]
    scaling: float


class FastGGUFMoeLora(torch.nn.Module, LoraLayer):
    """LoRA wrapper owning all four factor tensors of one packed ``GGUFExperts`` module."""

    adapter_layer_names = ("lora_A", "lora_B", "lora_A_down", "lora_B_down")

    def _get_in_out_features(self, module: torch.nn.Module) -> tuple[int, int]:
        module = module.get_base_layer() if isinstance(module, LoraLayer) else module
        if not isinstance(module, _GGUF_EXPERTS_TYPE):
            raise TypeError(f"Fast GGUF MoE LoRA requires GGUFExperts, got {type(module).__name__}.")
        return int(module.hidden_dim), 2 * int(module.intermediate_dim)

    def __init__(self, base_layer: torch.nn.Module, adapter_name: str, *, config: Any, r: int, lora_alpha: int, **kwargs: Any):
        ephemeral = bool(kwargs.pop("ephemeral_gpu_offload", False))
        super().__init__()
        if HAVE_PEFT:
            LoraLayer.__init__(self, base_layer, ephemeral_gpu_offload=ephemeral, **kwargs)
        else:
            LoraLayer.__init__(self, base_layer)
        self.lora_A_down = torch.nn.ModuleDict()
        self.lora_B_down = torch.nn.ModuleDict()
        self._active_adapter = adapter_name
        self.update_layer(adapter_name, r, lora_alpha, config=config, **kwargs)

    def update_layer(self, adapter_name: str, r: int, lora_alpha: int, config: Any, **kwargs: Any) -> None:
        del kwargs
        if r <= 0:
            raise ValueError(f"LoRA rank must be positive, got {r}.")
        if r > _ops.LORA_PAD:
            raise ValueError(f"The B200 expert LoRA kernels support rank <= {_ops.LORA_PAD}, got {r}.")
        if config.lora_dropout != 0.0:
            raise ValueError("Fast GGUF MoE LoRA currently requires lora_dropout=0.")
        if config.lora_bias:
            raise ValueError("Fast GGUF MoE LoRA does not support LoRA bias.")
        if config.use_dora or config.alora_invocation_tokens is not None:
            raise ValueError("Fast GGUF MoE LoRA does not support DoRA or aLoRA variants.")
        experts = cast(Any, self.get_base_layer())
        if not isinstance(experts, _GGUF_EXPERTS_TYPE):
            raise TypeError(f"Fast GGUF MoE LoRA requires GGUFExperts, got {type(experts).__name__}.")
        device, dtype = experts.gate_proj.device, experts.compute_dtype
        e, h, i = int(experts.num_experts), int(experts.hidden_dim), int(experts.intermediate_dim)
        self.r[adapter_name] = r
        self.lora_alpha[adapter_name] = lora_alpha
        self.scaling[adapter_name] = lora_alpha / (math.sqrt(r) if config.use_rslora else r)
        self.use_rslora[adapter_name] = config.use_rslora
        self.use_dora[adapter_name] = False
        self.lora_bias[adapter_name] = False
        self.lora_dropout[adapter_name] = torch.nn.Identity()
        self.lora_A[adapter_name] = _ExpertFactor((e, r, h), device=device, dtype=dtype)
        self.lora_B[adapter_name] = _ExpertFactor((e, 2 * i, r), device=device, dtype=dtype)
        self.lora_A_down[adapter_name] = _ExpertFactor((e, r, i), device=device, dtype=dtype)
        self.lora_B_down[adapter_name] = _ExpertFactor((e, h, r), device=device, dtype=dtype)
        a, b = self.lora_A[adapter_name].weight, self.lora_B[adapter_name].weight
        a_down, b_down = self.lora_A_down[adapter_name].weight, self.lora_B_down[adapter_name].weight
        init = config.init_lora_weights
        if init is True:
            torch.nn.init.kaiming_uniform_(a, a=math.sqrt(5))
            torch.nn.init.kaiming_uniform_(a_down, a=math.sqrt(5))
        elif init == "gaussian":
            torch.nn.init.normal_(a, std=1 / r)
            torch.nn.init.normal_(a_down, std=1 / r)
        elif init is not False:
            raise ValueError(f"Fast GGUF MoE LoRA does not support init_lora_weights={init!r}.")
        if init is not False:
            torch.nn.init.zeros_(b)
            torch.nn.init.zeros_(b_down)
        self.set_adapter(self.active_adapters, inference_mode=getattr(config, "inference_mode", False))

    def merge(self, safe_merge: bool = False, adapter_names: list[str] | None = None) -> None:
        raise RuntimeError("GGUF expert LoRA adapters cannot be merged into packed base weights.")

    def unmerge(self) -> None:
        raise RuntimeError("GGUF expert LoRA adapters cannot be unmerged because merging is unsupported.")

    def get_delta_weight(self, adapter_name: str, *args: Any, **kwargs: Any) -> torch.Tensor:
        raise RuntimeError("GGUF expert LoRA does not materialize a full expert delta weight.")

    def _active_lora_weights(self, adapter_names: Any) -> _ExpertLoraWeights | None:
        if self.disable_adapters:
            return None
        if adapter_names is not None:
            raise RuntimeError("Fast GGUF MoE LoRA does not support mixed-adapter batches.")
        if len(self.active_adapters) != 1:
            raise RuntimeError("Fast GGUF MoE LoRA requires exactly one active adapter.")
        name = self.active_adapters[0]
        if name not in self.lora_A:
            return None
        return _ExpertLoraWeights(gate_up_a=self.lora_A[name].weight, gate_up_b=self.lora_B[name].weight,
                                  down_a=self.lora_A_down[name].weight, down_b=self.lora_B_down[name].weight,
                                  scaling=float(self.scaling[name]))

    def forward(self, hidden_states: torch.Tensor, *args: Any, **kwargs: Any) -> torch.Tensor:
        adapter_names = kwargs.pop("adapter_names", None)
        weights = self._active_lora_weights(adapter_names)
        experts = cast(Any, self.get_base_layer())
        if experts.config._experts_implementation != EXPERTS_IMPLEMENTATION:
            raise RuntimeError(f"Fast GGUF MoE LoRA requires experts_implementation={EXPERTS_IMPLEMENTATION!r}, "
                               f"got {experts.config._experts_implementation!r}.")
        kwargs[_LORA_WEIGHTS_KWARG] = weights
        return self.base_layer(hidden_states, *args, **kwargs)


FastMoeParamWrapper = FastGGUFMoeLora


def _group_sizes_from_offsets(offsets: torch.Tensor) -> torch.Tensor:
    if offsets.ndim != 1:
        raise ValueError(f"GGUF grouped execution requires one-dimensional offsets, got {offsets.shape}.")
    if offsets.dtype != torch.int32 or offsets.stride() != (1,):
        raise ValueError("GGUF grouped offsets must be contiguous int32.")
    return torch.diff(offsets, prepend=offsets.new_zeros(1))


def _complete_group_sizes(active_group_sizes: torch.Tensor, expert_indices: torch.Tensor, num_experts: int) -> torch.Tensor:
    if expert_indices.numel() == num_experts:
        return active_group_sizes
    return active_group_sizes.new_zeros(num_experts).index_copy(0, expert_indices, active_group_sizes)


def _lora_grouped_linear(hidden_states, lora_a, lora_b, group_sizes):
    rank_states = aiter_grouped_mm(hidden_states, lora_a.transpose(1, 2), group_sizes)
    return aiter_grouped_mm(rank_states, lora_b.transpose(1, 2), group_sizes)


def _can_fuse(self: Any, lora: _ExpertLoraWeights | None) -> bool:
    ws = (self.gate_proj, self.up_proj, self.down_proj)
    if not all(isinstance(w, GGUFQuantizedTensor) and supports_native_mmq(w) for w in ws):
        return False
    if self.gate_proj.quant_type != self.up_proj.quant_type or self.gate_proj.logical_shape != self.up_proj.logical_shape:
        return False
    if self.compute_dtype != torch.bfloat16 or not getattr(self, "_b2g_fused", True):
        return False
    return lora is None or (lora.gate_up_a.shape[1] <= _ops.LORA_PAD and lora.gate_up_a.dtype == torch.bfloat16)


def qwen3_5_moe_gguf_mmq_aiter_lora_forward(self: Any, hidden_states: torch.Tensor, top_k_index: torch.Tensor,
                                            top_k_weights: torch.Tensor,
                                            _qwen3_5_moe_gguf_lora_weights: _ExpertLoraWeights | None = None) -> torch.Tensor:
    """Packed base projections with per-expert LoRA for one ``GGUFExperts`` module."""
    if not isinstance(self, _GGUF_EXPERTS_TYPE):
        raise TypeError(f"{EXPERTS_IMPLEMENTATION} requires GGUFExperts, got {type(self).__name__}.")
    if self.projection_layout != "split_gate_up" or self.has_bias or not self.has_gate:
        raise RuntimeError("The GGUF AITER LoRA path requires split, bias-free gate/up expert projections.")
    compute_states = self._prepare_expert_hidden_states(hidden_states)
    plan = prepare_expert_routing(compute_states, top_k_index, top_k_weights, int(self.num_experts))
    execution = self._prepare_expert_execution(plan, "grouped_mm")
    if execution.offsets is None:
        raise RuntimeError("GGUF AITER LoRA requires grouped expert offsets.")
    selected = plan.selected_hidden_states
    expert_indices = execution.expert_indices.to(device=selected.device, dtype=torch.long).contiguous()
    expert_offsets = execution.offsets.to(device=selected.device, dtype=torch.int32).contiguous()
    lora = _qwen3_5_moe_gguf_lora_weights

    limit = float(getattr(self, "swiglu_limit", None) or 0.0)
    if _can_fuse(self, lora) and hasattr(self, "swiglu_limit"):
        # whole expert block as one autograd node: pair launch (+LoRA), SwiGLU, down launch (+LoRA)
        offsets_full = getattr(execution, "offsets_full", None)
        if offsets_full is None:
            sizes = _complete_group_sizes(_group_sizes_from_offsets(expert_offsets), expert_indices, self.num_experts)
            offsets_full = _offsets_of(sizes)
        output = _ag.grouped_lora_experts(
            selected, self.gate_proj.as_subclass(torch.Tensor), self.up_proj.as_subclass(torch.Tensor),
            self.down_proj.as_subclass(torch.Tensor), int(self.gate_proj.quant_type), int(self.down_proj.quant_type),
            int(self.intermediate_dim), expert_indices, expert_offsets, offsets_full,
            None if lora is None else lora.gate_up_a, None if lora is None else lora.gate_up_b,
            None if lora is None else lora.down_a, None if lora is None else lora.down_b,
            1.0 if lora is None else lora.scaling, limit)
        return finalize_expert_routing(output, hidden_states, plan, execution.output_mask)

    # operator-by-operator composition (same order of operations as the reference forward)
    group_sizes = _group_sizes_from_offsets(expert_offsets)
    gate, up = _base_grouped_pair(selected, self.gate_proj, self.up_proj, expert_indices, expert_offsets, group_sizes, self.compute_dtype)
    if lora is not None:
        lora_sizes = _complete_group_sizes(group_sizes, expert_indices, self.num_experts)
        delta = _lora_grouped_linear(selected, lora.gate_up_a, lora.gate_up_b, lora_sizes)
        gate_delta, up_delta = delta.chunk(2, dim=-1)
        gate = torch.add(gate, gate_delta, alpha=lora.scaling)
        up = torch.add(up, up_delta, alpha=lora.scaling)
    intermediate = self._apply_split_gate(gate, up)
    output = _base_grouped_linear(intermediate, self.down_proj, expert_indices, expert_offsets, group_sizes, self.compute_dtype)
    if lora is not None:
        output = torch.add(output, _lora_grouped_linear(intermediate, lora.down_a, lora.down_b, lora_sizes), alpha=lora.scaling)
    return finalize_expert_routing(output, hidden_states, plan, execution.output_mask)


def register_fast_moe_lora(lora_config: Any, model: torch.nn.Module) -> Any:
    """Register the expert backend (process-wide registry) and its config-local LoRA wrapper."""
    register = getattr(lora_config, "_register_custom_module", None)
    if register is None:
        raise RuntimeError("This PEFT version has no LoraConfig._register_custom_module API. "
                           "Cannot install fast GGUF MoE LoRA without a global PEFT monkey patch.")
    if getattr(lora_config, "target_parameters", None):
        raise ValueError("Persistent GGUF expert LoRA targets the complete 'experts' module, not target_parameters.")
    if isinstance(lora_config.target_modules, str):
        raise TypeError("Fast GGUF MoE LoRA requires an explicit target_modules collection, not a regex string.")
    targets = set(lora_config.target_modules or ())
    targets.add("experts")
    lora_config.__dict__["target_modules"] = targets
    ALL_GGUF_EXPERTS_FUNCTIONS[EXPERTS_IMPLEMENTATION] = qwen3_5_moe_gguf_mmq_aiter_lora_forward
    setter = getattr(model, "set_experts_implementation", None)
    if callable(setter):
        setter(EXPERTS_IMPLEMENTATION)
    else:   # plain module tree: switch every expert bank directly
        for module in model.modules():
            if isinstance(module, _GGUF_EXPERTS_TYPE):
                module.config._experts_implementation = EXPERTS_IMPLEMENTATION
    register({GGUFExperts: FastGGUFMoeLora})
    return lora_config
