"""CPU: the drop-in module surface.  Every name the reference's two training scripts import from a module that this
package also provides must be importable from it (``train_qwen3.5_35b.py:22-29``, ``train_deepseek_v4.py:22-33``), the
DeepSeek expert wrapper registers and refuses like the reference's (``deepseek_v4_moe_lora.py:21-94``), and the adapter
state of an expert wrapper is exactly its four factor tensors (``test_deepseek_v4_serialization.py:73-107``)."""
import importlib
from pathlib import Path
from types import SimpleNamespace

import pytest
import torch

PKG = Path(__file__).resolve().parent.parent / "transformers5-qwen3.5-recipe_b200"

# (module, names) as the two training scripts import them; modules that this package does not provide (attention, mHC,
# RMSNorm, trainer, tuning) stay the reference's own and are not listed
TRAIN_SCRIPT_IMPORTS = {
    "fast_lora": ["register_fast_lora"],
    "fast_moe_lora": ["register_fast_moe_lora"],
    "fast_moe_ranking": ["configure_fast_moe_ranking"],
    "gguf_liger_loss": ["apply_gguf_liger_fused_linear_cross_entropy"],
    "deepseek_v4_liger_loss": ["apply_deepseek_v4_liger_loss"],
    "deepseek_v4_lora": ["DEEPSEEK_V4_TARGET_MODULES_PATTERN", "configure_deepseek_v4_grouped_mmq", "register_deepseek_v4_lora"],
    "deepseek_v4_moe_lora": ["register_deepseek_v4_moe_lora"],
}
# names the reference's audit script and tests take from the same modules
OTHER_IMPORTS = {
    "deepseek_v4_lora": ["audit_deepseek_v4_injection", "normalize_peft_path", "DeepseekV4LoraLinear", "DeepseekV4GGUFLoraLinear",
                         "ORDINARY_TARGET_MODULES", "EXPECTED_ORDINARY_WRAPPERS", "EXPECTED_EXPERT_WRAPPERS", "EXPECTED_RANK4_PARAMETERS"],
    "deepseek_v4_moe_lora": ["EXPERTS_IMPLEMENTATION", "DeepseekV4GGUFMoeLora", "deepseek_v4_gguf_dequant_aiter_lora_forward"],
    "deepseek_v4_liger_loss": ["deepseek_v4_liger_causal_lm_loss", "deepseek_v4_packed_liger_causal_lm_loss", "_deepseek_v4_liger_forward",
                               "_packed_q8_linear_cross_entropy_forward", "_PackedQ8LigerLinearCrossEntropyFunction"],
    "gguf_liger_loss": ["gguf_liger_lce_forward", "_packed_q8_liger_for_causal_lm_loss", "_packed_q8_linear_cross_entropy_forward"],
    "fast_moe_lora": ["FastGGUFMoeLora", "FastMoeParamWrapper", "EXPERTS_IMPLEMENTATION", "qwen3_5_moe_gguf_mmq_aiter_lora_forward",
                      "aiter_grouped_mm", "_base_grouped_linear", "_base_grouped_pair", "_group_sizes_from_offsets", "_complete_group_sizes",
                      "_aiter_forward", "_aiter_input_grad", "_aiter_weight_grad", "_ExpertLoraWeights", "_gmm_config", "_ptgmm_config"],
    "fast_moe_routing": ["ExpertRoutingPlan", "prepare_expert_routing", "finalize_expert_routing", "_is_supported_routing_geometry"],
    "fast_moe_ranking": ["router_topk_indices", "_is_supported_router_geometry", "_router_topk_launch"],
    "fast_lora": ["FastLoraLinear", "FastGGUFLoraLinear", "supports_native_mmq", "_fused_lora_add"],
    "moe_gmm_configs": ["gmm_config", "ptgmm_config"],
}


@pytest.mark.parametrize("table", [TRAIN_SCRIPT_IMPORTS, OTHER_IMPORTS], ids=["train_scripts", "tests_and_audit"])
def test_every_shadowed_module_exports_what_the_reference_imports(lib, table):
    for module_name, names in table.items():
        assert (PKG / f"{module_name}.py").exists(), module_name
        module = importlib.import_module(module_name)
        assert Path(module.__file__).resolve().parent == PKG, f"{module_name} was not taken from the drop-in directory"
        missing = [n for n in names if not hasattr(module, n)]
        assert not missing, f"{module_name} lacks {missing}"


def test_normalize_peft_path():
    from deepseek_v4_lora import normalize_peft_path as norm

    assert norm("base_model.model.model.layers.3.mlp.experts") == "model.layers.3.mlp.experts"
    assert norm("model.layers.0.self_attn.q_a_proj") == "model.layers.0.self_attn.q_a_proj"
    assert norm("layers.7.mlp.experts") == "model.layers.7.mlp.experts"
    assert norm("lm_head") == "lm_head"


def _toy_experts(e=2, h=32, i=16, qtype=8):
    from b2g.gguf_types import DeepseekV4GGUFExperts, GGUFQuantizedTensor
    from b2g.ops import payload_row_bytes

    cfg = SimpleNamespace(num_experts=e, hidden_size=h, moe_intermediate_size=i, hidden_act="silu", swiglu_limit=7.0,
                          _experts_implementation="eager")
    bank = DeepseekV4GGUFExperts(cfg, device="cpu", compute_dtype=torch.bfloat16)
    for name, (rows, cols) in (("gate_proj", (i, h)), ("up_proj", (i, h)), ("down_proj", (h, i))):
        cols_padded = max(cols, 32)
        payload = torch.zeros(e, rows, payload_row_bytes(qtype, cols_padded), dtype=torch.uint8)
        setattr(bank, name, GGUFQuantizedTensor(payload, quant_type=qtype, logical_shape=(e, rows, cols_padded)))
    return bank


class _ToyDeepseek(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.q_a_proj = torch.nn.Linear(32, 16, bias=False, dtype=torch.bfloat16)
        self.experts = _toy_experts()

    def set_experts_implementation(self, implementation: str) -> None:
        self.experts.config._experts_implementation = implementation


def _wrapped_bank(model=None):
    import fast_lora
    from deepseek_v4_lora import DEEPSEEK_V4_TARGET_MODULES_PATTERN, register_deepseek_v4_lora
    from deepseek_v4_moe_lora import DeepseekV4GGUFMoeLora, register_deepseek_v4_moe_lora

    if fast_lora.HAVE_PEFT:
        pytest.skip("PEFT present: the round trip runs through get_peft_model there")
    model = model or _ToyDeepseek()
    cfg = fast_lora.LoraConfig(target_modules=DEEPSEEK_V4_TARGET_MODULES_PATTERN, r=4, lora_alpha=4, lora_dropout=0.0, bias="none")
    register_deepseek_v4_lora(cfg)
    register_deepseek_v4_moe_lora(cfg, model)
    wrapper_type = cfg._custom_modules[type(model.experts)]
    assert wrapper_type is DeepseekV4GGUFMoeLora
    return model, cfg, wrapper_type(model.experts, "default", config=cfg, r=4, lora_alpha=4)


def test_register_deepseek_v4_moe_lora(lib):
    import fast_lora
    from b2g.gguf_types import ALL_GGUF_EXPERTS_FUNCTIONS
    from deepseek_v4_moe_lora import EXPERTS_IMPLEMENTATION, deepseek_v4_gguf_dequant_aiter_lora_forward, register_deepseek_v4_moe_lora

    model, cfg, layer = _wrapped_bank()
    assert EXPERTS_IMPLEMENTATION == "deepseek_v4_gguf_dequant_aiter_lora"
    assert model.experts.config._experts_implementation == EXPERTS_IMPLEMENTATION
    assert ALL_GGUF_EXPERTS_FUNCTIONS[EXPERTS_IMPLEMENTATION] is deepseek_v4_gguf_dequant_aiter_lora_forward
    # a collection of targets gets "experts" added; any other regex string is refused; target_parameters are refused
    listed = fast_lora.LoraConfig(target_modules=["q_a_proj"], r=4, lora_alpha=4)
    register_deepseek_v4_moe_lora(listed, model)
    assert listed.target_modules == {"q_a_proj", "experts"}
    with pytest.raises(ValueError, match="one exact indexer-excluding target pattern"):
        register_deepseek_v4_moe_lora(fast_lora.LoraConfig(target_modules=r".*experts$", r=4, lora_alpha=4), model)
    bad = fast_lora.LoraConfig(target_modules=["experts"], r=4, lora_alpha=4)
    bad.target_parameters = ["experts.gate_proj"]
    with pytest.raises(ValueError, match="not parameters"):
        register_deepseek_v4_moe_lora(bad, model)
    # the wrapper insists on its own implementation key and on a DeepSeek bank
    model.experts.config._experts_implementation = "eager"
    with pytest.raises(RuntimeError, match="requires experts_implementation="):
        layer(torch.zeros(1, 32, dtype=torch.bfloat16), torch.zeros(1, 1, dtype=torch.long), torch.ones(1, 1))
    with pytest.raises(TypeError, match="requires DeepseekV4GGUFExperts"):
        deepseek_v4_gguf_dequant_aiter_lora_forward(torch.nn.Linear(2, 2), None, None, None)


@pytest.mark.parametrize("flavour", ["deepseek", "qwen"])
def test_adapter_state_round_trip_holds_exactly_the_factor_tensors(lib, flavour):
    """``state_dict`` of an expert wrapper: the four factors per adapter under the PEFT names, no packed payload; a fresh
    wrapper loads them bit-identically; merging stays refused."""
    import fast_lora
    import fast_moe_lora as fml

    def make():
        if flavour == "deepseek":
            return _wrapped_bank()[2]
        if fast_lora.HAVE_PEFT:
            pytest.skip("PEFT present")
        bank = _toy_experts()
        bank.config._experts_implementation = fml.EXPERTS_IMPLEMENTATION
        cfg = fast_lora.LoraConfig(target_modules=["experts"], r=4, lora_alpha=4, lora_dropout=0.0, bias="none")
        return fml.FastGGUFMoeLora(bank, "default", config=cfg, r=4, lora_alpha=4)

    source = make()
    with torch.no_grad():
        for p in source.parameters():
            if p.requires_grad:
                p.normal_(std=0.03)
    state = source.state_dict()
    assert sorted(state) == ["lora_A.default.weight", "lora_A_down.default.weight", "lora_B.default.weight", "lora_B_down.default.weight"]
    assert not any("base_layer" in n or "gate_proj" in n or "up_proj" in n or "down_proj" in n for n in state)
    assert all(v.dtype == torch.bfloat16 for v in state.values())
    e, h, i, r = 2, 32, 16, 4
    assert {n: tuple(v.shape) for n, v in state.items()} == {
        "lora_A.default.weight": (e, r, h), "lora_B.default.weight": (e, 2 * i, r),
        "lora_A_down.default.weight": (e, r, i), "lora_B_down.default.weight": (e, h, r)}
    target = make()
    result = target.load_state_dict(state)
    assert not result.missing_keys and not result.unexpected_keys
    for name, value in target.state_dict().items():
        assert torch.equal(value, state[name]), name
    assert float(target.lora_B["default"].weight.detach().abs().max()) > 0       # the zeros of a fresh adapter were replaced
    with pytest.raises(RuntimeError, match="cannot be merged"):
        target.merge()
    with pytest.raises(RuntimeError, match="cannot be unmerged"):
        target.unmerge()
    with pytest.raises(RuntimeError, match="does not materialize"):
        target.get_delta_weight("default")


def test_injection_audit_lists_every_violation(lib):
    from deepseek_v4_lora import audit_deepseek_v4_injection
    from deepseek_v4_moe_lora import DeepseekV4GGUFMoeLora

    model, _, layer = _wrapped_bank()
    holder = torch.nn.Module()
    holder.layer = layer
    holder.stray = torch.nn.Linear(4, 4)            # trainable, fp32, CPU, not an adapter
    with pytest.raises(RuntimeError) as err:
        audit_deepseek_v4_injection(holder, expert_wrapper_type=DeepseekV4GGUFMoeLora, rank=4)
    text = str(err.value)
    for fragment in ("expected 383 ordinary wrappers, found 0", "expected 43 expert wrappers, found 1", "non-adapter trainable tensors",
                     "non-BF16 adapter tensors", "adapter tensors outside cuda:0", "rank-4 adapter parameters"):
        assert fragment in text, fragment


def test_loss_installers_check_their_model(lib):
    from b2g.gguf_types import GGUFLinear
    from deepseek_v4_liger_loss import _deepseek_v4_liger_forward, apply_deepseek_v4_liger_loss
    from gguf_liger_loss import apply_gguf_liger_fused_linear_cross_entropy

    with pytest.raises(TypeError, match="requires DeepseekV4ForCausalLM"):
        apply_deepseek_v4_liger_loss(torch.nn.Linear(2, 2))
    with pytest.raises(TypeError, match="requires Qwen3_5MoeForCausalLM"):
        apply_gguf_liger_fused_linear_cross_entropy(torch.nn.Linear(2, 2))

    class DeepseekV4ForCausalLM(torch.nn.Module):       # recognised by name when the fork is absent
        def __init__(self, head):
            super().__init__()
            self.lm_head = head

    import deepseek_v4_liger_loss as dl

    if dl.DeepseekV4ForCausalLM is not None:
        pytest.skip("transformers fork present")
    with pytest.raises(TypeError, match="requires GGUFLinear lm_head"):
        apply_deepseek_v4_liger_loss(DeepseekV4ForCausalLM(torch.nn.Linear(2, 2)))
    model = DeepseekV4ForCausalLM(GGUFLinear(32, 64))
    wrapped = SimpleNamespace(get_base_model=lambda: model)      # PEFT-style unwrap
    assert apply_deepseek_v4_liger_loss(wrapped) is model
    assert model.forward.__func__ is _deepseek_v4_liger_forward and model._deepseek_v4_liger_loss_enabled
    first = model.forward
    assert apply_deepseek_v4_liger_loss(model) is model and model.forward is first      # idempotent
