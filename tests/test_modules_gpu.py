"""GPU: the reference-named module surface (fast_lora, fast_moe_lora, fast_moe_routing,
fast_moe_ranking) on stand-in GGUF modules, against the CPU oracle."""
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from oracle import dense_ref, gguf_oracle as go, moe_ref

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _packed_linear(cuda, n, k, qtype, seed, bias=False):
    from b2g.gguf_types import GGUFLinear, GGUFQuantizedTensor

    payload = go.quantize((np.random.default_rng(seed).standard_normal((n, k)) * 0.02).astype(np.float32), qtype)
    lin = GGUFLinear(k, n, bias=bias, device=cuda, compute_dtype=torch.bfloat16)
    lin.weight = GGUFQuantizedTensor(torch.from_numpy(payload).to(cuda), quant_type=qtype, logical_shape=(n, k))
    return lin, payload


def test_fast_gguf_lora_linear_matches_dequantize_then_matmul(cuda):
    """The relation of test_fast_lora.py:110-134 (37 output rows, rank 4, 3x11 tokens, seed 2468)."""
    import fast_lora

    lin, payload = _packed_linear(cuda, 37, 2048, go.Q4_K, 1)
    cfg = fast_lora.LoraConfig(target_modules=["proj"], r=4, lora_alpha=4, lora_dropout=0.0, bias="none")
    fast_lora.register_fast_lora(cfg)
    if fast_lora.HAVE_PEFT:
        pytest.skip("PEFT present: covered through get_peft_model in an environment with the fork")
    assert cfg._custom_modules[type(lin)] is fast_lora.FastGGUFLoraLinear
    layer = fast_lora.FastGGUFLoraLinear(lin, "default", r=4, lora_alpha=4)
    g = torch.Generator().manual_seed(2468)
    b = (torch.randn(37, 4, generator=g) * 0.02).bfloat16()
    with torch.no_grad():
        layer.lora_B["default"].weight.copy_(b)
    a = layer.lora_A["default"].weight.detach().cpu()
    x = torch.randn(3, 11, 2048, generator=g).bfloat16()
    dy = torch.randn(3, 11, 37, generator=g).bfloat16()
    xc = x.to(cuda).requires_grad_(True)
    y = layer(xc)
    y.backward(dy.to(cuda))
    ref = dense_ref.lora_linear_fwd_bwd(x.reshape(33, 2048), dense_ref.dequant_bf16(payload, go.Q4_K), a, b, 1.0, dy.reshape(33, 37),
                                        torch.float32)
    assert y.shape == (3, 11, 37)
    assert dense_ref.rel_l2(y.reshape(33, 37), ref["y"]) < TOL
    assert dense_ref.rel_l2(xc.grad.reshape(33, 2048), ref["dx"]) < TOL
    assert dense_ref.rel_l2(layer.lora_A["default"].weight.grad, ref["da"]) < TOL
    assert dense_ref.rel_l2(layer.lora_B["default"].weight.grad, ref["db"]) < TOL
    assert layer.base_layer.weight.grad is None
    with pytest.raises(RuntimeError, match="cannot be merged"):
        layer.merge()
    with pytest.raises(RuntimeError, match="cannot be unmerged"):
        layer.unmerge()
    # the operator-by-operator route (base mmq + fused addmm) agrees with the one-kernel route
    base = layer._base_layer_forward(xc.detach())
    two_step = fast_lora._fused_lora_add(base, xc.detach(), layer.lora_A["default"], layer.lora_B["default"], torch.nn.Identity(), 1.0)
    assert dense_ref.rel_l2(two_step, y) < 5e-3


def test_fast_lora_linear_on_a_plain_linear(cuda):
    import fast_lora

    if fast_lora.HAVE_PEFT:
        pytest.skip("PEFT present")
    lin = torch.nn.Linear(256, 64, bias=True, device=cuda, dtype=torch.bfloat16)
    layer = fast_lora.FastLoraLinear(lin, "default", r=8, lora_alpha=16)
    with torch.no_grad():
        layer.lora_B["default"].weight.normal_(std=0.02)
    x = torch.randn(5, 256, device=cuda, dtype=torch.bfloat16)
    want = lin(x) + 2.0 * (x @ layer.lora_A["default"].weight.t()) @ layer.lora_B["default"].weight.t()
    assert dense_ref.rel_l2(layer(x), want) < 5e-3


def _experts(cuda, e, h, i, qtype, seed):
    from b2g.gguf_types import GGUFExperts, GGUFQuantizedTensor
    from b2g import gguf_quant

    payloads, tensors = [], []
    for j, shape in enumerate(((e, i, h), (e, i, h), (e, h, i))):
        p = gguf_quant.random_payload(qtype, shape, seed + j, device=cuda)
        payloads.append(p.cpu().numpy())
        tensors.append(GGUFQuantizedTensor(p, quant_type=qtype, logical_shape=shape))
    return GGUFExperts(e, h, i, *tensors, compute_dtype=torch.bfloat16), payloads


def test_fast_gguf_moe_lora_layer(cuda):
    import fast_lora
    import fast_moe_lora as fml

    e, h, i, t, k, r = 256, 2048, 256, 257, 4, 4       # (top-4, hidden 2048) is one of the supported routing geometries
    experts, payloads = _experts(cuda, e, h, i, go.Q4_K, 5)
    cfg = fast_lora.LoraConfig(target_modules=["q_proj"], r=r, lora_alpha=8, lora_dropout=0.0, init_lora_weights=True)
    holder = torch.nn.Module()
    holder.experts = experts
    fml.register_fast_moe_lora(cfg, holder)
    assert "experts" in cfg.target_modules and experts.config._experts_implementation == fml.EXPERTS_IMPLEMENTATION
    if fast_lora.HAVE_PEFT:
        pytest.skip("PEFT present")
    layer = fml.FastGGUFMoeLora(experts, "default", config=cfg, r=r, lora_alpha=8)
    assert float(layer.lora_B["default"].weight.abs().max()) == 0.0 and layer.lora_A["default"].weight.shape == (e, r, h)
    g = torch.Generator().manual_seed(8642)
    with torch.no_grad():
        layer.lora_B["default"].weight.copy_((torch.randn(e, 2 * i, r, generator=g) * 0.02).bfloat16())
        layer.lora_B_down["default"].weight.copy_((torch.randn(e, h, r, generator=g) * 0.02).bfloat16())
    hidden = torch.randn(t, h, generator=g).bfloat16()
    logits = torch.randn(t, e, generator=g)
    idx = logits.topk(k, 1).indices
    wts = torch.softmax(logits.gather(1, idx), -1)
    gout = torch.randn(t, h, generator=g).bfloat16()

    hc = hidden.to(cuda).requires_grad_(True)
    out = layer(hc, idx.to(cuda), wts.to(cuda))
    out.backward(gout.to(cuda))
    lora = dict(gate_up_a=layer.lora_A["default"].weight, gate_up_b=layer.lora_B["default"].weight,
                down_a=layer.lora_A_down["default"].weight, down_b=layer.lora_B_down["default"].weight)
    ws = [dense_ref.dequant_bf16(p, go.Q4_K) for p in payloads]
    ref = moe_ref.moe_layer(hidden, idx, wts, *ws, {n: v.detach().cpu() for n, v in lora.items()}, 2.0, gout, torch.float32)
    assert dense_ref.rel_l2(out, ref["out"]) < TOL and dense_ref.rel_l2(hc.grad, ref["d_hidden"]) < TOL
    for n, v in lora.items():
        assert dense_ref.rel_l2(v.grad, ref["d_" + n]) < TOL, n
    fused = (out.detach().clone(), hc.grad.clone(), {n: v.grad.clone() for n, v in lora.items()})

    # operator-by-operator composition (grouped_mmq_pair, grouped rank products, add, SwiGLU, grouped_mmq)
    experts._b2g_fused = False
    for v in lora.values():
        v.grad = None
    hc2 = hidden.to(cuda).requires_grad_(True)
    out2 = layer(hc2, idx.to(cuda), wts.to(cuda))
    out2.backward(gout.to(cuda))
    assert dense_ref.rel_l2(out2, fused[0]) < TOL and dense_ref.rel_l2(hc2.grad, fused[1]) < TOL
    for n, v in lora.items():
        assert dense_ref.rel_l2(v.grad, fused[2][n]) < TOL, n

    with pytest.raises(RuntimeError, match="cannot be merged"):
        layer.merge()
    with pytest.raises(RuntimeError, match="does not materialize"):
        layer.get_delta_weight("default")
    state = {n for n, _ in layer.named_parameters()}
    assert {"lora_A.default.weight", "lora_B.default.weight", "lora_A_down.default.weight", "lora_B_down.default.weight"} <= state


def test_group_size_helpers_and_grouped_mm_contract(cuda):
    import fast_moe_lora as fml

    off = torch.tensor([2, 5, 6], dtype=torch.int32, device=cuda)
    sizes = fml._group_sizes_from_offsets(off)
    assert sizes.tolist() == [2, 3, 1]
    full = fml._complete_group_sizes(sizes, torch.tensor([1, 4, 7], device=cuda), 8)
    assert full.tolist() == [0, 2, 0, 0, 3, 0, 0, 1]
    with pytest.raises(ValueError):
        fml._group_sizes_from_offsets(off.long())
    g = torch.Generator().manual_seed(1)
    lhs = torch.randn(6, 256, generator=g).bfloat16().to(cuda).requires_grad_(True)
    a = torch.randn(8, 4, 256, generator=g).bfloat16().to(cuda).requires_grad_(True)     # [E, r, K]
    y = fml.aiter_grouped_mm(lhs, a.transpose(1, 2), full)
    want = moe_ref.grouped_mm(lhs.detach().cpu(), a.detach().cpu().transpose(1, 2), full.cpu())
    assert y.shape == (6, 4) and dense_ref.rel_l2(y, want) < 5e-3
    y.backward(torch.ones_like(y))
    assert float(a.grad[0].abs().max()) == 0.0 and float(a.grad[1].abs().max()) > 0     # idle experts get exact zeros
    with pytest.raises(ValueError, match="neither side is a LoRA rank"):
        fml.aiter_grouped_mm(lhs.detach(), torch.zeros(8, 256, 64, dtype=torch.bfloat16, device=cuda), full)
    with pytest.raises(ValueError, match="int32"):
        fml.aiter_grouped_mm(lhs.detach(), a.detach().transpose(1, 2), full.long())


def test_routing_module_is_fail_closed(cuda):
    import fast_moe_routing as fmr

    assert fmr._is_supported_routing_geometry(2048, 8, 2048) and not fmr._is_supported_routing_geometry(2048, 8, 1024)
    assert not fmr._is_supported_routing_geometry(65537, 8, 2048)
    h = torch.zeros(16, 1024, dtype=torch.bfloat16, device=cuda)
    idx = torch.zeros(16, 8, dtype=torch.int64, device=cuda)
    with pytest.raises(RuntimeError, match="Unsupported optimized expert-routing geometry"):
        fmr.prepare_expert_routing(h, idx, torch.ones(16, 8, device=cuda))
    h = torch.zeros(16, 2048, dtype=torch.bfloat16, device=cuda)
    with pytest.raises(ValueError):
        fmr.prepare_expert_routing(h, idx[:8], torch.ones(8, 8, device=cuda))
    plan = fmr.prepare_expert_routing(h, idx, torch.ones(16, 8, device=cuda))
    with pytest.raises(RuntimeError, match="output masks"):
        fmr.finalize_expert_routing(plan.selected_hidden_states, h, plan, torch.ones(1, device=cuda))
    with pytest.raises(RuntimeError, match="requires contiguous CUDA BF16 output"):
        fmr.finalize_expert_routing(plan.selected_hidden_states[:5], h, plan, None)


def test_qwen_router_forward(cuda):
    import fast_moe_ranking as fmk

    g = torch.Generator().manual_seed(1234)
    router = SimpleNamespace(hidden_dim=2048, top_k=8, weight=(torch.randn(256, 2048, generator=g) * 0.02).bfloat16().to(cuda))
    hidden = torch.randn(257, 2048, generator=g).bfloat16().to(cuda)
    logits, weights, indices = fmk._qwen_router_forward(router, hidden)
    ref_idx = moe_ref.router_topk(logits.cpu(), 8)
    assert torch.equal(indices.cpu(), ref_idx)
    assert dense_ref.rel_l2(weights, moe_ref.qwen_router_weights(logits.cpu(), ref_idx)) < 1e-2
    with pytest.raises(RuntimeError, match="supports only 256-expert"):
        fmk.router_topk_indices(torch.zeros(8, 128, device=cuda), 4)
    with pytest.raises(ValueError, match="correction bias"):
        fmk.router_topk_indices(torch.zeros(8, 256, device=cuda), 8, correction_bias=torch.zeros(256, device=cuda))
