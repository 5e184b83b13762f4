"""GPU: the benchmark configurations at their full sizes against the CPU oracle.

Dense (all nine (M, N) points of the attention-shaped Q4_K LoRA linears) is cheap enough for the oracle to run whole.
The two MoE configurations are not, so they are checked in COMPLETE SLICES: for three experts (the first, a middle one and
the busiest) the oracle runs exactly that expert's rows through gate|up -> LoRA -> SwiGLU -> down -> LoRA forward and
backward, and the expert's output rows, input-gradient rows and four factor gradients must agree; the weighted combine,
the token gradient and the shared expert are checked on a 512-token prefix and suffix.  Relations as in
``test_fast_lora.py:110-134``, ``test_fast_moe_lora.py:106-130,192-203`` and ``test_deepseek_v4_moe_lora.py:67-118,194-196``.
Tolerance: rel-L2 <= 1e-2 (bf16) on every output and gradient.
"""
import numpy as np
import pytest
import torch

from oracle import dense_ref, gguf_oracle as go, moe_ref

pytestmark = pytest.mark.gpu
TOL = 1e-2


# ---------------------------------------------------------------------------------------------------------------------
# dense: K = 2048, N in {4096, 512, 2048}, M in {2048, 8192, 32768}, Q4_K, r = 16, alpha = 32
# ---------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("n", [4096, 512, 2048])
@pytest.mark.parametrize("m", [2048, 8192, 32768])
def test_dense_q4k_lora_linear_at_every_benchmark_point(cuda, m, n):
    from b2g import autograd as ag, gguf_quant

    k, r, scaling = 2048, 16, 2.0
    g = torch.Generator().manual_seed(19260817 + 1)
    w = torch.randn(n, k, generator=g) * 0.02
    payload = gguf_quant.quantize_q4_k(w)
    a = (torch.randn(r, k, generator=g) / 16).bfloat16()
    b = (torch.randn(n, r, generator=g) * 0.01).bfloat16()
    x = torch.randn(m, k, generator=g).bfloat16()
    dy = torch.randn(m, n, generator=g).bfloat16()
    w_ref = dense_ref.dequant_bf16(payload, go.Q4_K)
    ref = dense_ref.lora_linear_fwd_bwd(x, w_ref, a, b, scaling, dy, torch.float32)

    xc = x.to(cuda).requires_grad_(True)
    ac, bc = a.to(cuda).requires_grad_(True), b.to(cuda).requires_grad_(True)
    y = ag.lora_qlinear(xc, payload.to(cuda), go.Q4_K, n, ac, bc, scaling)
    y.backward(dy.to(cuda))
    for name, got in (("y", y), ("dx", xc.grad), ("da", ac.grad), ("db", bc.grad)):
        assert dense_ref.rel_l2(got, ref[name]) < TOL, name
    # the last (ragged or not) row tile by itself, where an off-by-one in the tile walk would hide in a whole-matrix norm
    for name, got in (("y", y), ("dx", xc.grad)):
        for rows in (slice(0, 1024), slice(m - 1024, m)):
            assert dense_ref.rel_l2(got[rows], ref[name][rows]) < TOL, (name, rows)


# ---------------------------------------------------------------------------------------------------------------------
# MoE helpers
# ---------------------------------------------------------------------------------------------------------------------
def _bank(cuda, qtype, e, h, i, seed):
    from b2g import gguf_quant

    return [gguf_quant.random_payload(qtype, shape, seed + j, device=cuda) for j, shape in enumerate(((e, i, h), (e, i, h), (e, h, i)))]


def _expert_weights(payloads, qtype, ex):
    return [dense_ref.dequant_bf16(p[ex].cpu().numpy(), qtype) for p in payloads]


def _run_routed(cuda, payloads, qtypes, e, h, i, hidden, idx, wts, lora, scaling, limit, gout, shared=None):
    """The routed layer piece by piece (plan, expert block, combine) so that the per-row intermediates can be read."""
    from b2g import autograd as ag, routing

    hc = hidden.clone().requires_grad_(True)
    wc = wts.clone().requires_grad_(True)
    plan = routing.build_plan(hc, idx, wc, e)
    sel = plan.selected_hidden_states
    sel.retain_grad()
    ids = torch.arange(e, device=cuda)
    out_e = ag.grouped_lora_experts(sel, *payloads, qtypes[0], qtypes[1], i, ids, plan.group_offsets, plan.group_offsets,
                                    lora["gate_up_a"], lora["gate_up_b"], lora["down_a"], lora["down_b"], scaling, limit)
    out_e.retain_grad()
    final = routing.combine(out_e, plan)
    total = final if shared is None else final + shared(hc)
    total.backward(gout)
    return dict(plan=plan, sel=sel, out_e=out_e, final=final, total=total, d_hidden=hc.grad, d_weights=wc.grad)


def _check_expert_slices(run, payloads, qtypes, lora, scaling, limit, experts):
    plan = run["plan"]
    ends = plan.group_offsets.cpu().tolist()
    sizes = plan.group_sizes.cpu().tolist()
    for ex in experts:
        b, en = ends[ex] - sizes[ex], ends[ex]
        assert en > b, f"expert {ex} received no rows; pick another"
        wg, wu = (dense_ref.dequant_bf16(p[ex].cpu().numpy(), qtypes[0]) for p in payloads[:2])
        wd = dense_ref.dequant_bf16(payloads[2][ex].cpu().numpy(), qtypes[1])
        own = {n: v[ex].detach().cpu() for n, v in lora.items()}
        ref = moe_ref.expert_slice(run["sel"][b:en].detach().cpu(), wg, wu, wd, own, scaling, run["out_e"].grad[b:en].cpu(),
                                   limit if limit else None)
        assert dense_ref.rel_l2(run["out_e"][b:en], ref["out"]) < TOL, (ex, "out")
        assert dense_ref.rel_l2(run["sel"].grad[b:en], ref["d_rows"]) < TOL, (ex, "d_rows")
        for n in lora:
            assert dense_ref.rel_l2(lora[n].grad[ex], ref["d_" + n]) < TOL, (ex, n)


def _check_permutes(run, hidden, idx, wts, gout, tokens, shared_dx=None, shared_y=None):
    """Gather, combine and their backwards on a token range, from the kernels' own per-row tensors."""
    t, k = idx.shape
    cpu_plan = moe_ref.route_plan(idx.cpu(), int(run["plan"].group_sizes.numel()))
    plan = run["plan"]
    assert torch.equal(plan.permutation.cpu(), cpu_plan["permutation"]) and torch.equal(plan.inverse_permutation.cpu(), cpu_plan["inverse_permutation"])
    assert torch.equal(plan.group_offsets.cpu(), cpu_plan["offsets"])
    assert torch.equal(run["sel"].detach().cpu(), moe_ref.route_gather(hidden.cpu(), cpu_plan["permutation"], k))
    out_e, d_sel = run["out_e"].detach().cpu(), run["sel"].grad.cpu()
    inv = cpu_plan["inverse_permutation"].view(t, k)[tokens]
    want_final = moe_ref.route_combine(out_e, wts.cpu()[tokens], inv.reshape(-1))
    torch.testing.assert_close(run["final"][tokens].cpu().float(), want_final.float(), rtol=0, atol=2 ** -6)
    want_dh = moe_ref.route_gather_bwd(d_sel, inv.reshape(-1), inv.shape[0], k).float()
    if shared_dx is not None:
        want_dh = want_dh + shared_dx.float()
    assert dense_ref.rel_l2(run["d_hidden"][tokens], want_dh) < TOL
    if shared_y is not None:
        assert dense_ref.rel_l2(run["total"][tokens], want_final.float() + shared_y.float()) < TOL
    # cotangent of the expert outputs: bf16(dFinal[token] * bf16(weight)), exact
    perm = cpu_plan["permutation"]
    w_sorted = wts.cpu().reshape(-1)[perm].to(torch.bfloat16).float()
    want_dout = (gout.cpu()[perm // k].float() * w_sorted[:, None]).to(torch.bfloat16)
    assert torch.equal(run["out_e"].grad.cpu(), want_dout)


def _lora(cuda, e, h, i, r, g):
    return dict(gate_up_a=(torch.randn(e, r, h, generator=g) / 16).bfloat16().to(cuda).requires_grad_(True),
                gate_up_b=(torch.randn(e, 2 * i, r, generator=g) * 0.01).bfloat16().to(cuda).requires_grad_(True),
                down_a=(torch.randn(e, r, i, generator=g) / 16).bfloat16().to(cuda).requires_grad_(True),
                down_b=(torch.randn(e, h, r, generator=g) * 0.01).bfloat16().to(cuda).requires_grad_(True))


# ---------------------------------------------------------------------------------------------------------------------
# Qwen-shaped grouped MoE: 256 Q4_K experts, top-8, hidden 2048, intermediate 512, r = 16, 16384 tokens
# ---------------------------------------------------------------------------------------------------------------------
def test_qwen_moe_layer_at_benchmark_size_in_expert_slices(cuda):
    from b2g import ops

    e, h, i, t, k, r, scaling = 256, 2048, 512, 16384, 8, 16, 2.0
    g = torch.Generator().manual_seed(19260817 + 2)
    payloads = _bank(cuda, go.Q4_K, e, h, i, 21)
    lora = _lora(cuda, e, h, i, r, g)
    hidden = torch.randn(t, h, generator=g).bfloat16().to(cuda)
    logits = torch.randn(t, e, generator=g).to(cuda)
    gout = torch.randn(t, h, generator=g).bfloat16().to(cuda)
    idx = ops.router_topk(logits, k, None, False)
    assert torch.equal(idx.cpu(), moe_ref.router_topk(logits.cpu(), k))
    wts = torch.softmax(logits.gather(1, idx), -1)
    run = _run_routed(cuda, payloads, (go.Q4_K, go.Q4_K), e, h, i, hidden, idx, wts, lora, scaling, 0.0, gout)
    busiest = int(run["plan"].group_sizes.argmax())
    _check_expert_slices(run, payloads, (go.Q4_K, go.Q4_K), lora, scaling, 0.0, sorted({0, 127, busiest}))
    for tokens in (slice(0, 512), slice(t - 512, t)):
        _check_permutes(run, hidden, idx, wts, gout, tokens)
    ops.check_status()


# ---------------------------------------------------------------------------------------------------------------------
# DeepSeek-shaped MoE block: 256 IQ2_XXS routed experts (top-6, hidden 4096, intermediate 2048, r = 8, clamped SwiGLU)
# plus the Q8_0 shared expert, 8192 tokens
# ---------------------------------------------------------------------------------------------------------------------
def test_deepseek_moe_block_at_benchmark_size_in_slices(cuda):
    import fast_lora
    from b2g import gguf_quant, ops
    from b2g.gguf_types import DeepseekV4GGUFExperts, GGUFQuantizedTensor
    from b2g.moe_block import SharedExpertLora, moe_block_forward
    from types import SimpleNamespace

    e, h, i, t, k, r, scaling, limit = 256, 4096, 2048, 8192, 6, 8, 2.0, 7.0
    g = torch.Generator().manual_seed(19260817 + 3)
    payloads = _bank(cuda, go.IQ2_XXS, e, h, i, 31)
    lora = _lora(cuda, e, h, i, r, g)
    hidden = torch.randn(t, h, generator=g).bfloat16().to(cuda)
    logits = torch.randn(t, e, generator=g).to(cuda)
    gout = torch.randn(t, h, generator=g).bfloat16().to(cuda)
    idx = ops.router_topk(logits, k, None, False)
    wts = torch.softmax(logits.gather(1, idx), -1)

    # shared expert: Q8_0, 4096 -> 2048 -> 4096, r = 8, alpha = 16
    sw = [torch.randn(shape, generator=g) * 0.02 for shape in ((i, h), (i, h), (h, i))]
    sp = [gguf_quant.quantize_q8_0(w).to(cuda) for w in sw]
    shared = SharedExpertLora(*(GGUFQuantizedTensor(p, quant_type=go.Q8_0, logical_shape=tuple(w.shape)) for p, w in zip(sp, sw)),
                              r=r, lora_alpha=16, swiglu_limit=limit)
    with torch.no_grad():
        for name in ("gate", "up", "down"):
            shared.lora_A[name].copy_((torch.randn(shared.lora_A[name].shape, generator=g) / 16).bfloat16())
            shared.lora_B[name].copy_((torch.randn(shared.lora_B[name].shape, generator=g) * 0.01).bfloat16())

    run = _run_routed(cuda, payloads, (go.IQ2_XXS, go.IQ2_XXS), e, h, i, hidden, idx, wts, lora, scaling, limit, gout, shared)
    busiest = int(run["plan"].group_sizes.argmax())
    _check_expert_slices(run, payloads, (go.IQ2_XXS, go.IQ2_XXS), lora, scaling, limit, sorted({0, 127, busiest}))

    # shared expert on the first and last 512 tokens (rows are independent), then its factor gradients on a 512-token call
    shared_w = [dense_ref.dequant_bf16(p.cpu().numpy(), go.Q8_0) for p in sp]
    shared_lora = {n: (shared.lora_A[n].detach().cpu(), shared.lora_B[n].detach().cpu()) for n in ("gate", "up", "down")}
    for tokens in (slice(0, 512), slice(t - 512, t)):
        sref = dense_ref.shared_expert_fwd_bwd(hidden[tokens].cpu(), *shared_w, shared_lora, scaling, gout[tokens].cpu(), limit)
        _check_permutes(run, hidden, idx, wts, gout, tokens, shared_dx=sref["dx"], shared_y=sref["y"])
    full_grads = {n: (shared.lora_A[n].grad.clone(), shared.lora_B[n].grad.clone()) for n in ("gate", "up", "down")}
    shared.zero_grad()
    xs = hidden[:512].clone().requires_grad_(True)
    ys = shared(xs)
    ys.backward(gout[:512])
    sref = dense_ref.shared_expert_fwd_bwd(hidden[:512].cpu(), *shared_w, shared_lora, scaling, gout[:512].cpu(), limit)
    assert dense_ref.rel_l2(ys, sref["y"]) < TOL and dense_ref.rel_l2(xs.grad, sref["dx"]) < TOL
    for n in ("gate", "up", "down"):
        assert dense_ref.rel_l2(shared.lora_A[n].grad, sref[f"d_{n}_a"]) < TOL, n
        assert dense_ref.rel_l2(shared.lora_B[n].grad, sref[f"d_{n}_b"]) < TOL, n

    # the same block through the module surface (wrapper, registry, one entry point) gives the same bits
    from deepseek_v4_moe_lora import DeepseekV4GGUFMoeLora, EXPERTS_IMPLEMENTATION, deepseek_v4_gguf_dequant_aiter_lora_forward
    from b2g.gguf_types import ALL_GGUF_EXPERTS_FUNCTIONS

    if fast_lora.HAVE_PEFT:
        return
    cfg = SimpleNamespace(num_experts=e, hidden_size=h, moe_intermediate_size=i, hidden_act="silu", swiglu_limit=limit,
                          _experts_implementation=EXPERTS_IMPLEMENTATION)
    bank = DeepseekV4GGUFExperts(cfg, device=cuda, compute_dtype=torch.bfloat16)
    for name, p, shape in zip(("gate_proj", "up_proj", "down_proj"), payloads, ((e, i, h), (e, i, h), (e, h, i))):
        setattr(bank, name, GGUFQuantizedTensor(p, quant_type=go.IQ2_XXS, logical_shape=shape))
    ALL_GGUF_EXPERTS_FUNCTIONS[EXPERTS_IMPLEMENTATION] = deepseek_v4_gguf_dequant_aiter_lora_forward
    layer = DeepseekV4GGUFMoeLora(bank, "default", config=fast_lora.LoraConfig(target_modules=["experts"], r=r, lora_alpha=16), r=r, lora_alpha=16)
    with torch.no_grad():
        for mod, key in ((layer.lora_A, "gate_up_a"), (layer.lora_B, "gate_up_b"), (layer.lora_A_down, "down_a"), (layer.lora_B_down, "down_b")):
            mod["default"].weight.copy_(lora[key])
    shared.zero_grad()
    hc = hidden.clone().requires_grad_(True)
    out = moe_block_forward(hc, idx, wts, layer, shared)
    out.backward(gout)
    assert torch.equal(out, run["total"]) and torch.equal(hc.grad, run["d_hidden"])
    assert torch.equal(layer.lora_B_down["default"].weight.grad, lora["down_b"].grad)
    for n in ("gate", "up", "down"):
        assert torch.equal(shared.lora_A[n].grad, full_grads[n][0]) and torch.equal(shared.lora_B[n].grad, full_grads[n][1])
    ops.check_status()
