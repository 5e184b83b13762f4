"""GPU: dense quantized LoRA linear against the dequantize-then-matmul oracle.

Tolerance: relative L2 <= 1e-2 on outputs and gradients (bf16), the bar the task states; the
kernels land near 2e-3, which is bf16 rounding of the result itself.
"""
import numpy as np
import pytest
import torch
from torch.utils._python_dispatch import TorchDispatchMode

from oracle import dense_ref, gguf_oracle as go

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _case(qtype, m, n, k, r, seed, encoder="quantize"):
    g = torch.Generator().manual_seed(seed)
    rng = np.random.default_rng(seed)
    if encoder == "quantize":
        payload = go.quantize((rng.standard_normal((n, k)) * 0.02).astype(np.float32), qtype)
    else:
        payload = go.random_payload(qtype, (n, k), seed)
    x = torch.randn(m, k, generator=g).bfloat16()
    dy = torch.randn(m, n, generator=g).bfloat16()
    a = (torch.randn(r, k, generator=g) / 16).bfloat16()
    b = (torch.randn(n, r, generator=g) * 0.01).bfloat16()
    return payload, x, dy, a, b


@pytest.mark.parametrize("qtype,m,n,k,r", [
    (go.Q4_K, 300, 512, 1024, 16), (go.Q4_K, 33, 37, 256, 4), (go.Q4_K, 1, 8, 256, 1), (go.Q4_K, 513, 768, 2048, 8),
    (go.Q8_0, 300, 512, 1024, 16), (go.Q8_0, 129, 200, 512, 4),
    (go.IQ2_XXS, 260, 512, 2048, 8), (go.IQ2_XXS, 64, 300, 4096, 16),
    (go.Q6_K, 700, 512, 2048, 16), (go.Q6_K, 130, 264, 4096, 4), (go.Q6_K, 1, 8, 2048, 1),
    (go.Q5_K, 600, 512, 1024, 16), (go.Q5_K, 77, 200, 256, 3),
    (go.Q2_K, 600, 512, 1024, 16), (go.Q2_K, 300, 264, 3072, 5),
    (go.Q3_K, 600, 512, 2048, 16), (go.Q3_K, 70, 136, 4096, 2),
    (go.IQ2_S, 400, 512, 2048, 16), (go.IQ2_S, 70, 72, 4096, 2),
])
def test_fused_lora_linear_forward_backward(cuda, qtype, m, n, k, r):
    from b2g import autograd as ag

    payload, x, dy, a, b = _case(qtype, m, n, k, r, 1000 + m)
    s = 2.0
    ref = dense_ref.lora_linear_fwd_bwd(x, dense_ref.dequant_bf16(payload, qtype), a, b, s, dy, torch.float32)
    xc = x.to(cuda).requires_grad_(True)
    ac, bc = a.to(cuda).requires_grad_(True), b.to(cuda).requires_grad_(True)
    pc = torch.from_numpy(payload).to(cuda)
    y = ag.lora_qlinear(xc, pc, qtype, n, ac, bc, s)
    y.backward(dy.to(cuda))
    assert dense_ref.rel_l2(y, ref["y"]) < TOL
    assert dense_ref.rel_l2(xc.grad, ref["dx"]) < TOL
    assert dense_ref.rel_l2(ac.grad, ref["da"]) < TOL
    assert dense_ref.rel_l2(bc.grad, ref["db"]) < TOL
    assert y.dtype == torch.bfloat16 and xc.grad.shape == x.shape and bc.grad.shape == b.shape


@pytest.mark.parametrize("qtype,m,n,k,r", [
    (go.IQ2_XXS, 200, 512, 512, 8), (go.IQ2_S, 200, 264, 256, 4), (go.Q3_K, 300, 512, 512, 16), (go.Q6_K, 130, 256, 768, 16),
    (go.Q2_K, 150, 520, 512, 2),
])
def test_row_pitches_that_are_not_16_byte_multiples(cuda, qtype, m, n, k, r):
    """Widths whose packed rows are not multiples of 16 bytes (a 512-wide IQ2_XXS row is 132 bytes: the down projection of
    the Qwen experts): the wrapper pads the rows and flags the type id, results as for any other width."""
    from b2g import autograd as ag, ops

    assert ops.payload_row_bytes(qtype, k) % 16 != 0
    payload, x, dy, a, b = _case(qtype, m, n, k, r, 2000 + m, encoder="random" if qtype in (go.IQ2_XXS, go.IQ2_S) else "quantize")
    ref = dense_ref.lora_linear_fwd_bwd(x, dense_ref.dequant_bf16(payload, qtype), a, b, 2.0, dy, torch.float32)
    xc = x.to(cuda).requires_grad_(True)
    ac, bc = a.to(cuda).requires_grad_(True), b.to(cuda).requires_grad_(True)
    y = ag.lora_qlinear(xc, torch.from_numpy(payload).to(cuda), qtype, n, ac, bc, 2.0)
    y.backward(dy.to(cuda))
    assert dense_ref.rel_l2(y, ref["y"]) < TOL
    assert dense_ref.rel_l2(xc.grad, ref["dx"]) < TOL
    assert dense_ref.rel_l2(ac.grad, ref["da"]) < TOL
    assert dense_ref.rel_l2(bc.grad, ref["db"]) < TOL


def test_config0_q8_lora_linear(cuda):
    """The CPU-runnable benchmark configuration: Q8_0 2048x2048, r=16, alpha=32, 4096 tokens; also the bf16 oracle itself
    must sit inside the same tolerance of the fp32 oracle."""
    from b2g import autograd as ag

    payload, x, dy, a, b = _case(go.Q8_0, 4096, 2048, 2048, 16, 19260817)
    w = dense_ref.dequant_bf16(payload, go.Q8_0)
    ref32 = dense_ref.lora_linear_fwd_bwd(x, w, a, b, 2.0, dy, torch.float32)
    ref16 = dense_ref.lora_linear_fwd_bwd(x, w, a, b, 2.0, dy, torch.bfloat16)
    xc = x.to(cuda).requires_grad_(True)
    ac, bc = a.to(cuda).requires_grad_(True), b.to(cuda).requires_grad_(True)
    y = ag.lora_qlinear(xc, torch.from_numpy(payload).to(cuda), go.Q8_0, 2048, ac, bc, 2.0)
    y.backward(dy.to(cuda))
    for got, key in ((y, "y"), (xc.grad, "dx"), (ac.grad, "da"), (bc.grad, "db")):
        assert dense_ref.rel_l2(got, ref32[key]) < TOL
        assert dense_ref.rel_l2(got, ref16[key]) < TOL


def test_mmq_operator_nd_input_bias_free_and_dispatch(cuda):
    """mmq accepts N-D activations (test_fast_lora.py:137), its autograd is mmq_grad_input
    (test_fast_lora.py:104-105) and the packed payload never receives a gradient (:135)."""
    from b2g import autograd as ag

    payload, x, dy, _, _ = _case(go.Q4_K, 33, 37, 2048, 4, 2468)
    w = dense_ref.dequant_bf16(payload, go.Q4_K)
    x3 = x.reshape(3, 11, 2048).to(cuda).requires_grad_(True)
    pc = torch.from_numpy(payload).to(cuda)
    seen = []

    class Rec(TorchDispatchMode):
        def __torch_dispatch__(self, func, types, args=(), kwargs=None):
            seen.append(str(func))
            return func(*args, **(kwargs or {}))

    with Rec():
        y = ag.mmq(x3, pc, go.Q4_K, 37)
        y.backward(dy.reshape(3, 11, 37).to(cuda))
    assert "b2g.mmq.default" in seen and "b2g.mmq_grad_input.default" in seen
    assert y.shape == (3, 11, 37)
    assert dense_ref.rel_l2(y.reshape(33, 37), x.float() @ w.float().t()) < TOL
    assert dense_ref.rel_l2(x3.grad.reshape(33, 2048), dy.float() @ w.float()) < TOL
    assert pc.grad is None
    direct = ag.mmq_grad_input(dy.to(cuda), pc, go.Q4_K, 2048)
    assert torch.equal(direct, x3.grad.reshape(33, 2048))


def test_bias_and_separate_lora_add(cuda):
    from b2g import ops

    payload, x, _, a, b = _case(go.Q4_K, 200, 256, 512, 16, 77)
    bias = torch.randn(256, generator=torch.Generator().manual_seed(1)).bfloat16()
    w = dense_ref.dequant_bf16(payload, go.Q4_K)
    y = ops.qlinear_fwd(x.to(cuda), torch.from_numpy(payload).to(cuda).reshape(-1), go.Q4_K, 256, bias.to(cuda))
    assert dense_ref.rel_l2(y, x.float() @ w.float().t() + bias.float()) < TOL


def test_results_are_bitwise_reproducible(cuda):
    from b2g import autograd as ag

    payload, x, dy, a, b = _case(go.Q4_K, 700, 512, 1024, 16, 5)
    outs = []
    for _ in range(2):
        xc = x.to(cuda).requires_grad_(True)
        ac, bc = a.to(cuda).requires_grad_(True), b.to(cuda).requires_grad_(True)
        y = ag.lora_qlinear(xc, torch.from_numpy(payload).to(cuda), go.Q4_K, 512, ac, bc, 2.0)
        y.backward(dy.to(cuda))
        outs.append((y.detach().clone(), xc.grad.clone(), ac.grad.clone(), bc.grad.clone()))
    for u, v in zip(*outs):
        assert torch.equal(u, v)


def test_linearity_at_full_width(cuda):
    """Size-independent property at a config-sized layer (N=4096, K=2048, M=8192):
    f(x1 + x2) = f(x1) + f(x2) up to bf16 rounding, and f(0) = 0 exactly."""
    from b2g import gguf_quant, ops

    g = torch.Generator(device=cuda).manual_seed(3)
    payload = gguf_quant.random_payload(12, (4096, 2048), 4, device=cuda).reshape(-1)
    x1 = torch.randn(8192, 2048, generator=g, device=cuda).bfloat16()
    x2 = torch.randn(8192, 2048, generator=g, device=cuda).bfloat16()
    xs = x1 + x2
    y1, y2, ys = (ops.qlinear_fwd(t, payload, 12, 4096) for t in (x1, x2, xs))
    exact_sum = (x1.float() + x2.float())
    # xs itself was rounded to bf16, so compare against the two-term sum with the rounding error of xs allowed
    assert dense_ref.rel_l2(ys, y1.float() + y2.float()) < 1e-2
    assert float(ops.qlinear_fwd(torch.zeros_like(x1), payload, 12, 4096).abs().max()) == 0.0
    del exact_sum


def test_full_width_every_element_repeated(cuda):
    """Every output element of a config-sized product (M=8192, N=4096, K=2048) against the product with the exactly
    dequantised weight, three runs in a row, forward and input gradient.  A norm hides a few hundred wrong elements;
    a hand-off race between the warp roles of the kernel shows up exactly so: in some runs, in some tiles."""
    from b2g import gguf_quant, ops

    g = torch.Generator(device=cuda).manual_seed(3)
    n, k, m = 4096, 2048, 8192
    payload = gguf_quant.random_payload(12, (n, k), 4, device=cuda).reshape(-1)
    w = ops.dequantize(payload, 12, (n, k)).float()
    x = torch.randn(m, k, generator=g, device=cuda).bfloat16()
    dy = torch.randn(m, n, generator=g, device=cuda).bfloat16()
    ref_y, ref_dx = x.float() @ w.t(), dy.float() @ w
    for _ in range(3):
        y = ops.qlinear_fwd(x, payload, 12, n).float()
        dx = ops.qlinear_dgrad(dy, payload, 12, k).float()
        for got, ref in ((y, ref_y), (dx, ref_dx)):
            bad = (got - ref).abs() > 0.02 * ref.abs() + 0.02 * float(ref.abs().mean())
            assert int(bad.sum()) == 0, f"{int(bad.sum())} elements off, first at {bad.nonzero()[0].tolist()}"


def test_fail_closed_arguments(cuda):
    from b2g import _lib, autograd as ag, ops

    p = torch.zeros(8 * 144, dtype=torch.uint8, device=cuda)
    x = torch.zeros(4, 256, dtype=torch.float32, device=cuda)
    with pytest.raises(TypeError):
        ag.mmq(x, p, 12, 8)
    xb = torch.zeros(4, 512, dtype=torch.bfloat16, device=cuda)[:, ::2]
    with pytest.raises(RuntimeError, match="contiguous"):
        ag.mmq(xb, p, 12, 8)
    with pytest.raises(ValueError):
        ops.qlinear_fwd(torch.zeros(4, 256, dtype=torch.bfloat16, device=cuda), p[:-1], 12, 8)
    # 66-byte rows are not TMA-compatible as they are: the wrapper pads them; the C entry point refuses them unpadded
    assert ops.qlinear_fwd(torch.zeros(4, 256, dtype=torch.bfloat16, device=cuda), torch.zeros(8 * 66, dtype=torch.uint8, device=cuda), 16, 8).shape == (4, 8)
    with pytest.raises(ValueError, match="B2G_PADDED_ROWS"):
        _lib.call("b2g_qlinear_fwd", 16, None, None, None, None, None, None, 4, 8, 256, None, None)
    with pytest.raises(ValueError):
        ag.lora_qlinear(torch.zeros(4, 256, dtype=torch.bfloat16, device=cuda), p, 12, 8,
                        torch.zeros(32, 256, device=cuda), torch.zeros(8, 32, device=cuda), 1.0)
    assert ag.mmq(torch.zeros(0, 256, dtype=torch.bfloat16, device=cuda), p, 12, 8).shape == (0, 8)


def test_a_bounded_wait_that_runs_out_reports_and_returns(cuda):
    """The give-up path of the kernel's waits, exercised without faulting or hanging anything: a test entry launches the forward
    product with its packed-weight producer held back and a short wait limit.  The unpack warps' wait (site 401) runs out, all
    roles drain, the kernel returns, the status word says which wait gave up, and the next ordinary launch is correct."""
    import ctypes as C

    from b2g import _lib, gguf_quant, ops

    m, n, k = 1024, 512, 1024
    g = torch.Generator().manual_seed(5)
    x = torch.randn(m, k, generator=g).bfloat16().to(cuda)
    payload = gguf_quant.quantize_q4_k(torch.randn(n, k, generator=g) * 0.02).to(cuda).reshape(-1)
    good = ops.qlinear_fwd(x, payload, go.Q4_K, n)
    ops.check_status()
    y = torch.empty(m, n, dtype=torch.bfloat16, device=cuda)
    status = ops.status_word(cuda)
    _lib.call("b2g_debug_stalled_qlinear_fwd", go.Q4_K, C.c_void_p(x.data_ptr()), C.c_void_p(payload.data_ptr()), C.c_void_p(y.data_ptr()),
              m, n, k, 256, C.c_void_p(status.data_ptr()), C.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()                                     # the kernel came back
    assert int(status.item()) == 401
    with pytest.raises(Exception, match="bounded wait"):
        ops.check_status()
    ops.check_status()                                           # the word was cleared by the report
    again = ops.qlinear_fwd(x, payload, go.Q4_K, n)
    assert torch.equal(again, good)
    with pytest.raises(ValueError, match="spin limit"):
        _lib.call("b2g_debug_stalled_qlinear_fwd", go.Q4_K, C.c_void_p(x.data_ptr()), C.c_void_p(payload.data_ptr()), C.c_void_p(y.data_ptr()),
                  m, n, k, 1 << 20, C.c_void_p(status.data_ptr()), None)
