"""GPU: the fixed-group packed projection (DeepSeek's frozen eight-group Q8_0 o_a_proj).

The reference's own check (test_deepseek_v4_lora.py:101-152) demands EXACT equality, forward and input gradient, with
per-group dense ``mmq`` calls on contiguous slices; that is asserted here through the same module surface
(``GGUFGroupedLinear`` + ``configure_deepseek_v4_grouped_mmq``), next to the tolerance check against the CPU oracle.
"""
import numpy as np
import pytest
import torch

from oracle import dense_ref, gguf_oracle as go

pytestmark = pytest.mark.gpu


def _grouped_case(m_shape, groups, n, k, qtype, seed, cuda):
    rng = np.random.default_rng(seed)
    logical = (rng.standard_normal((groups * n, k)) * 0.05).astype(np.float32)
    payload = go.quantize(logical, qtype) if qtype not in (go.IQ2_XXS, go.IQ2_S) else go.random_payload(qtype, (groups * n, k), seed)
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(*m_shape, groups, k, generator=g).bfloat16()
    dy = torch.randn(*m_shape, groups, n, generator=g).bfloat16()
    return payload, x, dy


def test_deepseek_layout_equals_per_group_mmq_exactly(cuda):
    import deepseek_v4_lora as dsl
    from b2g import autograd as ag
    from b2g.gguf_types import GGUFGroupedLinear, GGUFQuantizedTensor

    payload, x, dy = _grouped_case((2, 3), 8, 1024, 4096, go.Q8_0, 42, cuda)
    packed = torch.from_numpy(payload).to(cuda)
    layer = GGUFGroupedLinear(4096, 8192, 8, device=cuda, dtype=torch.bfloat16, compute_dtype=torch.bfloat16)
    layer.weight = GGUFQuantizedTensor(packed, quant_type=go.Q8_0, logical_shape=(8192, 4096))
    assert dsl.configure_deepseek_v4_grouped_mmq(layer)["enabled"] == 1

    hidden = x.to(cuda).requires_grad_(True)
    out = layer(hidden)
    out.backward(dy.to(cuda))
    assert out.shape == (2, 3, 8, 1024) and out.dtype == torch.bfloat16

    ref_in = x.to(cuda).requires_grad_(True)
    groups = packed.reshape(8, 1024, -1)
    ref = torch.stack([ag.mmq(ref_in[..., g, :].contiguous(), groups[g].clone(), go.Q8_0, 1024) for g in range(8)], dim=-2)
    ref.backward(dy.to(cuda))
    assert torch.equal(out, ref)
    assert torch.equal(hidden.grad, ref_in.grad)
    assert layer.weight.grad is None

    w = dense_ref.dequant_bf16(payload, go.Q8_0).reshape(8, 1024, 4096)
    assert dense_ref.rel_l2(out, dense_ref.fixed_grouped(x, w)) < 1e-2
    assert dense_ref.rel_l2(hidden.grad, dense_ref.fixed_grouped_grad_input(dy, w)) < 1e-2


@pytest.mark.parametrize("qtype,groups,n,k,rows", [(go.Q4_K, 4, 512, 1024, 700), (go.Q8_0, 2, 48, 256, 33), (go.IQ2_XXS, 3, 256, 2048, 130),
                                                  (go.Q6_K, 2, 256, 2048, 300), (go.Q5_K, 3, 128, 512, 90), (go.Q2_K, 2, 128, 1024, 200), (go.Q3_K, 2, 256, 2048, 150), (go.IQ2_S, 2, 128, 2048, 100)])
def test_other_types_and_ragged_rows(cuda, qtype, groups, n, k, rows):
    from b2g import autograd as ag

    payload, x, dy = _grouped_case((rows,), groups, n, k, qtype, 7 + rows, cuda)
    packed = torch.from_numpy(payload).to(cuda).reshape(groups, n, -1)
    w = dense_ref.dequant_bf16(payload, qtype).reshape(groups, n, k)
    xc = x.to(cuda).requires_grad_(True)
    y = ag.fixed_grouped_mmq(xc, packed, qtype)
    y.backward(dy.to(cuda))
    assert dense_ref.rel_l2(y, dense_ref.fixed_grouped(x, w)) < 1e-2
    assert dense_ref.rel_l2(xc.grad, dense_ref.fixed_grouped_grad_input(dy, w)) < 1e-2


def test_fail_closed(cuda):
    from b2g import autograd as ag

    packed = torch.zeros(8, 1024, 4352, dtype=torch.uint8, device=cuda)
    with pytest.raises(ValueError, match="groups"):
        ag.fixed_grouped_mmq(torch.zeros(2, 4, 4096, dtype=torch.bfloat16, device=cuda), packed, 8)
    with pytest.raises(ValueError, match="width"):
        ag.fixed_grouped_mmq(torch.zeros(2, 8, 2048, dtype=torch.bfloat16, device=cuda), packed, 8)
    with pytest.raises(RuntimeError, match="contiguous"):
        ag.fixed_grouped_mmq(torch.zeros(2, 8, 8192, dtype=torch.bfloat16, device=cuda)[..., ::2], packed, 8)
    with pytest.raises(ValueError, match="not supported natively"):
        ag.fixed_grouped_mmq(torch.zeros(2, 8, 4096, dtype=torch.bfloat16, device=cuda), packed, 2)
    empty = ag.fixed_grouped_mmq(torch.zeros(0, 8, 4096, dtype=torch.bfloat16, device=cuda), packed, 8)
    assert empty.shape == (0, 8, 1024)
