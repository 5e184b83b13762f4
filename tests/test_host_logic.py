"""CPU: host-side logic of the package (no kernels run)."""
import numpy as np
import pytest
import torch

from oracle import gguf_oracle as go


def test_payload_geometry():
    from b2g import ops

    assert ops.payload_row_bytes(12, 2048) == 1152 and ops.payload_row_bytes(8, 2048) == 2176
    assert ops.payload_row_bytes(16, 4096) == 1056
    with pytest.raises(ValueError):
        ops.payload_row_bytes(12, 100)


def test_torch_encoders_match_oracle_encoders():
    from b2g import gguf_quant

    w = torch.randn(32, 1024, generator=torch.Generator().manual_seed(1)) * 0.02
    assert np.array_equal(gguf_quant.quantize_q8_0(w).numpy(), go.quantize(w.numpy(), go.Q8_0))
    assert np.array_equal(gguf_quant.quantize_q4_k(w).numpy(), go.quantize(w.numpy(), go.Q4_K))
    for qt in (8, 10, 11, 12, 13, 14, 16, 22):
        p = gguf_quant.random_payload(qt, (3, 2, 2048), 5)
        d = go.dequantize(p.numpy(), qt)
        assert np.isfinite(d).all() and 0.005 < d.std() < 0.06


def test_rank_padding():
    from b2g import ops

    b = torch.randn(5, 4).bfloat16()
    pb = ops.pad_rank_cols(b)
    assert pb.shape == (5, 16) and torch.equal(pb[:, :4], b) and float(pb[:, 4:].abs().max()) == 0
    a = torch.randn(3, 8, 32).bfloat16()
    pa = ops.pad_rank_rows(a)
    assert pa.shape == (3, 16, 32) and torch.equal(pa[:, :8], a)
    full = torch.randn(7, 16).bfloat16()
    assert ops.pad_rank_cols(full).data_ptr() == full.data_ptr()


def test_cpu_tensors_are_rejected_not_routed_elsewhere():
    from b2g import autograd as ag, ops

    x = torch.zeros(4, 256, dtype=torch.bfloat16)
    p = torch.zeros(8 * 144, dtype=torch.uint8)
    with pytest.raises(RuntimeError, match="CUDA"):
        ops.qlinear_fwd(x, p, 12, 8)
    with pytest.raises((RuntimeError, NotImplementedError)):
        ag.mmq(x, p, 12, 8)
    with pytest.raises(RuntimeError, match="CUDA"):
        ops.dequantize(p, 12, (8, 256))


def test_operators_registered_with_meta_kernels():
    from b2g import autograd as ag  # noqa: F401

    x = torch.empty(3, 5, 256, dtype=torch.bfloat16, device="meta")
    p = torch.empty(64 * 144, dtype=torch.uint8, device="meta")
    assert torch.ops.b2g.mmq(x, p, 12, 64).shape == (3, 5, 64)
    g = torch.empty(7, 64, dtype=torch.bfloat16, device="meta")
    assert torch.ops.b2g.mmq_grad_input(g, p, 12, 256).shape == (7, 256)
    idx = torch.empty(2, dtype=torch.int64, device="meta")
    off = torch.empty(2, dtype=torch.int32, device="meta")
    y0, y1 = torch.ops.b2g.grouped_mmq_pair(g.new_empty(7, 256), p, p, idx, off, 12, 32)
    assert y0.shape == (7, 32) and y1.shape == (7, 32)


def test_bench_flop_formula():
    import bench

    m = 32768
    assert bench.flops_per_step(m) == sum(4 * m * n * 2048 + 6 * m * 16 * (2048 + n) for n in (4096, 512, 2048))


def test_oracle_dense_reference_shapes():
    from oracle import dense_ref

    g = torch.Generator().manual_seed(0)
    w = go.quantize((np.random.default_rng(0).standard_normal((24, 256)) * 0.02).astype(np.float32), go.Q4_K)
    wb = dense_ref.dequant_bf16(w, go.Q4_K)
    x = torch.randn(9, 256, generator=g).bfloat16()
    a = torch.randn(4, 256, generator=g).bfloat16()
    b = torch.randn(24, 4, generator=g).bfloat16()
    out = dense_ref.lora_linear_fwd_bwd(x, wb, a, b, 1.0, torch.randn(9, 24, generator=g).bfloat16())
    assert out["y"].shape == (9, 24) and out["dx"].shape == (9, 256) and out["da"].shape == (4, 256) and out["db"].shape == (24, 4)


def test_oracle_routing_reference_is_stable_and_consistent():
    from oracle import moe_ref

    idx = torch.tensor([[3, 1], [1, 3], [0, 1]])
    plan = moe_ref.route_plan(idx, 4)
    assert plan["expert_indices"].tolist() == [0, 1, 1, 1, 3, 3]
    assert plan["permutation"].tolist() == [4, 1, 2, 5, 0, 3]           # equal ids keep flat order
    assert plan["group_sizes"].tolist() == [1, 3, 0, 2] and plan["offsets"].tolist() == [1, 4, 4, 6]
    logits = torch.zeros(2, 256)
    assert moe_ref.router_topk(logits, 8).tolist() == [list(range(8))] * 2  # ties -> smaller id


def test_bench_clock_sampler_reads_samples_under_load(tmp_path, monkeypatch):
    """The bench's clock sampler against a fake `nvidia-smi` (a script printing one CSV row every 20 ms): only rows that
    arrive while the load runs are summarised, and a too-short timed region is extended by untimed steps."""
    import os
    import stat
    import time

    import bench

    fake = tmp_path / "nvidia-smi"
    fake.write_text("#!/bin/sh\nwhile true; do echo '0, 1905, 1965, 801.5, 0x4, Not Active, Not Active, Not Active, Active'; sleep 0.02; done\n")
    fake.chmod(fake.stat().st_mode | stat.S_IEXEC)
    monkeypatch.setenv("PATH", f"{tmp_path}{os.pathsep}{os.environ['PATH']}")
    s = bench.ClockSampler(0)
    s.start()
    time.sleep(0.1)
    s.begin()
    s.end()                                             # a timed region too short for any sample
    steps = []
    s.extend(lambda: (steps.append(1), time.sleep(0.01)), lambda: None)
    out = s.stop()
    assert out["samples"] >= bench.ClockSampler.MIN_SAMPLES and steps
    assert out["sm_mhz"] == 1905 and out["sm_max_mhz"] == 1965 and out["reasons"] == ["sw_power_cap"]
    assert "untimed" in out["window"]


def test_deepseek_fixed_group_module_contract():
    """configure_deepseek_v4_grouped_mmq (deepseek_v4_lora.py:128-162): patches matching frozen grouped projections, fails
    closed on anything else, refuses grouped adapters; the operator has a Meta kernel with the reference's shapes."""
    import deepseek_v4_lora as dsl
    from b2g.gguf_types import GGUFGroupedLinear, GGUFQuantizedTensor

    good = GGUFGroupedLinear(4096, 8192, 8)
    good.weight = GGUFQuantizedTensor(torch.zeros(8192, 4352, dtype=torch.uint8), quant_type=8, logical_shape=(8192, 4096))
    holder = torch.nn.Sequential(good)
    assert dsl.configure_deepseek_v4_grouped_mmq(holder) == {"enabled": 1, "paths": ["0"]}
    assert good._deepseek_v4_grouped_mmq_enabled and dsl.configure_deepseek_v4_grouped_mmq(holder)["enabled"] == 1
    with pytest.raises(RuntimeError, match="contiguous|CUDA|cuda"):          # no CPU route behind the patched forward
        good(torch.zeros(2, 8, 4096, dtype=torch.bfloat16))

    small = GGUFGroupedLinear(32, 24, 4)
    small.weight = GGUFQuantizedTensor(torch.zeros(24, 34, dtype=torch.uint8), quant_type=8, logical_shape=(24, 32))
    with pytest.raises(RuntimeError, match="fixed eight-group"):
        dsl.configure_deepseek_v4_grouped_mmq(small)
    plain = GGUFGroupedLinear(4096, 8192, 8)
    plain.weight = torch.zeros(8192, 4352, dtype=torch.uint8)
    with pytest.raises(TypeError, match="not GGUF-quantized"):
        dsl.configure_deepseek_v4_grouped_mmq(plain)
    with pytest.raises(RuntimeError, match="grouped o_a_proj LoRA is unsupported"):
        dsl._RejectedDeepseekV4GroupedLora(good, "default")

    y = torch.ops.b2g.fixed_grouped_mmq(torch.empty(3, 2, 8, 4096, device="meta", dtype=torch.bfloat16),
                                        torch.empty(8, 1024, 4352, device="meta", dtype=torch.uint8), 8)
    assert tuple(y.shape) == (3, 2, 8, 1024)
    dx = torch.ops.b2g.fixed_grouped_mmq_grad_input(torch.empty(5, 8, 1024, device="meta", dtype=torch.bfloat16),
                                                    torch.empty(8, 1024, 4352, device="meta", dtype=torch.uint8), 8)
    assert tuple(dx.shape) == (5, 8, 4096)


def test_oracle_fixed_groups_equal_per_group_linear():
    from oracle import dense_ref

    g = torch.Generator().manual_seed(7)
    x, w, dy = torch.randn(3, 4, 64, generator=g), torch.randn(4, 24, 64, generator=g), torch.randn(3, 4, 24, generator=g)
    y = dense_ref.fixed_grouped(x, w)
    for k in range(4):
        assert torch.equal(y[:, k], x[:, k] @ w[k].t())
    xr = x.clone().requires_grad_(True)
    dense_ref.fixed_grouped(xr, w).backward(dy)
    assert torch.allclose(xr.grad, dense_ref.fixed_grouped_grad_input(dy, w), atol=1e-5)


def test_packed_lm_head_loss_argument_contract():
    """Argument checks of the packed LM-head loss run before anything touches a device (gguf_liger_loss.py:60-86,
    deepseek_v4_liger_loss.py:235-272)."""
    import deepseek_v4_liger_loss as dl
    from b2g.gguf_types import GGUFLinear, GGUFQuantizedTensor

    fwd = dl._packed_q8_linear_cross_entropy_forward
    h, p, t = torch.zeros(4, 256, dtype=torch.bfloat16), torch.zeros(37 * 272, dtype=torch.uint8), torch.zeros(4, dtype=torch.long)
    with pytest.raises(ValueError, match="two-dimensional"):
        fwd(h[None], p, t, 8, 37, 512, -100, 0.0, 0.0, "mean", None)
    with pytest.raises(TypeError, match="BF16"):
        fwd(h.float(), p, t, 8, 37, 512, -100, 0.0, 0.0, "mean", None)
    with pytest.raises(ValueError, match="match the hidden-state row count"):
        fwd(h, p, t[:3], 8, 37, 512, -100, 0.0, 0.0, "mean", None)
    with pytest.raises(TypeError, match="torch.long"):
        fwd(h, p, t.int(), 8, 37, 512, -100, 0.0, 0.0, "mean", None)
    with pytest.raises(ValueError, match="mean or sum"):
        fwd(h, p, t, 8, 37, 512, -100, 0.0, 0.0, "none", None)
    with pytest.raises(ValueError, match="chunk_size"):
        fwd(h, p, t, 8, 37, 0, -100, 0.0, 0.0, "mean", None)

    head = GGUFLinear(256, 37)
    head.weight = GGUFQuantizedTensor(torch.zeros(37, 272, dtype=torch.uint8), quant_type=8, logical_shape=(37, 256))
    labels = torch.zeros(1, 4, dtype=torch.long)
    for kw, msg in (({"label_smoothing": 0.1}, "label_smoothing"), ({"return_z_loss": True}, "return_z_loss"),
                    ({"accum_dtype": torch.bfloat16}, "FP32 internal accumulation")):
        with pytest.raises(RuntimeError, match=msg):
            dl.deepseek_v4_packed_liger_causal_lm_loss(h[None], head, labels, hidden_size=256, loss_kwargs=kw)
    with pytest.raises(RuntimeError, match="hidden size does not match"):
        dl.deepseek_v4_packed_liger_causal_lm_loss(h[None], head, labels, hidden_size=128)
    head.weight = GGUFQuantizedTensor(torch.zeros(37, 144, dtype=torch.uint8), quant_type=2, logical_shape=(37, 256))   # Q4_0
    with pytest.raises(RuntimeError, match="validated only for Q8_0"):
        dl.deepseek_v4_packed_liger_causal_lm_loss(h[None], head, labels, hidden_size=256)


def test_oracle_lm_head_loss_matches_autograd_of_plain_torch():
    from oracle import loss_ref

    g = torch.Generator().manual_seed(11)
    h = torch.randn(19, 64, generator=g).bfloat16()
    w = (torch.randn(37, 64, generator=g) * 0.3).bfloat16()
    t = torch.randint(0, 37, (19,), generator=g)
    t[5] = -100
    for reduction in ("mean", "sum"):
        o = loss_ref.packed_linear_cross_entropy(h, w, t, -100, reduction)
        logits = o["logits"].clone().requires_grad_(True)
        ref = torch.nn.functional.cross_entropy(logits, t, ignore_index=-100, reduction=reduction)
        ref.backward()
        assert torch.allclose(o["loss"], ref, rtol=1e-6, atol=1e-6)
        assert torch.allclose(o["grad_input"], logits.grad.bfloat16().float() @ w.float(), rtol=1e-5, atol=1e-6)
        assert int(o["predicted"][5]) == -1
