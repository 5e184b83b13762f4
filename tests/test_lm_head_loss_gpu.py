"""GPU: packed LM-head chunked cross-entropy against the CPU oracle.

Tolerances: the loss within rtol = atol = 1e-3 (the reference's own bar between its packed and logical losses,
test_deepseek_v4_liger_loss.py:134); the input gradient within relative L2 <= 1e-2; predicted tokens exact wherever the
top two logits differ.
"""
import numpy as np
import pytest
import torch
from torch.utils._python_dispatch import TorchDispatchMode

from oracle import dense_ref, gguf_oracle as go, loss_ref

pytestmark = pytest.mark.gpu


def _head(vocab, hidden, qtype, seed):
    rng = np.random.default_rng(seed)
    payload = go.quantize((rng.standard_normal((vocab, hidden)) * 0.08).astype(np.float32), qtype)
    return payload, dense_ref.dequant_bf16(payload, qtype)


@pytest.mark.parametrize("qtype,vocab,hidden,rows,chunk,reduction", [
    (go.Q8_0, 37, 256, 34, 512, "mean"),          # the reference's toy shape: odd vocabulary -> element path of the kernel
    (go.Q8_0, 4096, 512, 700, 256, "mean"),       # several chunks, ragged last one
    (go.Q4_K, 2048, 1024, 300, 128, "sum"),
    (go.Q6_K, 1032, 2048, 520, 256, "mean"),      # the Qwen head's type and hidden size
])
def test_loss_and_input_gradient(cuda, qtype, vocab, hidden, rows, chunk, reduction):
    import deepseek_v4_liger_loss as dl

    payload, w = _head(vocab, hidden, qtype, 100 + vocab)
    g = torch.Generator().manual_seed(vocab)
    h = torch.randn(rows, hidden, generator=g).bfloat16()
    t = torch.randint(0, vocab, (rows,), generator=g)
    t[::7] = -100
    ref = loss_ref.packed_linear_cross_entropy(h, w, t, -100, reduction)

    hc = h.to(cuda).requires_grad_(True)
    loss, acc, pred = dl._PackedQ8LigerLinearCrossEntropyFunction.apply(
        hc, torch.from_numpy(payload).to(cuda), t.to(cuda), qtype, vocab, chunk, -100, 0.0, 0.0, reduction, None, True, True)
    (loss * 3.0).backward()
    torch.testing.assert_close(loss.cpu(), ref["loss"], rtol=1e-3, atol=1e-3)
    assert dense_ref.rel_l2(hc.grad, 3.0 * ref["grad_input"]) < 1e-2
    top2 = ref["logits"].topk(2, dim=-1).values
    clear = (top2[:, 0] - top2[:, 1]) > 0
    assert torch.equal(pred.cpu()[clear], ref["predicted"][clear])
    assert abs(float(acc) - float(ref["accuracy"])) < 2.0 / rows


def test_module_surface_dispatches_packed_products(cuda):
    """deepseek_v4_packed_liger_causal_lm_loss on a packed head: shifted labels, no logical weight, the two packed operators
    in the dispatch trace (test_deepseek_v4_liger_loss.py:90-138)."""
    import deepseek_v4_liger_loss as dl
    from b2g.gguf_types import GGUFLinear, GGUFQuantizedTensor

    payload, w = _head(37, 256, go.Q8_0, 9753)
    head = GGUFLinear(256, 37)
    head.weight = GGUFQuantizedTensor(torch.from_numpy(payload).to(cuda), quant_type=go.Q8_0, logical_shape=(37, 256))
    g = torch.Generator().manual_seed(9753)
    hidden = torch.randn(2, 17, 256, generator=g).bfloat16()
    labels = torch.randint(0, 37, (2, 17), generator=g)
    labels[1, 4] = -100
    shifted = torch.nn.functional.pad(labels, (0, 1), value=-100)[..., 1:].reshape(-1)
    ref = loss_ref.packed_linear_cross_entropy(hidden.reshape(-1, 256), w, shifted, -100, "mean")

    seen = []

    class Rec(TorchDispatchMode):
        def __torch_dispatch__(self, func, types, args=(), kwargs=None):
            seen.append(str(func))
            return func(*args, **(kwargs or {}))

    hc = hidden.to(cuda).requires_grad_(True)
    with Rec():
        loss = dl.deepseek_v4_packed_liger_causal_lm_loss(hc, head, labels.to(cuda), hidden_size=256)
        loss.backward()
    torch.testing.assert_close(loss.cpu(), ref["loss"], rtol=1e-3, atol=1e-3)
    assert dense_ref.rel_l2(hc.grad.reshape(-1, 256), ref["grad_input"]) < 1e-2
    assert "b2g.mmq.default" in seen and "b2g.mmq_grad_input.default" in seen
    assert head.weight.grad is None and torch.isfinite(hc.grad).all()

    # gradient accumulation: sum reduction divided by the caller's count
    hc2 = hidden.to(cuda).requires_grad_(True)
    n = int((shifted != -100).sum())
    loss2 = dl.deepseek_v4_packed_liger_causal_lm_loss(hc2, head, labels.to(cuda), hidden_size=256, loss_kwargs={"num_items_in_batch": n})
    torch.testing.assert_close(loss2.cpu(), ref["loss"], rtol=1e-3, atol=1e-3)


def test_all_targets_ignored_and_bad_label(cuda):
    from b2g import ops

    logits = torch.randn(5, 64, device=cuda).bfloat16()
    target = torch.full((5,), -100, dtype=torch.long, device=cuda)
    loss = torch.empty(5, device=cuda)
    count = (target != -100).sum().reshape(1)
    ops.cross_entropy_inplace(logits, target, loss, count, True)
    assert float(loss.abs().sum()) == 0.0 and float(logits.float().abs().sum()) == 0.0
    ops.check_status()
    logits = torch.randn(2, 64, device=cuda).bfloat16()
    target = torch.tensor([3, 64], dtype=torch.long, device=cuda)      # 64 is outside the vocabulary
    ops.cross_entropy_inplace(logits, target, torch.empty(2, device=cuda), (target != -100).sum().reshape(1), True)
    with pytest.raises(Exception, match="902"):
        ops.check_status()


def test_qwen_entry_point_q6k_head(cuda):
    """gguf_liger_loss._packed_q8_liger_for_causal_lm_loss (gguf_liger_loss.py:268-355): Q6_K head, hidden 2048, with the
    optional token accuracy and predicted tokens; anything else is refused."""
    import gguf_liger_loss as gl
    from b2g.gguf_types import GGUFLinear, GGUFQuantizedTensor

    payload, w = _head(520, 2048, go.Q6_K, 31)
    head = GGUFLinear(2048, 520)
    head.weight = GGUFQuantizedTensor(torch.from_numpy(payload).to(cuda), quant_type=go.Q6_K, logical_shape=(520, 2048))
    g = torch.Generator().manual_seed(5)
    hidden = torch.randn(3, 40, 2048, generator=g).bfloat16()
    labels = torch.randint(0, 520, (3, 40), generator=g)
    labels[0, :5] = -100
    shifted = torch.nn.functional.pad(labels, (0, 1), value=-100)[..., 1:].reshape(-1)
    ref = loss_ref.packed_linear_cross_entropy(hidden.reshape(-1, 2048), w, shifted, -100, "mean")
    hc = hidden.to(cuda).requires_grad_(True)
    loss, z, acc, pred = gl._packed_q8_liger_for_causal_lm_loss(hc, head, labels.to(cuda), 2048, return_token_accuracy=True,
                                                                 return_predicted_tokens=True)
    loss.backward()
    assert z is None and pred.shape == (120,)
    torch.testing.assert_close(loss.cpu(), ref["loss"], rtol=1e-3, atol=1e-3)
    assert dense_ref.rel_l2(hc.grad.reshape(-1, 2048), ref["grad_input"]) < 1e-2
    assert abs(float(acc) - float(ref["accuracy"])) < 2.0 / 120
    q8_payload, _ = _head(520, 2048, go.Q8_0, 32)
    head.weight = GGUFQuantizedTensor(torch.from_numpy(q8_payload).to(cuda), quant_type=go.Q8_0, logical_shape=(520, 2048))
    with pytest.raises(RuntimeError, match="validated only for Q6_K"):
        gl._packed_q8_liger_for_causal_lm_loss(hc, head, labels.to(cuda), 2048)


def _fake_body(hidden_states, router_logits=None):
    """What a decoder stack returns to the causal-LM forward: the fields both patched forwards read."""
    from types import SimpleNamespace

    return SimpleNamespace(last_hidden_state=hidden_states, router_logits=router_logits, past_key_values=None, hidden_states=None,
                           attentions=None)


def test_deepseek_model_forward_patch_takes_the_packed_loss(cuda):
    """apply_deepseek_v4_liger_loss on a model instance (deepseek_v4_liger_loss.py:321-416): with labels the patched forward
    returns the packed-head loss and no logits, agrees with the loss that materialises the head (loss rel-err <= 5e-3, hidden
    gradient cosine >= 0.999, the gates of docs/plan_deepseek_v4.md:379-388), adds the router auxiliary loss when asked, and
    without labels runs the head on the kept positions."""
    import deepseek_v4_liger_loss as dl
    from types import SimpleNamespace
    from b2g.gguf_types import GGUFLinear, GGUFQuantizedTensor

    if dl.DeepseekV4ForCausalLM is not None:
        pytest.skip("transformers fork present: its own model class is patched there")
    vocab, hidden, batch, seq = 1024, 256, 2, 48
    payload, w = _head(vocab, hidden, go.Q8_0, 4242)

    class DeepseekV4ForCausalLM(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.lm_head = GGUFLinear(hidden, vocab)
            self.lm_head.weight = GGUFQuantizedTensor(torch.from_numpy(payload).to(cuda), quant_type=go.Q8_0, logical_shape=(vocab, hidden))
            self.config = SimpleNamespace(hidden_size=hidden, output_router_logits=False)
            self.num_experts, self.num_experts_per_tok, self.router_aux_loss_coef = 8, 2, 0.01
            self.embed = torch.nn.Embedding(vocab, hidden, device=cuda, dtype=torch.bfloat16)
            self.router_logits = None

        def model(self, input_ids=None, **kwargs):
            return _fake_body(self.embed(input_ids), self.router_logits)

    model = DeepseekV4ForCausalLM()
    assert dl.apply_deepseek_v4_liger_loss(model) is model
    g = torch.Generator().manual_seed(7)
    ids = torch.randint(0, vocab, (batch, seq), generator=g).to(cuda)
    labels = ids.clone()
    labels[:, -5:] = -100
    out = model(input_ids=ids, labels=labels)
    assert out.logits is None and out.loss.ndim == 0
    out.loss.backward()
    got_grad = model.embed.weight.grad.clone()
    model.embed.weight.grad = None
    want = dl.deepseek_v4_liger_causal_lm_loss(model.embed(ids), model.lm_head, labels, hidden_size=hidden)
    want.backward()
    assert abs(float(out.loss.detach()) - float(want.detach())) / float(want.detach()) <= 5e-3
    cos = torch.nn.functional.cosine_similarity(got_grad.float().flatten(), model.embed.weight.grad.float().flatten(), dim=0)
    assert float(cos) >= 0.999
    # CPU oracle of the same loss: shifted labels, mean over the kept positions
    h = model.embed(ids).detach().reshape(-1, hidden).cpu()
    shifted = torch.nn.functional.pad(labels, (0, 1), value=-100)[..., 1:].reshape(-1).cpu()
    ref = loss_ref.packed_linear_cross_entropy(h, w, shifted, -100, "mean")
    torch.testing.assert_close(out.loss.detach().cpu().float(), ref["loss"].float(), rtol=2e-3, atol=2e-3)
    # router auxiliary loss on top, as the stock forward adds it
    model.router_logits = tuple(torch.randn(batch * seq, 8, generator=g).to(cuda) for _ in range(3))
    with_aux = model(input_ids=ids, labels=labels, output_router_logits=True)
    assert with_aux.aux_loss is not None
    torch.testing.assert_close(with_aux.loss.detach(), out.loss.detach() + 0.01 * with_aux.aux_loss, rtol=1e-3, atol=1e-4)
    # inference: logits of the kept positions from the packed head
    logits = model(input_ids=ids, logits_to_keep=1).logits
    assert logits.shape == (batch, 1, vocab) and model(input_ids=ids).loss is None


def test_qwen_model_forward_patch_takes_the_packed_loss(cuda):
    """apply_gguf_liger_fused_linear_cross_entropy on a Qwen3.5-MoE model instance (gguf_liger_loss.py:359-532): in training with
    labels the logits are skipped and the loss is the packed Q6_K head's; logits together with labels in training are refused; in
    evaluation the head runs as usual."""
    import gguf_liger_loss as gl
    from types import SimpleNamespace
    from b2g.gguf_types import GGUFLinear, GGUFQuantizedTensor

    model_cls, _, _ = gl._model_types()
    vocab, hidden, batch, seq = 1032, 2048, 2, 24
    payload, w = _head(vocab, hidden, go.Q6_K, 515)

    class Tiny(model_cls):
        def __init__(self):
            torch.nn.Module.__init__(self)                     # none of the real model is built
            self.lm_head = GGUFLinear(hidden, vocab)
            self.lm_head.weight = GGUFQuantizedTensor(torch.from_numpy(payload).to(cuda), quant_type=go.Q6_K, logical_shape=(vocab, hidden))
            self.cfg = SimpleNamespace(hidden_size=hidden, output_attentions=False, output_router_logits=False, output_hidden_states=False,
                                       use_return_dict=True)
            self.embed = torch.nn.Embedding(vocab, hidden, device=cuda, dtype=torch.bfloat16)
            self.vocab_size = vocab

        config = property(lambda self: self.cfg)

        def model(self, input_ids=None, **kwargs):
            return _fake_body(self.embed(input_ids))

    model = Tiny()
    assert gl.apply_gguf_liger_fused_linear_cross_entropy(model) is model
    g = torch.Generator().manual_seed(11)
    ids = torch.randint(0, vocab, (batch, seq), generator=g).to(cuda)
    model.train()
    out = model(input_ids=ids, labels=ids)
    assert out.logits is None
    h = model.embed(ids).detach().reshape(-1, hidden).cpu()
    shifted = torch.nn.functional.pad(ids, (0, 1), value=-100)[..., 1:].reshape(-1).cpu()
    ref = loss_ref.packed_linear_cross_entropy(h, w, shifted, -100, "mean")
    torch.testing.assert_close(out.loss.detach().cpu().float(), ref["loss"].float(), rtol=2e-3, atol=2e-3)
    out.loss.backward()
    assert model.embed.weight.grad is not None and torch.isfinite(model.embed.weight.grad.float()).all()
    with pytest.raises(RuntimeError, match="no-full-logits fused loss"):
        model(input_ids=ids, labels=ids, skip_logits=False)
    with pytest.raises(RuntimeError, match="logits_to_keep=0"):
        model(input_ids=ids, labels=ids, logits_to_keep=1)
    model.eval()
    assert model(input_ids=ids, logits_to_keep=2).logits.shape == (batch, 2, vocab)
