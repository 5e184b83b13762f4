"""GGUF file loader: files written with gguf-py's own writer come back byte for byte, with the right type ids and
logical shapes; on the GPU the loaded payload multiplies like the oracle's decode of the same bytes."""
import numpy as np
import pytest
import torch

from oracle import dense_ref, gguf_oracle as go

gguf = pytest.importorskip("gguf")


def _write(path, tensors):
    w = gguf.GGUFWriter(str(path), "llama")
    for name, (arr, qt, shape) in tensors.items():
        if qt is None:
            w.add_tensor(name, arr)
        else:
            w.add_tensor(name, arr, raw_shape=arr.shape, raw_dtype=gguf.GGMLQuantizationType(qt))
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()


@pytest.fixture(scope="module")
def small_file(tmp_path_factory):
    rng = np.random.default_rng(5)
    dense = go.quantize((rng.standard_normal((24, 2048)) * 0.05).astype(np.float32), go.Q6_K)
    bank = go.quantize((rng.standard_normal((3, 16, 512)) * 0.05).astype(np.float32), go.Q4_K)
    q8 = go.quantize((rng.standard_normal((40, 256)) * 0.05).astype(np.float32), go.Q8_0)
    other = np.zeros((4, 144), dtype=np.uint8)                                   # Q4_0: not native
    norm = rng.standard_normal(64).astype(np.float32)
    path = tmp_path_factory.mktemp("gguf") / "tiny.gguf"
    _write(path, {"output.weight": (dense, go.Q6_K, (24, 2048)), "blk.0.ffn_gate_exps.weight": (bank, go.Q4_K, (3, 16, 512)),
                  "blk.0.attn_q.weight": (q8, go.Q8_0, (40, 256)), "blk.0.odd.weight": (other, 2, (4, 256)),
                  "blk.0.attn_norm.weight": (norm, None, (64,))})
    return path, {"dense": dense, "bank": bank, "q8": q8, "norm": norm}


def test_round_trip_bytes_types_and_shapes(small_file):
    from b2g import gguf_file

    path, src = small_file
    assert set(gguf_file.tensor_names(path)) == {"output.weight", "blk.0.ffn_gate_exps.weight", "blk.0.attn_q.weight", "blk.0.odd.weight",
                                                 "blk.0.attn_norm.weight"}
    head = gguf_file.load_tensor(path, "output.weight", "cpu")
    assert head.quant_type == go.Q6_K and head.logical_shape == (24, 2048) and head.dtype == torch.uint8
    assert np.array_equal(head.as_subclass(torch.Tensor).numpy(), src["dense"])
    bank = gguf_file.load_tensor(path, "blk.0.ffn_gate_exps.weight", "cpu")
    assert bank.quant_type == go.Q4_K and bank.logical_shape == (3, 16, 512) and tuple(bank.shape) == (3, 16, 288)
    assert np.array_equal(bank.as_subclass(torch.Tensor).numpy(), src["bank"])
    cut = gguf_file.load_tensor(path, "blk.0.ffn_gate_exps.weight", "cpu", leading=2, rows=8)
    assert cut.logical_shape == (2, 8, 512) and np.array_equal(cut.as_subclass(torch.Tensor).numpy(), src["bank"][:2, :8])
    norm = gguf_file.load_tensor(path, "blk.0.attn_norm.weight", "cpu")
    assert norm.dtype == torch.float32 and np.array_equal(norm.numpy(), src["norm"])
    with pytest.raises(ValueError, match="cannot multiply natively"):
        gguf_file.load_tensor(path, "blk.0.odd.weight", "cpu")
    with pytest.raises(KeyError):
        gguf_file.load_tensor(path, "missing", "cpu")
    assert gguf_file.type_census(path) == {go.Q6_K: 1, go.Q4_K: 1, go.Q8_0: 1, 2: 1, 0: 1}
    names = [n for n, _ in gguf_file.iter_tensors(path, "cpu", skip_unsupported=True)]
    assert "blk.0.odd.weight" not in names and len(names) == 4


@pytest.mark.gpu
def test_loaded_payload_multiplies_like_the_oracle(cuda, small_file):
    from b2g import autograd as ag, gguf_file

    path, src = small_file
    head = gguf_file.load_tensor(path, "output.weight", cuda)
    x = torch.randn(50, 2048, generator=torch.Generator().manual_seed(1)).bfloat16()
    y = ag.mmq(x.to(cuda), head.as_subclass(torch.Tensor), head.quant_type, 24)
    w = dense_ref.dequant_bf16(src["dense"], go.Q6_K)
    assert dense_ref.rel_l2(y, x.float() @ w.float().t()) < 1e-2
