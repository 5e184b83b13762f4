"""GPU: the CUDA dequantiser is bit-exact with the oracle (and so with gguf-py)."""
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import gguf_oracle as go

pytestmark = pytest.mark.gpu
GOLDEN = np.load(Path(__file__).parent / "golden" / "gguf_dequant.npz")
CASES = sorted({k.split("__")[0] for k in GOLDEN.files if "__" in k})


def _bits(t: torch.Tensor) -> np.ndarray:
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


@pytest.mark.parametrize("case", CASES)
def test_golden_vectors_bit_exact(cuda, case):
    from b2g import ops

    payload = GOLDEN[case + "__payload"]
    qtype = int(GOLDEN[case + "__qtype"])
    want = go.bf16_bits(GOLDEN[case + "__f32bits"].view(np.float32))
    rows = payload.shape[0]
    k = want.shape[1]
    got = ops.dequantize(torch.from_numpy(payload).to(cuda), qtype, (rows, k))
    assert np.array_equal(_bits(got), want)


@pytest.mark.parametrize("qtype", [go.Q8_0, go.Q4_K, go.IQ2_XXS, go.Q6_K, go.Q5_K, go.Q2_K, go.Q3_K, go.IQ2_S])
@pytest.mark.parametrize("shape", [(1, 256), (37, 2048), (3, 5, 1024)])
def test_encoded_and_random_payloads_bit_exact(cuda, qtype, shape):
    from b2g import ops

    rng = np.random.default_rng(qtype * 100 + shape[-1])
    w = (rng.standard_normal(shape) * 0.02).astype(np.float32)
    for payload in (go.quantize(w, qtype), go.random_payload(qtype, shape, 9)):
        got = ops.dequantize(torch.from_numpy(payload).to(cuda), qtype, shape)
        assert got.shape == shape and got.dtype == torch.bfloat16
        assert np.array_equal(_bits(got), go.dequantize_bf16_bits(payload, qtype))


def test_full_size_weight_checksum(cuda):
    """A config-sized weight (4096 x 2048 Q4_K): compare a 64-bit checksum of all output bits."""
    from b2g import ops

    payload = go.random_payload(go.Q4_K, (4096, 2048), 123)
    got = _bits(ops.dequantize(torch.from_numpy(payload).to(cuda), go.Q4_K, (4096, 2048)))
    want = go.dequantize_bf16_bits(payload, go.Q4_K)
    assert int(got.astype(np.uint64).sum()) == int(want.astype(np.uint64).sum())
    assert np.array_equal(got, want)


def test_empty_and_bad_arguments(cuda):
    from b2g import ops

    assert ops.dequantize(torch.empty(0, dtype=torch.uint8, device=cuda), go.Q4_K, (0, 256)).shape == (0, 256)
    with pytest.raises(ValueError):
        ops.dequantize(torch.zeros(100, dtype=torch.uint8, device=cuda), go.Q4_K, (1, 256))
    with pytest.raises(ValueError):
        ops.dequantize(torch.zeros(144, dtype=torch.uint8, device=cuda), 2, (1, 256))  # Q4_0: not native here
