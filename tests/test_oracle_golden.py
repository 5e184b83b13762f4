"""CPU: pin the oracle's GGUF decoders against gguf-py outputs (committed vectors and, when the
package is importable, live)."""
from pathlib import Path

import numpy as np
import pytest

from oracle import gguf_oracle as go

GOLDEN = np.load(Path(__file__).parent / "golden" / "gguf_dequant.npz")
CASES = sorted({k.split("__")[0] for k in GOLDEN.files if "__" in k})


@pytest.mark.parametrize("case", CASES)
def test_oracle_decode_matches_golden_bits(case):
    payload = GOLDEN[case + "__payload"]
    qtype = int(GOLDEN[case + "__qtype"])
    got = go.dequantize(payload, qtype)
    assert got.dtype == np.float32
    assert np.array_equal(got.view(np.uint32), GOLDEN[case + "__f32bits"])


def test_sign_table_matches_golden():
    assert np.array_equal(go.iq2xxs_signs_u8(), GOLDEN["iq2_xxs_ksigns"])


@pytest.mark.parametrize("qtype", [go.Q8_0, go.Q4_K, go.IQ2_XXS, go.Q6_K, go.Q5_K, go.Q2_K, go.Q3_K, go.IQ2_S])
def test_oracle_matches_gguf_py_live(qtype):
    gguf = pytest.importorskip("gguf")
    from gguf import quants as gq

    rng = np.random.default_rng(7 + qtype)
    w = (rng.standard_normal((16, 1024)) * 0.02).astype(np.float32)
    for payload in (go.quantize(w, qtype), go.random_payload(qtype, (8, 1024), 11)):
        ref = gq.dequantize(payload, gguf.GGMLQuantizationType(qtype))
        assert np.array_equal(go.dequantize(payload, qtype).view(np.uint32), ref.astype(np.float32).view(np.uint32))


def test_q8_encoder_is_gguf_py_encoder():
    gguf = pytest.importorskip("gguf")
    from gguf import quants as gq

    w = (np.random.default_rng(3).standard_normal((8, 2048)) * 0.02).astype(np.float32)
    assert np.array_equal(go.quantize(w, go.Q8_0), gq.quantize(w, gguf.GGMLQuantizationType.Q8_0))


@pytest.mark.parametrize("qtype,tol", [(go.Q8_0, 0.01), (go.Q4_K, 0.12), (go.IQ2_XXS, 0.5), (go.Q6_K, 0.03), (go.Q5_K, 0.06), (go.Q2_K, 0.45), (go.Q3_K, 0.25), (go.IQ2_S, 0.45)])
def test_encoders_round_trip(qtype, tol):
    w = (np.random.default_rng(5).standard_normal((8, 2048)) * 0.02).astype(np.float32)
    p = go.quantize(w, qtype)
    assert p.shape == (8, go.row_bytes(qtype, 2048)) and p.dtype == np.uint8
    back = go.dequantize(p, qtype)
    assert np.linalg.norm(back - w) / np.linalg.norm(w) < tol
    # encode(decode(p)) decodes to the same values for the lossless-at-grid formats
    if qtype == go.Q8_0:
        assert np.array_equal(go.dequantize(go.quantize(back, qtype), qtype), back)


def test_bf16_rounding_is_nearest_even():
    import torch

    x = np.random.default_rng(1).standard_normal(4096).astype(np.float32)
    x[:4] = [1.00390625, 1.01171875, -1.00390625, 0.0]   # exact ties between bf16 neighbours
    ref = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(go.bf16_bits(x), ref)


def test_empty_and_ragged_inputs():
    assert go.dequantize(np.zeros((0, 144), np.uint8), go.Q4_K).shape == (0, 256)
    with pytest.raises(ValueError):
        go.dequantize(np.zeros((2, 143), np.uint8), go.Q4_K)
    with pytest.raises(ValueError):
        go.row_bytes(go.Q4_K, 300)
