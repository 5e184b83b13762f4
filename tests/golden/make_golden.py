"""Generate tests/golden/gguf_dequant.npz: packed payloads and their float32 decode by gguf-py.

Run in the build container (needs the `gguf` package, which is the normative restatement of the
GGUF block formats the reference's dequantiser implements):

    python tests/golden/make_golden.py

Payload sources: gguf-py's own Q8_0 encoder; this repository's oracle encoders for Q2_K, Q3_K, Q4_K, Q5_K, Q6_K and
IQ2_XXS (gguf-py has none); uniformly random valid blocks; and the constant-byte payload of the
reference's own grouped test (test_deepseek_v4_moe_lora.py:55-64: every byte = 32).  The answers
always come from gguf.quants.dequantize, never from this repository's code.
"""
import sys
from pathlib import Path

import gguf
import numpy as np
from gguf import quants as gq

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import gguf_oracle as go  # noqa: E402


def main() -> None:
    rng = np.random.default_rng(19260817)
    out = {}
    w = (rng.standard_normal((12, 512)) * 0.02).astype(np.float32)
    w[3] = 0.0                                     # an all-zero row: zero scales
    w[5, :256] *= 50.0                             # a block with a large dynamic range
    cases = {
        "q8_0_gguf_encoder": (go.Q8_0, gq.quantize(w, gguf.GGMLQuantizationType.Q8_0)),
        "q4_k_oracle_encoder": (go.Q4_K, go.quantize(w, go.Q4_K)),
        "iq2_xxs_oracle_encoder": (go.IQ2_XXS, go.quantize(w, go.IQ2_XXS)),
        "q8_0_random": (go.Q8_0, go.random_payload(go.Q8_0, (6, 512), 1)),
        "q4_k_random": (go.Q4_K, go.random_payload(go.Q4_K, (6, 512), 2)),
        "iq2_xxs_random": (go.IQ2_XXS, go.random_payload(go.IQ2_XXS, (6, 512), 3)),
        "iq2_xxs_const32": (go.IQ2_XXS, np.full((4, 66), 32, dtype=np.uint8)),
        "q4_k_const32": (go.Q4_K, np.full((4, 144), 32, dtype=np.uint8)),
        "q2_k_oracle_encoder": (go.Q2_K, go.quantize(w, go.Q2_K)),
        "q2_k_random": (go.Q2_K, go.random_payload(go.Q2_K, (6, 512), 6)),
        "q2_k_const32": (go.Q2_K, np.full((4, 84), 32, dtype=np.uint8)),
        "q3_k_oracle_encoder": (go.Q3_K, go.quantize(w, go.Q3_K)),
        "q3_k_random": (go.Q3_K, go.random_payload(go.Q3_K, (6, 512), 7)),
        "q3_k_const32": (go.Q3_K, np.full((4, 110), 32, dtype=np.uint8)),
        "iq2_s_oracle_encoder": (go.IQ2_S, go.quantize(w, go.IQ2_S)),
        "iq2_s_random": (go.IQ2_S, go.random_payload(go.IQ2_S, (6, 512), 8)),
        "iq2_s_const32": (go.IQ2_S, np.full((4, 82), 32, dtype=np.uint8)),
        "q5_k_oracle_encoder": (go.Q5_K, go.quantize(w, go.Q5_K)),
        "q5_k_random": (go.Q5_K, go.random_payload(go.Q5_K, (6, 512), 5)),
        "q5_k_const32": (go.Q5_K, np.full((4, 176), 32, dtype=np.uint8)),
        "q6_k_oracle_encoder": (go.Q6_K, go.quantize(w, go.Q6_K)),
        "q6_k_random": (go.Q6_K, go.random_payload(go.Q6_K, (6, 512), 4)),
        "q6_k_const32": (go.Q6_K, np.full((4, 210), 32, dtype=np.uint8)),
    }
    for name, (qt, payload) in cases.items():
        ref = gq.dequantize(payload, gguf.GGMLQuantizationType(qt)).astype(np.float32)
        out[name + "__payload"] = payload
        out[name + "__f32bits"] = ref.view(np.uint32)
        out[name + "__qtype"] = np.int32(qt)
    gq.IQ2_XXS.init_grid()
    out["iq2_xxs_ksigns"] = np.frombuffer(gq.IQ2_XXS.ksigns, dtype=np.uint8).copy()
    np.savez_compressed(Path(__file__).with_name("gguf_dequant.npz"), **out)
    print("wrote", len(cases), "cases")


if __name__ == "__main__":
    main()
