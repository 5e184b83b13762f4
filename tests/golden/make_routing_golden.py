#!/usr/bin/env python
"""Golden vectors for the token permute kernels, taken from the REFERENCE's own implementation.

The reference's ``fast_moe_routing.py`` (Triton kernels for gather, combine and their backwards, ``torch.sort`` for the
plan) imports without the rest of the reference and runs on an NVIDIA GPU.  This script runs that file UNMODIFIED:

    python tests/golden/make_routing_golden.py --stage /path/to/reference      # copies the one file to baseline/_ref/ (git-ignored)
    python tests/golden/make_routing_golden.py --out routing_golden.npz        # on a machine with a GPU and Triton

and stores, per case, what ``prepare_expert_routing`` / ``finalize_expert_routing`` and their backwards returned
(relations checked by ``test_fast_moe_routing.py:125-236``).  Inputs are drawn from numpy's PCG64 stream, so the test
regenerates them from the seed; the file keeps a digest of every input to prove that it did.  Large exact outputs
(selected rows, gradients) are kept as SHA-256 digests of their bytes, the outputs that are compared within a tolerance
(combined rows, routing-weight gradients) as values (the combined rows of every ``row_stride``-th token).
Nothing in the package imports this script or ``baseline/_ref``.
"""
from __future__ import annotations

import argparse
import hashlib
import importlib.util
import shutil
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
STAGED = ROOT / "baseline" / "_ref" / "fast_moe_routing.py"

# (name, tokens, top_k, hidden, weights dtype, seed); seeds follow the reference's tests (2468 gather, 97531 combine)
CASES = [
    ("qwen_257_f32", 257, 8, 2048, "float32", 2468),
    ("deepseek_257_f32", 257, 6, 4096, "float32", 97531),
    ("qwen_2048_bf16", 2048, 8, 2048, "bfloat16", 97531),
    ("deepseek_2048_f32", 2048, 6, 4096, "float32", 2468),
]
NUM_EXPERTS = 256
ROW_STRIDE = 16


def bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> bf16 bit patterns (uint16), round to nearest even."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def digest(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def make_inputs(tokens: int, top_k: int, hidden: int, seed: int) -> dict[str, np.ndarray]:
    """hidden / expert outputs / cotangents as bf16 bit patterns, distinct expert ids per token, normalised weights."""
    rng = np.random.default_rng(seed)
    routes = tokens * top_k
    ids = np.argsort(rng.random((tokens, NUM_EXPERTS)), axis=1)[:, :top_k].astype(np.int64)
    raw = rng.random((tokens, top_k), dtype=np.float32)
    return {
        "hidden": bf16_bits(rng.standard_normal((tokens, hidden), dtype=np.float32)),
        "top_k_index": ids,
        "weights": (raw / raw.sum(axis=1, keepdims=True)).astype(np.float32),
        "expert_out": bf16_bits(rng.standard_normal((routes, hidden), dtype=np.float32)),
        "grad_selected": bf16_bits(rng.standard_normal((routes, hidden), dtype=np.float32)),
        "grad_final": bf16_bits(rng.standard_normal((tokens, hidden), dtype=np.float32)),
    }


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--stage", metavar="REFERENCE_DIR", help="copy the reference's fast_moe_routing.py to baseline/_ref/ and exit")
    ap.add_argument("--out", default="routing_golden.npz")
    args = ap.parse_args()
    if args.stage:
        STAGED.parent.mkdir(parents=True, exist_ok=True)
        shutil.copyfile(Path(args.stage) / "fast_moe_routing.py", STAGED)
        print(f"staged {STAGED}")
        return 0

    import torch

    if not STAGED.exists():
        print(f"{STAGED} is missing: run with --stage first", file=sys.stderr)
        return 2
    spec = importlib.util.spec_from_file_location("reference_fast_moe_routing", STAGED)
    ref = importlib.util.module_from_spec(spec)
    sys.modules["reference_fast_moe_routing"] = ref
    spec.loader.exec_module(ref)
    dev = torch.device("cuda", 0)

    def to_bf16(bits):
        return torch.from_numpy(bits.view(np.int16)).to(dev).view(torch.bfloat16)

    def bits_of(t):
        return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)

    store: dict[str, np.ndarray] = {"source_sha256": np.array(digest(np.frombuffer(STAGED.read_bytes(), dtype=np.uint8)))}
    for name, tokens, top_k, hidden, wdtype, seed in CASES:
        inp = make_inputs(tokens, top_k, hidden, seed)
        hid = to_bf16(inp["hidden"]).requires_grad_(True)
        idx = torch.from_numpy(inp["top_k_index"]).to(dev)
        w = torch.from_numpy(inp["weights"]).to(dev).to(getattr(torch, wdtype)).requires_grad_(True)
        expert_out = to_bf16(inp["expert_out"]).requires_grad_(True)
        plan = ref.prepare_expert_routing(hid, idx, w)
        final = ref.finalize_expert_routing(expert_out, hid, plan, None)
        torch.autograd.backward((plan.selected_hidden_states, final), (to_bf16(inp["grad_selected"]), to_bf16(inp["grad_final"])))
        torch.cuda.synchronize()
        store[f"{name}/inputs_sha256"] = np.array(" ".join(digest(inp[k]) for k in sorted(inp)))
        store[f"{name}/expert_indices"] = plan.expert_indices.cpu().numpy()
        store[f"{name}/permutation"] = plan.permutation.cpu().numpy()
        store[f"{name}/inverse_permutation"] = plan.inverse_permutation.cpu().numpy()
        store[f"{name}/selected_sha256"] = np.array(digest(bits_of(plan.selected_hidden_states)))
        store[f"{name}/grad_hidden_sha256"] = np.array(digest(bits_of(hid.grad)))
        store[f"{name}/grad_expert_out_sha256"] = np.array(digest(bits_of(expert_out.grad)))
        store[f"{name}/final_rows"] = bits_of(final)[::ROW_STRIDE]
        store[f"{name}/grad_weights"] = w.grad.float().cpu().numpy()
        print(name, "ok", flush=True)
    np.savez_compressed(args.out, **store)
    print(f"wrote {args.out}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
