"""GPU: the permute kernels against outputs of the REFERENCE's own ``fast_moe_routing.py`` (its Triton kernels, run unmodified on
a B200 by ``tests/golden/make_routing_golden.py``; the vectors are committed as ``tests/golden/routing_golden.npz``).
Plan indices, gathered rows, the gather backward and the combine backward's row gradients are compared bit for bit; the
combined rows within 2^-6 and the routing-weight gradients within the bounds of ``test_fast_moe_routing.py:125-236``."""
import hashlib
import importlib.util
from pathlib import Path

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).parent / "golden" / "routing_golden.npz"


def _generator():
    spec = importlib.util.spec_from_file_location("make_routing_golden", Path(__file__).parent / "golden" / "make_routing_golden.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _digest(t: torch.Tensor) -> str:
    return hashlib.sha256(t.detach().contiguous().view(torch.int16).cpu().numpy().tobytes()).hexdigest()


@pytest.mark.parametrize("case", range(4))
def test_permute_kernels_equal_the_reference_implementation(cuda, case):
    from b2g import routing

    gen = _generator()
    assert GOLDEN.exists(), "tests/golden/routing_golden.npz is missing (tests/golden/make_routing_golden.py writes it on a GPU box)"
    gold = np.load(GOLDEN)
    name, tokens, top_k, hidden, wdtype, seed = gen.CASES[case]
    inp = gen.make_inputs(tokens, top_k, hidden, seed)
    assert " ".join(gen.digest(inp[k]) for k in sorted(inp)) == str(gold[f"{name}/inputs_sha256"]), "regenerated inputs differ from the generator's"

    def to_bf16(bits):
        return torch.from_numpy(bits.view(np.int16)).to(cuda).view(torch.bfloat16)

    hid = to_bf16(inp["hidden"]).requires_grad_(True)
    idx = torch.from_numpy(inp["top_k_index"]).to(cuda)
    w = torch.from_numpy(inp["weights"]).to(cuda).to(getattr(torch, wdtype)).requires_grad_(True)
    expert_out = to_bf16(inp["expert_out"]).requires_grad_(True)
    plan = routing.build_plan(hid, idx, w, gen.NUM_EXPERTS)
    final = routing.combine(expert_out, plan)
    torch.autograd.backward((plan.selected_hidden_states, final), (to_bf16(inp["grad_selected"]), to_bf16(inp["grad_final"])))

    assert np.array_equal(plan.expert_indices.cpu().numpy(), gold[f"{name}/expert_indices"])
    assert np.array_equal(plan.permutation.cpu().numpy(), gold[f"{name}/permutation"])
    assert np.array_equal(plan.inverse_permutation.cpu().numpy(), gold[f"{name}/inverse_permutation"])
    assert _digest(plan.selected_hidden_states) == str(gold[f"{name}/selected_sha256"])
    assert _digest(hid.grad) == str(gold[f"{name}/grad_hidden_sha256"]), "gather backward is not bit-identical to the reference kernel"
    assert _digest(expert_out.grad) == str(gold[f"{name}/grad_expert_out_sha256"]), "combine backward rows are not bit-identical"
    want_final = torch.from_numpy(gold[f"{name}/final_rows"].view(np.int16)).view(torch.bfloat16).float()
    torch.testing.assert_close(final[::gen.ROW_STRIDE].detach().cpu().float(), want_final, rtol=0, atol=2 ** -6)
    want_dw = torch.from_numpy(gold[f"{name}/grad_weights"])
    got_dw = w.grad.float().cpu()
    assert float((got_dw - want_dw).norm() / want_dw.norm()) < (2e-2 if wdtype == "bfloat16" else 1e-4)
