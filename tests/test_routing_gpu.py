"""GPU: router top-k, routing plan and permute kernels against the CPU oracle.
Index work is compared bit-exactly; floating point within the tolerance written at each check."""
import pytest
import torch

from oracle import dense_ref, moe_ref

pytestmark = pytest.mark.gpu


def _sorted_equal_up_to_threshold_ties(scores, got, want, k):
    """Identity-free comparison (test_fast_moe_ranking.py:113-121): selections may differ only among
    experts whose score equals the k-th threshold."""
    gs, ws = got.sort(1).values, want.sort(1).values
    rows = (gs != ws).any(1).nonzero().flatten()
    for r in rows.tolist():
        thr = scores[r, want[r]].min()
        diff = set(got[r].tolist()) ^ set(want[r].tolist())
        assert all(scores[r, e] == thr for e in diff)
    return True


@pytest.mark.parametrize("tokens,top_k,dtype", [(257, 8, torch.bfloat16), (2048, 8, torch.float32), (1, 6, torch.float32), (4100, 6, torch.bfloat16)])
def test_router_topk_identity(cuda, tokens, top_k, dtype):
    from b2g import ops

    logits = torch.randn(tokens, 256, generator=torch.Generator().manual_seed(tokens)).to(dtype)
    got = ops.router_topk(logits.to(cuda), top_k, None, False).cpu()
    want = moe_ref.router_topk(logits, top_k)
    assert got.dtype == torch.int64 and torch.equal(got, want)       # order included: best first, ties to the smaller id


def test_router_topk_all_ties_pick_smallest_ids(cuda):
    from b2g import ops

    got = ops.router_topk(torch.zeros(5, 256, device=cuda), 8, None, False).cpu()
    assert got.tolist() == [list(range(8))] * 5
    lg = torch.zeros(3, 256)
    lg[:, 200] = 1.0
    lg[:, 17] = -0.0                                                   # -0.0 orders below +0.0 in the key
    got = ops.router_topk(lg.to(cuda), 6, None, False).cpu()
    assert got[:, 0].tolist() == [200] * 3 and got[:, 1:].tolist() == [[0, 1, 2, 3, 4]] * 3


def test_router_topk_sqrt_softplus_with_bias(cuda):
    from b2g import ops

    g = torch.Generator().manual_seed(8642)
    logits = torch.randn(3000, 256, generator=g)
    bias = torch.randn(256, generator=g) * 0.1
    got = ops.router_topk(logits.to(cuda), 6, bias.to(cuda), True).cpu()
    want = moe_ref.router_topk(logits, 6, bias, "sqrtsoftplus")
    scores = moe_ref.router_scores(logits, bias, "sqrtsoftplus")
    same = (got.sort(1).values == want.sort(1).values).all(1)
    assert same.float().mean() > 0.999                                 # libm vs device exp/log differ in the last ulp
    for r in (~same).nonzero().flatten().tolist():                     # and only across near-equal scores
        a, b = set(got[r].tolist()), set(want[r].tolist())
        for e in a ^ b:
            assert abs(float(scores[r, e]) - float(scores[r, want[r]].min())) < 1e-5


def test_router_geometry_is_fail_closed(cuda):
    from b2g import ops

    with pytest.raises(ValueError, match="256 experts"):
        ops.router_topk(torch.zeros(4, 128, device=cuda), 4, None, False)
    with pytest.raises(ValueError, match="bias"):
        ops.router_topk(torch.zeros(4, 256, device=cuda), 6, torch.zeros(256, device=cuda), False)


@pytest.mark.parametrize("tokens,top_k,idx_dtype", [(2048, 8, torch.int64), (257, 6, torch.int32), (1, 1, torch.int64), (5000, 4, torch.int64)])
def test_route_plan_is_the_stable_sort(cuda, tokens, top_k, idx_dtype):
    from b2g import ops

    idx = torch.randint(0, 256, (tokens, top_k), generator=torch.Generator().manual_seed(19260817)).to(idx_dtype)
    want = moe_ref.route_plan(idx)
    se, perm, inv, sizes, offs = (t.cpu() for t in ops.route_plan(idx.to(cuda)))
    assert torch.equal(se, want["expert_indices"]) and torch.equal(perm, want["permutation"])
    assert torch.equal(inv, want["inverse_permutation"])
    assert torch.equal(sizes, want["group_sizes"]) and torch.equal(offs, want["offsets"])


def test_route_plan_skewed_and_empty_experts(cuda):
    from b2g import ops

    idx = torch.zeros(3000, 8, dtype=torch.int64)
    idx[:, 1:] = torch.randint(250, 256, (3000, 7), generator=torch.Generator().manual_seed(1))
    want = moe_ref.route_plan(idx)
    se, perm, inv, sizes, offs = (t.cpu() for t in ops.route_plan(idx.to(cuda)))
    assert torch.equal(perm, want["permutation"]) and torch.equal(sizes, want["group_sizes"])
    assert int(sizes[1:250].sum()) == 0 and int(sizes[0]) == 3000


@pytest.mark.parametrize("top_k,hidden", [(8, 2048), (6, 4096), (4, 2048), (1, 256)])
def test_gather_and_its_backward_are_exact(cuda, top_k, hidden):
    from b2g import routing

    tokens = 300
    g = torch.Generator().manual_seed(2468)
    idx = torch.randint(0, 256, (tokens, top_k), generator=g)
    h = torch.randn(tokens, hidden, generator=g).bfloat16()
    w = torch.rand(tokens, top_k, generator=g)
    hc = h.to(cuda).requires_grad_(True)
    plan = routing.build_plan(hc, idx.to(cuda), w.to(cuda))
    ref = moe_ref.route_plan(idx)
    assert torch.equal(plan.selected_hidden_states.cpu(), moe_ref.route_gather(h, ref["permutation"], top_k))
    gs = torch.randn(tokens * top_k, hidden, generator=g).bfloat16()
    plan.selected_hidden_states.backward(gs.to(cuda))
    assert torch.equal(hc.grad.cpu(), moe_ref.route_gather_bwd(gs, ref["inverse_permutation"], tokens, top_k))


@pytest.mark.parametrize("w_dtype", [torch.bfloat16, torch.float32])
def test_combine_forward_backward(cuda, w_dtype):
    from b2g import ops

    tokens, top_k, hidden = 300, 8, 2048
    g = torch.Generator().manual_seed(97531)
    idx = torch.randint(0, 256, (tokens, top_k), generator=g)
    ref = moe_ref.route_plan(idx)
    out = torch.randn(tokens * top_k, hidden, generator=g).bfloat16()
    w = torch.rand(tokens, top_k, generator=g)
    w = (w / w.sum(1, keepdim=True)).to(w_dtype)
    perm, inv = ref["permutation"].to(cuda), ref["inverse_permutation"].to(cuda)
    got = ops.route_combine(out.to(cuda), w.to(cuda), inv).cpu()
    want = moe_ref.route_combine(out, w, ref["inverse_permutation"])
    # fp32 accumulation with one final rounding; the reference allows one bf16 step (atol 2^-6,
    # test_fast_moe_routing.py:214)
    torch.testing.assert_close(got, want, rtol=0, atol=0.015625)
    gf = torch.randn(tokens, hidden, generator=g).bfloat16()
    d_out, d_w = ops.route_combine_bwd(out.to(cuda), w.to(cuda), perm, gf.to(cuda))
    r_out, r_w = moe_ref.route_combine_bwd(out, w, ref["permutation"], gf)
    assert torch.equal(d_out.cpu(), r_out)                              # one product, one rounding: exact
    assert d_w.dtype == w_dtype
    assert dense_ref.rel_l2(d_w, r_w) < (5e-3 if w_dtype == torch.bfloat16 else 1e-5)


def test_swiglu_forward_backward(cuda):
    from b2g import ops

    g = torch.Generator().manual_seed(4)
    gate = (torch.randn(999, 512, generator=g) * 3).bfloat16()
    up = (torch.randn(999, 512, generator=g) * 3).bfloat16()
    dz = torch.randn(999, 512, generator=g).bfloat16()
    for limit in (0.0, 2.0):
        gr, ur = gate.clone().requires_grad_(True), up.clone().requires_grad_(True)
        zr = moe_ref.swiglu(gr, ur, limit if limit > 0 else None)
        zr.backward(dz)
        z = ops.swiglu_fwd(gate.to(cuda), up.to(cuda), limit)
        dg, du = ops.swiglu_bwd(gate.to(cuda), up.to(cuda), dz.to(cuda), limit)
        assert dense_ref.rel_l2(z, zr) < 2e-3 and dense_ref.rel_l2(du, ur.grad) < 4e-3 and dense_ref.rel_l2(dg, gr.grad) < 1e-2
        # the pair-at-a-time form (a width that is no multiple of eight values) gives the same bits as the 16-byte form
        narrow = slice(0, 6)
        zn = ops.swiglu_fwd(gate[:, narrow].contiguous().to(cuda), up[:, narrow].contiguous().to(cuda), limit)
        dgn, dun = ops.swiglu_bwd(gate[:, narrow].contiguous().to(cuda), up[:, narrow].contiguous().to(cuda),
                                  dz[:, narrow].contiguous().to(cuda), limit)
        assert torch.equal(zn, z[:, narrow]) and torch.equal(dgn, dg[:, narrow]) and torch.equal(dun, du[:, narrow])


def test_an_expert_id_outside_the_expert_count_is_reported_and_contained(cuda):
    """One route names expert E (one past the last).  The plan does not count or place it, the status word reports it (903),
    every index the plan returns stays inside its tensor (the skipped slots keep the zeros they were created with), and the
    permutes that follow the plan run without touching memory outside their tensors."""
    from b2g import ops, routing

    e, t, k, h = 256, 64, 8, 2048
    g = torch.Generator().manual_seed(12)
    idx = torch.stack([torch.randperm(e, generator=g)[:k] for _ in range(t)]).to(cuda)
    idx[5, 3] = e
    hidden = torch.randn(t, h, generator=g).bfloat16().to(cuda)
    wts = torch.rand(t, k, generator=g).to(cuda)
    ops.check_status()
    plan = routing.build_plan(hidden, idx, wts, e)
    out = routing.combine(plan.selected_hidden_states, plan)
    torch.cuda.synchronize()
    assert int(plan.group_sizes.sum()) == t * k - 1
    for index in (plan.permutation, plan.inverse_permutation):
        assert int(index.min()) >= 0 and int(index.max()) < t * k
    assert int(plan.expert_indices.max()) < e and torch.isfinite(out.float()).all()
    with pytest.raises(Exception, match="903"):
        ops.check_status()
    ops.check_status()
    good = routing.build_plan(hidden, idx.clamp(max=e - 1), wts, e)          # the next plan is unaffected
    torch.cuda.synchronize()
    assert int(good.group_sizes.sum()) == t * k
    ops.check_status()
