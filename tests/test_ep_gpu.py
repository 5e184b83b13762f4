"""GPU: the expert-parallel layer on the libb2g kernels.  With one GPU the process group has a single
rank (the exchange degenerates to a local copy through NCCL); the result must equal the plain
single-device expert layer bit for bit."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist

from oracle import gguf_oracle as go

pytestmark = pytest.mark.gpu


def test_single_rank_expert_parallel_equals_local_layer(cuda):
    from b2g import autograd as ag, ep, routing

    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29577")
    if not dist.is_initialized():
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=cuda)
    try:
        e, h, i, t, k, r = 16, 512, 256, 300, 4, 16
        g = torch.Generator().manual_seed(3)
        rng = np.random.default_rng(3)
        pk = [torch.from_numpy(go.quantize((rng.standard_normal(s) * 0.02).astype(np.float32), go.Q4_K)).to(cuda).reshape(-1)
              for s in ((e, i, h), (e, i, h), (e, h, i))]
        lora = {"gate_up_a": (torch.randn(e, r, h, generator=g) / 16).bfloat16().to(cuda), "gate_up_b": (torch.randn(e, 2 * i, r, generator=g) * 0.01).bfloat16().to(cuda),
                "down_a": (torch.randn(e, r, i, generator=g) / 16).bfloat16().to(cuda), "down_b": (torch.randn(e, h, r, generator=g) * 0.01).bfloat16().to(cuda)}
        hidden = torch.randn(t, h, generator=g).bfloat16().to(cuda)
        logits = torch.randn(t, e, generator=g)
        idx = logits.topk(k, 1).indices.to(cuda)
        wts = torch.softmax(logits.gather(1, idx.cpu()), -1).to(cuda)
        gout = torch.randn(t, h, generator=g).bfloat16().to(cuda)

        h1 = hidden.clone().requires_grad_(True)
        l1 = {n: v.clone().requires_grad_(True) for n, v in lora.items()}
        out1 = ep.cuda_moe_layer(h1, idx, wts, *pk, go.Q4_K, i, e, l1, 2.0, always_exchange=True)   # through NCCL and the regroup
        out1.backward(gout)

        h2 = hidden.clone().requires_grad_(True)
        l2 = {n: v.clone().requires_grad_(True) for n, v in lora.items()}
        plan = routing.build_plan(h2, idx, wts, e)
        ex = ag.grouped_lora_experts(plan.selected_hidden_states, *pk, go.Q4_K, go.Q4_K, i, torch.arange(e, device=cuda), plan.group_offsets,
                                     plan.group_offsets, l2["gate_up_a"], l2["gate_up_b"], l2["down_a"], l2["down_b"], 2.0, 0.0)
        out2 = routing.combine(ex, plan)
        out2.backward(gout)
        assert torch.equal(out1, out2) and torch.equal(h1.grad, h2.grad)
        for n in lora:
            assert torch.equal(l1[n].grad, l2[n].grad), n

        # the peer-store exchange (symmetric memory; with one rank every peer pointer is the rank's own buffer)
        from b2g import ep_peer

        xchg = ep_peer.PeerExchange(t * k, h, e, device=cuda)
        for _ in range(2):                                   # twice: the second call reuses the buffers
            h3 = hidden.clone().requires_grad_(True)
            l3 = {n: v.clone().requires_grad_(True) for n, v in lora.items()}
            w3 = wts.clone().requires_grad_(True)
            out3 = ep_peer.peer_moe_layer(xchg, h3, idx, w3, *pk, go.Q4_K, i, l3, 2.0)
            out3.backward(gout)
            assert torch.equal(out3, out2) and torch.equal(h3.grad, h2.grad)
            for n in lora:
                assert torch.equal(l3[n].grad, l2[n].grad), n
        w2 = wts.clone().requires_grad_(True)
        plan = routing.build_plan(hidden, idx, w2, e)
        routing.combine(ex.detach(), plan).backward(gout)
        assert torch.equal(w3.grad, w2.grad)

        # the experts in three groups on two streams (one group's exchange beside another group's products): the same kernels
        # on the same rows in the same order, so every result is the same bits
        xchg3 = ep_peer.PeerExchange(t * k, h, e, device=cuda, chunks=3)
        assert xchg3.groups == [(0, 6), (6, 11), (11, 16)]
        xchg3.profile = True
        for _ in range(2):
            h4 = hidden.clone().requires_grad_(True)
            l4 = {n: v.clone().requires_grad_(True) for n, v in lora.items()}
            out4 = ep_peer.peer_moe_layer(xchg3, h4, idx, wts, *pk, go.Q4_K, i, l4, 2.0)
            out4.backward(gout)
            assert torch.equal(out4, out2) and torch.equal(h4.grad, h2.grad)
            for n in lora:
                assert torch.equal(l4[n].grad, l2[n].grad), n

        # experts placed by load: the router's ids go through the placement table, each rank holds the experts it was given.
        # Outputs stay the same bits (the combine adds a token's routes in router order); the token gradient adds them in
        # sorted-position order with a bf16 rounding per add, and the placement changes that order, so it agrees to rounding
        load = torch.bincount(idx.flatten().cpu(), minlength=e).float()
        placement = ep_peer.balanced_placement(load, 1)
        order = ep_peer.experts_of_rank(placement, 0, 1).to(cuda)
        pk_placed = [p.reshape(e, -1).index_select(0, order).reshape(-1) for p in pk]
        lora_placed = {n: v.index_select(0, order) for n, v in lora.items()}
        xchg4 = ep_peer.PeerExchange(t * k, h, e, device=cuda, chunks=2, placement=placement)
        h7 = hidden.clone().requires_grad_(True)
        l7 = {n: v.clone().requires_grad_(True) for n, v in lora_placed.items()}
        out7 = ep_peer.peer_moe_layer(xchg4, h7, idx, wts, *pk_placed, go.Q4_K, i, l7, 2.0)
        out7.backward(gout)
        assert torch.equal(out7, out2)
        assert float((h7.grad.float() - h2.grad.float()).norm() / h2.grad.float().norm()) < 5e-3
        for n in lora:
            want = l2[n].grad.index_select(0, order).float()
            assert float((l7[n].grad.float() - want).norm() / want.norm()) < 1e-2, n
        phases = xchg3.phase_ms()
        assert {"dispatch", "experts_forward", "return", "combine", "experts_backward", "gather_backward"} <= set(phases)

        # a receive buffer smaller than the routed rows: rows beyond it are dropped, everything downstream is clamped to it,
        # the status word says so, and the next ordinary call is untouched by it
        from b2g import ops

        ops.check_status()
        small = ep_peer.PeerExchange(t * k, h, e, device=cuda, capacity_factor=0.5)
        assert small.capacity < t * k
        h5 = hidden.clone().requires_grad_(True)
        out5 = ep_peer.peer_moe_layer(small, h5, idx, wts, *pk, go.Q4_K, i, {n: v.clone().requires_grad_(True) for n, v in lora.items()}, 2.0)
        out5.backward(gout)
        torch.cuda.synchronize()
        assert int(small.plan.local_offsets[-1]) == small.capacity and int(small.plan.blk_start[-1]) == small.capacity
        assert int(small.plan.local_sizes.sum()) == small.capacity
        with pytest.raises(Exception, match="901"):
            ops.check_status()
        h6 = hidden.clone().requires_grad_(True)
        out6 = ep_peer.peer_moe_layer(xchg, h6, idx, wts, *pk, go.Q4_K, i, {n: v.clone().requires_grad_(True) for n, v in lora.items()}, 2.0)
        out6.backward(gout)
        assert torch.equal(out6, out2) and torch.equal(h6.grad, h2.grad)
        ops.check_status()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,experts", [(1, 16), (2, 256), (4, 64), (8, 256), (8, 8)])
def test_peer_plan_kernel_equals_the_host_side_slot_arithmetic(cuda, world, experts):
    """One launch of b2g_ep_peer_plan gives, for every rank, exactly the slots that the tensor-op formulation
    (checked on the CPU against a simulated four-rank exchange) computes; empty experts and empty ranks included."""
    from b2g import ep_peer

    rng = np.random.default_rng(100 * world + experts)
    counts = rng.integers(0, 400, size=(world, experts)).astype(np.int32)
    counts[:, rng.integers(0, experts)] = 0          # an expert nobody routes to
    counts[rng.integers(0, world)] = 0               # a rank without tokens
    counts_dev = torch.from_numpy(counts).to(cuda)
    from b2g import ops

    for rank in range(world):
        for capacity in (None, int(counts[:, rank * (experts // world):(rank + 1) * (experts // world)].sum()) // 2):
            want = ep_peer.build_peer_plan(counts_dev, rank, capacity)
            got = ep_peer.build_peer_plan_device(counts_dev, rank, capacity)
            for name in ("my_start", "dest_base", "blk_start", "src_pos", "local_sizes", "local_offsets"):
                a, b = getattr(want, name), getattr(got, name)
                assert a.dtype == b.dtype == torch.int32 and a.shape == b.shape, name
                assert torch.equal(a, b), (name, rank, capacity)
            overflowed = capacity is not None and int(want.local_offsets[-1]) == capacity and capacity > 0
            torch.cuda.synchronize()
            code = int(ops.status_word(cuda).item())
            ops.status_word(cuda).zero_()
            assert code == (901 if overflowed else 0), (rank, capacity, code)
