"""One rank of the multi-GPU expert-parallel check (started by tests/test_ep_multi_gpu.py through torch.distributed.run).

Every rank holds its own tokens and its own experts.  The layer is evaluated three ways on the same inputs:
  1. peer stores over NVLink (b2g/ep_peer.py), twice, so that the second call reuses the symmetric buffers;
  2. NCCL all-to-all (b2g/ep.py);
  3. on one device: all ranks' tokens and all experts gathered onto this rank, plain single-GPU layer;
  4. peer stores again with every rank's experts in two groups (one group's exchange beside another group's products) and
     the experts placed over the ranks by load instead of in contiguous blocks.
1 and 2 run the same kernels on the same rows in the same order and must agree bit for bit.  Against 3 the outputs
and token gradients are compared exactly (a row's result does not depend on which rows share its tile) and the factor
gradients within rel-L2 1e-2 (their sums over rows run in a different order).  Under a placement the token gradient adds a
token's routes in another order (the permute backward rounds to bf16 after every add, in sorted-position order), so 4
is run twice: groups alone, exact; groups and placement, token gradients to rounding.
Prints one line "rank R: OK" or raises.
"""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT / "transformers5-qwen3.5-recipe_b200"))


def _gather(t: torch.Tensor) -> torch.Tensor:
    out = [torch.empty_like(t) for _ in range(dist.get_world_size())]
    dist.all_gather(out, t.contiguous())
    return torch.cat(out, 0)


def main() -> int:
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from b2g import autograd as ag, ep, ep_peer, gguf_quant, ops, routing

    q4k = 12
    e, h, i, k, r, t = 16, 512, 256, 4, 4, 384
    el = e // world
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    pk = [gguf_quant.random_payload(q4k, s, 10 * rank + j, device=dev) for j, s in enumerate(((el, i, h), (el, i, h), (el, h, i)))]
    lora = {"gate_up_a": (torch.randn(el, r, h, generator=g, device=dev) / 16).bfloat16(),
            "gate_up_b": (torch.randn(el, 2 * i, r, generator=g, device=dev) * 0.01).bfloat16(),
            "down_a": (torch.randn(el, r, i, generator=g, device=dev) / 16).bfloat16(),
            "down_b": (torch.randn(el, h, r, generator=g, device=dev) * 0.01).bfloat16()}
    hidden = torch.randn(t, h, generator=g, device=dev).bfloat16()
    gout = torch.randn(t, h, generator=g, device=dev).bfloat16()
    logits = torch.randn(t, e, generator=g, device=dev)
    logits[:, :3] += 1.5                                   # a skewed router: rank 0's experts are busier
    logits[:, e - 1] = -1e4                                # and one expert that nobody routes to
    idx = logits.topk(k, 1).indices                        # (the router kernel itself is fixed at 256 experts)
    wts = torch.softmax(logits.gather(1, idx), -1)

    def run(fn, hid, lo, go_):
        hh = hid.clone().requires_grad_(True)
        ll = {n: v.clone().requires_grad_(True) for n, v in lo.items()}
        out = fn(hh, ll)
        out.backward(go_)
        torch.cuda.synchronize()
        return [out.detach().clone(), hh.grad.clone()] + [ll[n].grad.clone() for n in lo]

    flat = [p.reshape(-1) for p in pk]
    via_nccl = run(lambda hh, ll: ep.cuda_moe_layer(hh, idx, wts, *flat, q4k, i, e, ll, 2.0), hidden, lora, gout)
    # receive buffers default to the worst case (every routed row of every rank lands here), so the skewed router above fits
    xchg = ep_peer.PeerExchange(t * k, h, e, device=dev)
    assert xchg.capacity >= world * t * k
    for _ in range(2):
        via_peer = run(lambda hh, ll: ep_peer.peer_moe_layer(xchg, hh, idx, wts, *flat, q4k, i, ll, 2.0), hidden, lora, gout)
        for a, b in zip(via_nccl, via_peer):
            assert torch.equal(a, b), "peer-store exchange and NCCL exchange differ"

    # the whole job on this one device
    all_hidden, all_gout, all_idx, all_wts = _gather(hidden), _gather(gout), _gather(idx), _gather(wts)
    all_pk = [_gather(p).reshape(-1) for p in pk]
    all_lora = {n: _gather(v) for n, v in lora.items()}

    def single(hh, ll):
        plan = routing.build_plan(hh, all_idx, all_wts, e)
        ex = ag.grouped_lora_experts(plan.selected_hidden_states, *all_pk, q4k, q4k, i, torch.arange(e, device=dev), plan.group_offsets,
                                     plan.group_offsets, ll["gate_up_a"], ll["gate_up_b"], ll["down_a"], ll["down_b"], 2.0, 0.0)
        return routing.combine(ex, plan)

    whole = run(single, all_hidden, all_lora, all_gout)
    rows = slice(rank * t, (rank + 1) * t)
    assert torch.equal(via_peer[0], whole[0][rows]), "outputs differ from the single-device layer"
    assert torch.equal(via_peer[1], whole[1][rows]), "token gradients differ from the single-device layer"
    mine = slice(rank * el, (rank + 1) * el)
    for got, want, name in zip(via_peer[2:], whole[2:], lora):
        want = want[mine].float()
        err = float((got.float() - want).norm() / want.norm().clamp_min(1e-20))
        assert err <= 1e-2, (name, err)

    # two chunks, load-aware placement: this rank now holds the experts the placement gives it
    load = torch.bincount(all_idx.flatten(), minlength=e).float()
    placement = ep_peer.balanced_placement(load, world)
    order = ep_peer.experts_of_rank(placement, rank, world).to(dev)
    pk_placed = [p.reshape(e, -1).index_select(0, order).reshape(-1) for p in all_pk]
    lora_placed = {n: v.index_select(0, order) for n, v in all_lora.items()}
    xchg_c = ep_peer.PeerExchange(t * k, h, e, device=dev, chunks=2)
    for _ in range(2):
        chunked = run(lambda hh, ll: ep_peer.peer_moe_layer(xchg_c, hh, idx, wts, *flat, q4k, i, ll, 2.0), hidden, lora, gout)
        assert torch.equal(chunked[0], whole[0][rows]), "chunked outputs differ from the single-device layer"
        assert torch.equal(chunked[1], whole[1][rows]), "chunked token gradients differ from the single-device layer"
        for got, want, name in zip(chunked[2:], whole[2:], lora):
            want = want[mine].float()
            err = float((got.float() - want).norm() / want.norm().clamp_min(1e-20))
            assert err <= 1e-2, (name, err)
    xchg2 = ep_peer.PeerExchange(t * k, h, e, device=dev, chunks=2, placement=placement)
    for _ in range(2):
        placed = run(lambda hh, ll: ep_peer.peer_moe_layer(xchg2, hh, idx, wts, *pk_placed, q4k, i, ll, 2.0), hidden, lora_placed, gout)
        assert torch.equal(placed[0], whole[0][rows]), "chunked / placed outputs differ from the single-device layer"
        d = float((placed[1].float() - whole[1][rows].float()).norm() / whole[1][rows].float().norm())
        assert d < 5e-3, ("token gradients under a placement", d)
        for got, want, name in zip(placed[2:], whole[2:], lora):
            want = want.index_select(0, order).float()
            err = float((got.float() - want).norm() / want.norm().clamp_min(1e-20))
            assert err <= 1e-2, (name, err)
    ops.check_status()
    print(f"rank {rank}: OK", flush=True)
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
