#!/usr/bin/env python
"""Benchmark of the quantized LoRA-linear hot path on B200.

One "step" = forward + backward of the three Q4_K LoRA linears of a Qwen3.5-35B-A3B attention
block (K = 2048, N in {4096, 512, 2048}, r = 16, alpha = 32) over M = 32768 tokens of synthetic
bf16 activations: Y = X.deq(W)^T + s.(X.A^T).B^T, then dX, dA, dB from a given dY.
Prints one JSON line (tokens/s, roofline of the dominant kernel, host-buffer e2e, CPU baseline).

    python bench.py                        # 1 GPU
    torchrun ... bench.py --gpus N ...     # N independent replicas (the dense path does not shard)
    python bench.py --impl reference       # the reference's dequantize-then-matmul path on the host CPU
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
PKG = ROOT / "transformers5-qwen3.5-recipe_b200"
sys.path.insert(0, str(PKG))
sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

K_DIM = 2048
N_DIMS = (4096, 512, 2048)
RANK, ALPHA = 16, 32
SCALING = ALPHA / RANK
Q4_K = 12
SEED = 19260817 + 1
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
# dram__bytes_read.sum + dram__bytes_write.sum of one qgemm_kernel<Q4_K, forward> launch at N=4096, K=2048, keyed by M
# (ncu captures summarised under profiles/)
DRAM_TRAFFIC_BYTES = {16384: 157.8e6, 32768: 359.6e6}


def flops_per_step(m: int) -> float:
    return float(sum(4 * m * n * K_DIM + 6 * m * RANK * (K_DIM + n) for n in N_DIMS))


def load_peaks() -> tuple[dict, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return json.loads(p.read_text()), "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


def make_inputs(m: int, device, with_payload=True):
    """Seeded synthetic weights/activations of the configuration, drawn on the CPU in a fixed order."""
    from b2g import gguf_quant

    g = torch.Generator().manual_seed(SEED)
    layers = []
    for n in N_DIMS:
        w = torch.randn(n, K_DIM, generator=g) * 0.02
        a = (torch.randn(RANK, K_DIM, generator=g) / 16).to(torch.bfloat16)
        b = (torch.randn(n, RANK, generator=g) * 0.01).to(torch.bfloat16)
        payload = gguf_quant.quantize_q4_k(w)
        layers.append({"n": n, "payload": payload.to(device) if with_payload else payload, "a": a.to(device), "b": b.to(device)})
    x = torch.randn(m, K_DIM, generator=g).to(torch.bfloat16)
    dys = [torch.randn(m, n, generator=g).to(torch.bfloat16) for n in N_DIMS]
    return layers, x, dys


class ClockSampler:
    """nvidia-smi clocks / throttle reasons, one sample every 100 ms, each stamped on arrival.

    The sampler is started before the warm-up so that it is already delivering when the timed region begins;
    ``begin()`` / ``end()`` mark the timed region and only samples that arrived while the load was running are
    summarised.  A timed region shorter than a few sampling periods is followed by ``extend(step)``: the same step
    keeps running, untimed, until at least ``MIN_SAMPLES`` samples have been taken under that load."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    MIN_SAMPLES = 3

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.rows = []                  # (arrival time, fields)
        self.t_begin = self.t_end = None
        self.extra_steps = 0

    def _pump(self):
        for line in self.proc.stdout:
            fields = [f.strip() for f in line.split(",")]
            if len(fields) >= 9:
                self.rows.append((time.monotonic(), fields))

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-i", str(self.gpu_index), "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:
            self.proc = None

    def begin(self):
        self.t_begin = time.monotonic()

    def end(self):
        self.t_end = time.monotonic()

    def _under_load(self):
        return [f for (t, f) in self.rows if self.t_begin is not None and t >= self.t_begin and (self.t_end is None or t <= self.t_end)]

    def extend(self, step, sync, limit_s: float = 4.0):
        """Keep the load of the timed region running (untimed) until enough samples were taken under it."""
        if self.proc is None or len(self._under_load()) >= self.MIN_SAMPLES:
            return
        self.t_end = None
        t0 = time.monotonic()
        while len(self._under_load()) < self.MIN_SAMPLES and time.monotonic() - t0 < limit_s:
            step()
            sync()
            self.extra_steps += 1
        self.t_end = time.monotonic()

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        try:
            self.proc.terminate()
            self.proc.wait(timeout=5)
        except Exception:
            pass
        rows = self._under_load()
        try:
            sm = [float(r[1]) for r in rows]
            names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
            reasons = set()
            for r in rows:
                for name, val in zip(names, r[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            if sm:
                out.update(sm_mhz=statistics.median(sm), sm_max_mhz=float(rows[0][2]), reasons=sorted(reasons), samples=len(sm),
                           power_w=statistics.median(float(r[3]) for r in rows),
                           window="timed region" + (f" + {self.extra_steps} identical untimed steps run directly after it" if self.extra_steps else ""))
        except Exception:
            pass
        return out


# ---------------------------------------------------------------------------------------------
# CPU arm: the reference's dequantize-then-matmul path (oracle port) on the host cores
# ---------------------------------------------------------------------------------------------
def cpu_step_fn(layers_cpu):
    from oracle import dense_ref

    weights = [dense_ref.dequant_bf16(l["payload"].numpy(), Q4_K) for l in layers_cpu]   # outside the timed region

    def step(x, dys):
        for l, w, dy in zip(layers_cpu, weights, dys):
            dense_ref.lora_linear_fwd_bwd(x, w, l["a"], l["b"], SCALING, dy, torch.bfloat16)

    return step


def run_cpu(steps: int, warmup: int, budget_s: float, m_full: int) -> dict:
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    layers, x, dys = make_inputs(m_full, "cpu")
    step = cpu_step_fn(layers)
    step(x[:64], [d[:64] for d in dys])                      # first-call overheads
    t0 = time.perf_counter()
    step(x[:512], [d[:512] for d in dys])
    per_row = (time.perf_counter() - t0) / 512
    per_step_budget = max(0.05, budget_s / max(1, steps + warmup))
    m = int(min(m_full, max(64, per_step_budget / per_row)))   # the whole workload when the budget allows, else a prefix of it
    m = max(64, m // 64 * 64)
    xs, ds = x[:m].contiguous(), [d[:m].contiguous() for d in dys]
    for _ in range(warmup):
        step(xs, ds)
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        step(xs, ds)
        times.append(time.perf_counter() - t0)
    total = sum(times)
    return {"tokens_per_s": m * steps / total, "ms_per_step": 1e3 * total / steps, "cores": threads, "m": m,
            "sample": f"{m} of {m_full} tokens per step through the same three linears, weights dequantised once outside the timed region, "
                      f"{steps} timed steps, torch {torch.get_num_threads()} threads"}


# ---------------------------------------------------------------------------------------------
# MoE workloads: the grouped Q4_K expert layer (256 experts, top-8, hidden 2048, intermediate 512, r = 16)
#   "qwen16k"  16384 tokens on one GPU, unbiased router                       (configuration 2 of the benchmark specification)
#   "skew64k"  65536 tokens in total, router logits N(0,1) + a per-expert bias N(0,0.5): on one GPU, or expert-parallel
#              over N ranks with the experts sharded 256/N per GPU              (configuration 4)
#   "deepseek" 8192 tokens, 256 IQ2_XXS experts top-6 (hidden 4096, intermediate 2048, r = 8, clamped SwiGLU) plus the Q8_0
#              shared expert, one GPU                                            (configuration 3)
# ---------------------------------------------------------------------------------------------
MOE = {"E": 256, "H": 2048, "I": 512, "K": 8, "R": 16, "Q": 12}
DSK = {"E": 256, "H": 4096, "I": 2048, "K": 6, "R": 8, "Q": 16, "limit": 7.0}


def moe_flops(tokens: int, g=MOE, shared: bool = False) -> float:
    rows = tokens * g["K"]
    f = 4.0 * rows * 3 * g["H"] * g["I"] + 6.0 * rows * g["R"] * ((g["H"] + 2 * g["I"]) + (g["I"] + g["H"]))
    if shared:
        f += 3 * (4.0 * tokens * g["H"] * g["I"] + 6.0 * tokens * g["R"] * (g["H"] + g["I"]))
    return f


def _expert_bank(dev, qtype: int, expert_ids, num_experts: int, rows: int, cols: int, seed: int):
    """Packed weights of the experts ``expert_ids`` (in that order), flattened.  The whole bank of ``num_experts`` experts is
    drawn from one seeded stream in expert-id order, 32 experts at a time, and the wanted ones are kept, so that an expert has
    the same bytes whichever rank holds it and the set-up costs a few dozen launches: N(0, 0.02) through the Q4_K encoder, or
    seeded random valid blocks of that spread for the types without an encoder."""
    from b2g import gguf_quant

    g = torch.Generator(device=dev).manual_seed(seed)
    want = torch.as_tensor(list(expert_ids), dtype=torch.int64, device=dev)
    keep = [None] * len(want)
    for e0 in range(0, num_experts, 32):
        n = min(32, num_experts - e0)
        if qtype == 12:
            chunk = gguf_quant.quantize_q4_k(torch.randn(n, rows, cols, generator=g, device=dev) * 0.02)
        else:
            chunk = gguf_quant.random_payload(qtype, (n, rows, cols), seed + e0, device=dev)
        for pos, e in enumerate(want.tolist()):
            if e0 <= e < e0 + n:
                keep[pos] = chunk[e - e0]
    return torch.stack(keep).reshape(-1)


def _moe_factors(dev, expert_ids, g, seed: int, requires_grad=True):
    gen = torch.Generator(device=dev).manual_seed(seed)
    e = g["E"]
    full = {"gate_up_a": torch.randn(e, g["R"], g["H"], generator=gen, device=dev) / 16,
            "gate_up_b": torch.randn(e, 2 * g["I"], g["R"], generator=gen, device=dev) * 0.01,
            "down_a": torch.randn(e, g["R"], g["I"], generator=gen, device=dev) / 16,
            "down_b": torch.randn(e, g["H"], g["R"], generator=gen, device=dev) * 0.01}
    mine = torch.as_tensor(list(expert_ids), dtype=torch.int64, device=dev)
    return {n: v.index_select(0, mine).bfloat16().requires_grad_(requires_grad) for n, v in full.items()}


def _time_steps(step, steps: int, barrier) -> float:
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    barrier()
    return e0.elapsed_time(e1) / steps


def measure_moe(kind: str, args, dev, dist, rank: int, world: int, steps: int, warmup: int, cpu_baseline: bool = True) -> dict:
    """One MoE workload in this process (all ranks call it together); returns the object rank 0 prints."""
    from b2g import _lib, autograd as ag, ep_peer, ops, routing

    g = DSK if kind == "deepseek" else MOE
    E, H, I, TOPK, QT = g["E"], g["H"], g["I"], g["K"], g["Q"]
    if getattr(args, "qtype", None):
        QT = int(args.qtype)                             # the same layer in another packed format (side measurement)
    scaling = 2.0
    limit = g.get("limit", 0.0)
    t_total = {"qwen16k": 16384, "skew64k": 65536, "deepseek": 8192}[kind]
    skew = kind == "skew64k"
    t_local = t_total // world
    gen = torch.Generator(device=dev).manual_seed(SEED + 1 + rank)
    hidden = torch.randn(t_local, H, generator=gen, device=dev).bfloat16()
    g_out = torch.randn(t_local, H, generator=gen, device=dev).bfloat16()
    logits = torch.randn(t_local, E, generator=gen, device=dev)
    if skew:
        logits = logits + torch.randn(E, generator=torch.Generator(device=dev).manual_seed(SEED + 4), device=dev) * 0.5   # same bias on every rank

    # expert load of this batch (what a static placement is fitted to) and the placement
    idx0 = ops.router_topk(logits, TOPK, None, False)
    load = torch.bincount(idx0.flatten(), minlength=E).double()
    if world > 1:
        dist.all_reduce(load)
    contiguous = ep_peer.contiguous_placement(E)
    placement = ep_peer.balanced_placement(load, world, args.chunks) if (world > 1 and args.placement == "balanced") else contiguous
    loads = ep_peer.rank_loads(load, placement, world)
    loads_contiguous = ep_peer.rank_loads(load, contiguous, world)
    mine = ep_peer.experts_of_rank(placement, rank, world).tolist()
    gate_p, up_p, down_p = (_expert_bank(dev, QT, mine, E, I, H, 1000), _expert_bank(dev, QT, mine, E, I, H, 2000), _expert_bank(dev, QT, mine, E, H, I, 3000))
    lora = _moe_factors(dev, mine, g, 4000)
    ids = torch.arange(E // world, device=dev, dtype=torch.int64)
    shared = None
    if kind == "deepseek":
        from b2g.gguf_types import GGUFQuantizedTensor
        from b2g.moe_block import SharedExpertLora
        from b2g import gguf_quant

        sg = torch.Generator(device=dev).manual_seed(SEED + 7)
        sp = [gguf_quant.quantize_q8_0(torch.randn(*shape, generator=sg, device=dev) * 0.02) for shape in ((I, H), (I, H), (H, I))]
        shared = SharedExpertLora(*(GGUFQuantizedTensor(p, quant_type=8, logical_shape=shape) for p, shape in zip(sp, ((I, H), (I, H), (H, I)))),
                                  r=g["R"], lora_alpha=2 * g["R"], swiglu_limit=limit)
        with torch.no_grad():
            for name in ("gate", "up", "down"):
                shared.lora_B[name].normal_(std=0.01, generator=sg)
    xchg = None
    if world > 1:
        xchg = ep_peer.PeerExchange(t_local * TOPK, H, E, device=dev, chunks=args.chunks, placement=None if placement is contiguous else placement,
                                    exchange_tpcs=args.exchange_tpcs)

    def layer(h, lg):
        idx = ops.router_topk(lg, TOPK, None, False)
        wts = torch.softmax(lg.gather(1, idx), dim=-1)
        if xchg is not None:
            return ep_peer.peer_moe_layer(xchg, h, idx, wts, gate_p, up_p, down_p, QT, I, lora, scaling)
        plan = routing.build_plan(h, idx, wts, E)
        out_e = ag.grouped_lora_experts(plan.selected_hidden_states, gate_p, up_p, down_p, QT, QT, I, ids, plan.group_offsets, plan.group_offsets,
                                        lora["gate_up_a"], lora["gate_up_b"], lora["down_a"], lora["down_b"], scaling, limit)
        out = routing.combine(out_e, plan)
        return out if shared is None else out + shared(h)

    def zero_grads():
        for v in lora.values():
            v.grad = None
        if shared is not None:
            shared.zero_grad(set_to_none=True)

    def step():
        h = hidden.detach().requires_grad_(True)
        zero_grads()
        out = layer(h, logits)
        out.backward(g_out)
        return out, h.grad

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(3, warmup)):
        step()
    barrier()
    ops.check_status()
    _lib.COUNT_LAUNCHES, _lib.LAUNCHES = True, 0
    ms = _time_steps(step, steps, barrier)
    launches = _lib.LAUNCHES // max(1, steps)
    _lib.COUNT_LAUNCHES = False

    # per-kernel device times of a few more steps (CUDA events around the entry points, on the launching stream)
    kernel_ms: dict[str, float] = {}
    _lib.TIMED = {"b2g_grouped_fwd", "b2g_grouped_dgrad", "b2g_route_gather", "b2g_route_gather_bwd", "b2g_route_combine", "b2g_route_combine_bwd",
                  "b2g_ep_scatter_rows", "b2g_ep_return_rows"}
    _lib.EVENTS.clear()
    prof_steps = 3
    if xchg is not None:
        xchg.profile, xchg.trace = True, []
    for _ in range(prof_steps):
        step()
    torch.cuda.synchronize()
    for name, key, a, b in _lib.EVENTS:
        label = name[4:] + ("" if name not in ("b2g_grouped_fwd", "b2g_grouped_dgrad") else f"[N={key[0]},K={key[1]}]")
        kernel_ms[label] = kernel_ms.get(label, 0.0) + a.elapsed_time(b) / prof_steps
    _lib.TIMED = set()
    _lib.EVENTS.clear()
    phases = None
    if xchg is not None:
        if args.timeline and rank == 0:
            spans = xchg.timeline()
            per_step = len(spans) // prof_steps
            t0 = spans[-per_step][1]
            sys.stderr.write("timeline of the last profiled step on rank 0 (ms):\n" + "".join(
                f"  {name:18s} {a - t0:7.3f} -> {b - t0:7.3f}\n" for name, a, b in spans[-per_step:]))
        phases = {k: v / prof_steps for k, v in xchg.phase_ms().items()}
        xchg.profile, xchg.trace = False, []
    barrier()

    # end to end: hidden states, router logits and the output cotangent from pinned host memory, output and token gradient back
    pins = [t.cpu().pin_memory() for t in (hidden, logits, g_out)]
    stage = [torch.empty_like(t) for t in (hidden, logits, g_out)]
    back = [torch.empty(t_local, H, dtype=torch.bfloat16).pin_memory() for _ in range(2)]

    def step_e2e():
        for dst, src in zip(stage, pins):
            dst.copy_(src, non_blocking=True)
        h = stage[0].detach().requires_grad_(True)
        zero_grads()
        out = layer(h, stage[1])
        out.backward(stage[2])
        back[0].copy_(out.detach(), non_blocking=True)
        back[1].copy_(h.grad, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for _ in range(2):
        step_e2e()
    ms_e2e = _time_steps(step_e2e, max(3, min(steps, 10)), barrier)
    if world > 1:
        t = torch.tensor([ms, ms_e2e], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_e2e = float(t[0]), float(t[1])
        if phases:
            names = sorted(phases)
            pt = torch.tensor([phases[n] for n in names], device=dev, dtype=torch.float64)
            dist.all_reduce(pt, op=dist.ReduceOp.MAX)
            phases = {n: float(v) for n, v in zip(names, pt)}
    ops.check_status()
    del xchg

    peaks, peak_src = load_peaks()
    peak_tf = float(peaks.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]))
    hbm = float(peaks.get("hbm_gbs", FALLBACK_PEAKS["hbm_gbs"]))
    flops = moe_flops(t_total, g, shared is not None)
    rows_local = t_local * TOPK
    out = {"workload": {"qwen16k": "grouped MoE Q4_K LoRA, 256 experts top-8, hidden 2048, intermediate 512, r=16, 16384 tokens (configuration 2 of the benchmark specification)",
                        "skew64k": "the same experts, 65536 tokens in total, router logits N(0,1) + per-expert bias N(0,0.5) (configuration 4)",
                        "deepseek": "grouped MoE IQ2_XXS LoRA, 256 experts top-6, hidden 4096, intermediate 2048, r=8, clamped SwiGLU, plus the Q8_0 shared expert, 8192 tokens (configuration 3)"}[kind],
           "n_gpus": world, "tokens_total": t_total, "scaling": "strong" if skew else "weak", "steps": steps, "expert_quant_type": QT,
           "parallelism": "1 GPU" if world == 1 else f"ep{world}: {E // world} experts per GPU, peer-store dispatch / combine over NVLink, {args.chunks} expert groups pipelined on an exchange stream ({('%d TPCs of its own' % args.exchange_tpcs) if args.exchange_tpcs and args.chunks > 1 else 'sharing the SMs'}), {args.placement} placement",
           "ms_per_step": ms, "tokens_per_s": t_total / (ms * 1e-3), "step_tflops": flops / (ms * 1e-3) / 1e12,
           "frac_of_tensor_peak_all_gpus": flops / (ms * 1e-3) / 1e12 / (peak_tf * world), "peak_source": peak_src,
           "max_over_mean_rows": float(loads.max() / loads.mean()), "max_over_mean_rows_contiguous_blocks": float(loads_contiguous.max() / loads_contiguous.mean()),
           "kernel_ms_per_step": {k: round(v, 4) for k, v in sorted(kernel_ms.items())}, "gpu_launches_per_step": launches,
           "e2e": {"value": t_total / (ms_e2e * 1e-3), "unit": "tokens/s", "ms_per_step": ms_e2e,
                   "h2d_bytes_per_step": sum(p.numel() * p.element_size() for p in pins), "d2h_bytes_per_step": 2 * t_local * H * 2,
                   "result": "layer output and token gradient"}}
    if phases:
        out["phases_ms_max_over_ranks"] = {k: round(v, 4) for k, v in phases.items()}
    pair = kernel_ms.get(f"grouped_fwd[N={I},K={H}]")
    if pair:
        achieved = 2.0 * rows_local * (2 * I) * H / (pair * 1e-3) / 1e12       # this rank's rows x both payloads; ragged rows counted once
        out["roofline"] = {"bound": "tensor", "kernel": f"qgemm_kernel grouped forward, gate|up pair, rows={rows_local} (this rank: mean over ranks), N=2x{I}, K={H}",
                           "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s", "frac": achieved / peak_tf, "kernel_ms": pair, "traffic": None}
    perm_ms = sum(kernel_ms.get(n, 0.0) for n in ("route_gather", "route_gather_bwd", "route_combine", "route_combine_bwd"))
    if perm_ms and world == 1:
        nbytes = 2.0 * H * (5 * rows_local + 4 * t_local)
        out["permute_roofline"] = {"bound": "hbm", "kernels": "gather, combine and their backwards", "achieved": nbytes / (perm_ms * 1e-3) / 1e9, "peak": hbm,
                                   "unit": "GB/s", "frac": nbytes / (perm_ms * 1e-3) / 1e9 / hbm, "kernels_ms": perm_ms, "traffic": None}
    if cpu_baseline and rank == 0 and world == 1:
        res = run_cpu_moe(kind, budget_s=12.0)
        out["cpu_baseline"] = {"value": res["tokens_per_s"], "unit": "tokens/s", "cores": res["cores"], "kind": "port", "sample": res["sample"]}
    return out


def run_cpu_moe(kind: str, budget_s: float = 12.0, steps: int = 2) -> dict:
    """The reference's CPU path for the MoE layer (per-expert loop of matmuls on dequantised weights, autograd backward:
    ``oracle/moe_ref.moe_layer``) on a bounded sample: 1/8 (Qwen shape) or 1/32 (DeepSeek shape) of the experts and the same
    fraction of the tokens, routed among those experts, so that the work per token and the rows per expert are those of the
    full layer.  Weights are dequantised once outside the timed region."""
    from concurrent.futures import ThreadPoolExecutor

    from b2g import gguf_quant
    from oracle import dense_ref, gguf_oracle as go, moe_ref

    g = DSK if kind == "deepseek" else MOE
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    frac = 32 if kind == "deepseek" else 8
    e_s = g["E"] // frac
    t_full = {"qwen16k": 16384, "skew64k": 65536, "deepseek": 8192}[kind]
    t_s = t_full // frac
    qt = g["Q"]
    gen = torch.Generator().manual_seed(SEED + 11)
    shapes = ((e_s, g["I"], g["H"]), (e_s, g["I"], g["H"]), (e_s, g["H"], g["I"]))
    payloads = [gguf_quant.random_payload(qt, s, 50 + j).numpy() for j, s in enumerate(shapes)]
    with ThreadPoolExecutor(max_workers=min(threads, e_s)) as ex:
        weights = [torch.stack(list(ex.map(lambda one: dense_ref.dequant_bf16(one, qt), list(p)))) for p in payloads]
    lora = {"gate_up_a": (torch.randn(e_s, g["R"], g["H"], generator=gen) / 16).bfloat16(), "gate_up_b": (torch.randn(e_s, 2 * g["I"], g["R"], generator=gen) * 0.01).bfloat16(),
            "down_a": (torch.randn(e_s, g["R"], g["I"], generator=gen) / 16).bfloat16(), "down_b": (torch.randn(e_s, g["H"], g["R"], generator=gen) * 0.01).bfloat16()}
    hidden = torch.randn(t_s, g["H"], generator=gen).bfloat16()
    gout = torch.randn(t_s, g["H"], generator=gen).bfloat16()
    logits = torch.randn(t_s, e_s, generator=gen)
    idx = logits.topk(g["K"], 1).indices
    wts = torch.softmax(logits.gather(1, idx), -1)

    def step():
        moe_ref.moe_layer(hidden, idx, wts, *weights, lora, 2.0, gout, torch.bfloat16, swiglu_limit=g.get("limit"))

    t0 = time.perf_counter()
    step()
    first = time.perf_counter() - t0
    steps = max(1, min(steps, int(budget_s / max(first, 1e-3))))
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
    sec = statistics.median(times)
    return {"tokens_per_s": t_s / sec, "ms_per_step": 1e3 * sec, "cores": threads,
            "sample": f"{t_s} of {t_full} tokens routed top-{g['K']} among {e_s} of {g['E']} experts (same rows per expert and work per token as the full layer"
                      f"{', routed experts only: the shared expert is left out' if kind == 'deepseek' else ''}), weights dequantised once outside the timed region, "
                      f"{steps} timed steps after one warm-up, torch {torch.get_num_threads()} threads"}


def run_moe(args) -> int:
    """`--workload moe` (qwen16k on one GPU / skew64k expert-parallel on several), `--workload moe64k`, `--workload moe3`."""
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    kind = {"moe": "qwen16k" if world == 1 else "skew64k", "moe64k": "skew64k", "moe3": "deepseek"}[args.workload]
    if args.impl == "reference":
        if rank == 0:
            res = run_cpu_moe(kind, budget_s=120.0, steps=max(1, args.steps))
            print(json.dumps({"impl": "reference", "metric": "quantized MoE fwd+bwd tokens/s", "value": res["tokens_per_s"], "unit": "tokens/s",
                              "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": res["ms_per_step"], "higher_is_better": True,
                              "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": {"workload": kind},
                              "cpu_baseline": {"value": res["tokens_per_s"], "unit": "tokens/s", "cores": res["cores"], "kind": "port", "sample": res["sample"]},
                              "e2e": {"value": res["tokens_per_s"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return 0
    if kind == "deepseek" and world > 1:
        if rank == 0:
            print(json.dumps({"error": "the DeepSeek-shaped workload is measured on one GPU"}))
        return 1
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist = dist_mod
        dist.init_process_group("nccl", device_id=dev)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        sampler.begin()
    torch.cuda.profiler.start()                   # `ncu --profile-from-start off` then skips set-up
    res = measure_moe(kind, args, dev, dist, rank, world, args.steps, args.warmup, cpu_baseline=not args.no_cpu_baseline)
    torch.cuda.profiler.stop()
    if rank == 0:
        sampler.end()
        clocks = sampler.stop()
        print(json.dumps({"metric": "quantized MoE (grouped experts + LoRA) fwd+bwd tokens/s", "value": res["tokens_per_s"], "unit": "tokens/s",
                          "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": res["ms_per_step"],
                          "higher_is_better": True, "scaling": res["scaling"], "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                          "config": {"workload": res["workload"], "parallelism": res["parallelism"], "l2": "routed rows far larger than L2"},
                          "clocks": clocks, "gpu_launches": res["gpu_launches_per_step"] * args.steps, **{k: v for k, v in res.items() if k not in ("workload", "parallelism")}}))
    if dist is not None:
        dist.destroy_process_group()
    return 0


def _event_ms(fn, warmup: int, steps: int) -> float:
    for _ in range(max(3, warmup)):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / steps


def run_side(args) -> int:
    """Single-GPU measurements of the rows next to the headline path, one JSON line each run:
      formats : forward / input-gradient product of every native GGUF type at M=32768, N=4096, K=2048
      fixed   : the fixed-group projection (Q8_0, 8 x (4096 -> 1024), 16384 rows), forward and input gradient
      lmhead  : packed LM-head chunked cross-entropy, loss + hidden-state gradient (Q8_0 129280 x 4096 and Q6_K 248320 x 2048
                heads, 4096 tokens)
    Inputs are seeded random valid blocks and normal activations, all larger than L2; CUDA events on the launching stream."""
    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device: the product path has no CPU fallback"}))
        return 1
    if int(os.environ.get("RANK", "0")) != 0:
        return 0
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    from b2g import gguf_quant, ops

    peaks, peak_src = load_peaks()
    peak_tf = float(peaks.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]))
    gen = torch.Generator(device=dev).manual_seed(SEED)
    base = {"n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup), "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
            "peak_tflops": peak_tf, "peak_source": peak_src}
    if args.workload == "formats":
        m, n, k = args.tokens, 4096, K_DIM
        x = torch.randn(m, k, generator=gen, device=dev).bfloat16()
        dy = torch.randn(m, n, generator=gen, device=dev).bfloat16()
        tf = 2.0 * m * n * k / 1e12
        names = {8: "Q8_0", 10: "Q2_K", 11: "Q3_K", 12: "Q4_K", 13: "Q5_K", 14: "Q6_K", 16: "IQ2_XXS", 22: "IQ2_S"}
        out = {}
        for qt, name in names.items():
            p = gguf_quant.random_payload(qt, (n, k), 1, device=dev).reshape(-1)
            f = _event_ms(lambda: ops.qlinear_fwd(x, p, qt, n), args.warmup, args.steps)
            g = _event_ms(lambda: ops.qlinear_dgrad(dy, p, qt, k), args.warmup, args.steps)
            out[name] = {"forward_ms": f, "forward_tflops": tf / f * 1e3, "dgrad_ms": g, "dgrad_tflops": tf / g * 1e3}
        ops.check_status()
        print(json.dumps({**base, "metric": "packed-weight product TFLOP/s per GGUF type", "unit": "TFLOP/s",
                          "config": {"workload": "dense product, every native type", "M": m, "N": n, "K": k}, "kernels": out}))
        return 0
    if args.workload == "fixed":
        rows, groups, n, k = 16384, 8, 1024, 4096
        x = torch.randn(rows, groups, k, generator=gen, device=dev).bfloat16()
        dy = torch.randn(rows, groups, n, generator=gen, device=dev).bfloat16()
        p = gguf_quant.random_payload(8, (groups * n, k), 3, device=dev).reshape(groups, n, -1)
        tf = 2.0 * rows * groups * n * k / 1e12
        f = _event_ms(lambda: ops.fixed_grouped_fwd(x, p, 8), args.warmup, args.steps)
        g = _event_ms(lambda: ops.fixed_grouped_dgrad(dy, p, 8), args.warmup, args.steps)
        ops.check_status()
        print(json.dumps({**base, "metric": "fixed-group projection rows/s (forward + input gradient)", "value": rows / ((f + g) * 1e-3),
                          "unit": "rows/s", "ms_per_step": f + g,
                          "config": {"workload": "fixed groups Q8_0", "rows": rows, "groups": groups, "in": k, "out": n},
                          "forward_tflops": tf / f * 1e3, "dgrad_tflops": tf / g * 1e3}))
        return 0
    import deepseek_v4_liger_loss as dl

    tokens = 4096
    out = {}
    for name, qt, vocab, hidden in (("Q8_0 129280x4096", 8, 129280, 4096), ("Q6_K 248320x2048", 14, 248320, 2048)):
        head = gguf_quant.random_payload(qt, (vocab, hidden), 5, device=dev)
        h = torch.randn(tokens, hidden, generator=gen, device=dev).bfloat16()
        t = torch.randint(0, vocab, (tokens,), generator=gen, device=dev)
        ms = _event_ms(lambda: dl._packed_q8_linear_cross_entropy_forward(h, head, t, qt, vocab, dl._PACKED_LM_HEAD_CHUNK_SIZE, -100, 0.0, 0.0,
                                                                            "mean", None), args.warmup, args.steps)
        out[name] = {"ms": ms, "tokens_per_s": tokens / (ms * 1e-3), "tflops_both_products": 4.0 * tokens * vocab * hidden / ms / 1e9}
        del head
    ops.check_status()
    print(json.dumps({**base, "metric": "packed LM-head loss + hidden gradient tokens/s", "unit": "tokens/s",
                      "config": {"workload": "packed LM-head chunked cross-entropy", "tokens": tokens, "chunk_rows": dl._PACKED_LM_HEAD_CHUNK_SIZE},
                      "heads": out}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--tokens", type=int, default=32768, help="M: tokens per step and per GPU")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--workload", default="dense", choices=["dense", "moe", "moe64k", "moe3", "formats", "fixed", "lmhead"],
                    help="dense: the Q4_K attention-shape linears plus a `moe` object (default; dense replicas and the expert-parallel MoE layer at N>1); "
                         "moe: grouped Q4_K experts alone, 16384 tokens on one GPU / 65536 tokens expert-parallel at N>1; moe64k: the 65536-token "
                         "layer at any N; moe3: the DeepSeek-shaped IQ2_XXS layer with its shared expert; formats / fixed / lmhead: single-GPU side measurements (see run_side)")
    ap.add_argument("--chunks", type=int, default=2, help="expert-parallel MoE: token chunks whose exchanges overlap the expert products")
    ap.add_argument("--exchange-tpcs", type=int, default=12,
                    help="expert-parallel MoE: TPCs (pairs of SMs) set aside for the exchanges that run beside expert products; 0 = they share the GEMM's SMs")
    ap.add_argument("--placement", default="balanced", choices=["balanced", "contiguous"],
                    help="expert-parallel MoE: experts placed over the ranks by measured load (default) or in contiguous blocks")
    ap.add_argument("--no-moe", action="store_true", help="dense workload: leave the `moe` object out")
    ap.add_argument("--qtype", type=int, default=None, help="MoE workloads: GGML type id of the expert weights instead of the workload's own (8, 10-14, 16, 22)")
    ap.add_argument("--timeline", action="store_true", help="expert-parallel MoE: print rank 0's phase timeline of one step to stderr")
    args = ap.parse_args()
    if args.workload in ("moe", "moe64k", "moe3"):
        return run_moe(args)
    if args.workload in ("formats", "fixed", "lmhead"):
        return run_side(args)
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    m = args.tokens
    config = {"workload": "dense Q4_K LoRA linears, Qwen3.5-35B-A3B attention shapes (configuration 1 of the benchmark specification)",
              "K": K_DIM, "N": list(N_DIMS), "M_tokens_per_gpu": m, "lora_rank": RANK, "lora_alpha": ALPHA,
              "parallelism": f"replicas x{args.gpus} (dense path does not shard)", "l2": "inputs larger than L2 (X 128 MiB, dY up to 256 MiB)"}

    if args.impl == "reference":
        if rank != 0:
            return 0
        res = run_cpu(args.steps, max(1, args.warmup), budget_s=150.0, m_full=m)
        line = {"impl": "reference", "metric": "quantized LoRA-linear fwd+bwd tokens/s", "value": res["tokens_per_s"], "unit": "tokens/s",
                "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": res["ms_per_step"],
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": config,
                "cpu_baseline": {"value": res["tokens_per_s"], "unit": "tokens/s", "cores": res["cores"], "kind": "port", "sample": res["sample"]},
                "e2e": {"value": res["tokens_per_s"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        if not args.no_moe:
            # the same CPU path for the MoE layers of the `moe` object of the other arm (the sample has the per-token work of
            # both the 16384- and the 65536-token layer: same experts, same top-8)
            cpu_moe = run_cpu_moe("qwen16k", budget_s=20.0, steps=3)
            line["moe"] = {"cpu_tokens_per_s": cpu_moe["tokens_per_s"], "ms_per_step": cpu_moe["ms_per_step"], "cores": cpu_moe["cores"],
                           "kind": "port", "sample": cpu_moe["sample"]}
        print(json.dumps(line))
        return 0

    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device: the product path has no CPU fallback"}))
        return 1
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist = dist_mod
        dist.init_process_group("nccl", device_id=dev)

    from b2g import _lib, autograd as ag, ops

    layers, x_cpu, dys_cpu = make_inputs(m, dev)
    x_pin = x_cpu.pin_memory()
    dys_pin = [d.pin_memory() for d in dys_cpu]
    x_dev = x_cpu.to(dev)
    dys_dev = [d.to(dev) for d in dys_cpu]
    for l in layers:
        l["a"].requires_grad_(True)
        l["b"].requires_grad_(True)

    def step(x, dys):
        x = x.detach().requires_grad_(True)
        for l in layers:
            l["a"].grad = None
            l["b"].grad = None
        outs = [ag.lora_qlinear(x, l["payload"], Q4_K, l["n"], l["a"], l["b"], SCALING) for l in layers]
        torch.autograd.backward(outs, dys)
        return x.grad

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(max(3, args.warmup)):
        step(x_dev, dys_dev)
    torch.cuda.synchronize()
    ops.check_status()

    # ---- timed region: inputs resident in HBM ----
    _lib.COUNT_LAUNCHES = True
    _lib.LAUNCHES = 0
    _lib.TIMED = {"b2g_qlinear_fwd"}
    _lib.EVENTS.clear()
    barrier()
    sampler.begin()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    torch.cuda.profiler.start()                   # `ncu --profile-from-start off` then sees only the timed steps (all threads)
    for _ in range(args.steps):
        step(x_dev, dys_dev)
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    e1.record()
    barrier()
    sampler.end()
    ms_total = e0.elapsed_time(e1)
    launches = _lib.LAUNCHES
    _lib.COUNT_LAUNCHES = False
    _lib.TIMED = set()
    if rank == 0:
        sampler.extend(lambda: step(x_dev, dys_dev), torch.cuda.synchronize)    # replicas are independent: rank 0 may run on alone
    clocks = sampler.stop() if rank == 0 else {}
    ops.check_status()

    # dominant kernel: the quantized forward GEMM of the widest layer, timed by CUDA events on its stream
    n_big = max(N_DIMS)
    durs = [a.elapsed_time(b) for (name, key, a, b) in _lib.EVENTS if key == (m, n_big, K_DIM)]
    _lib.EVENTS.clear()
    kernel_ms = statistics.mean(durs) if durs else None

    # ---- e2e: host buffers in, host buffers out ----
    grads_host = [(torch.empty_like(l["a"], device="cpu").pin_memory(), torch.empty_like(l["b"], device="cpu").pin_memory()) for l in layers]
    x_stage = torch.empty_like(x_dev)
    dys_stage = [torch.empty_like(d) for d in dys_dev]

    # The step is bound by the host link (0.57 GB in, 10 ms), so the copies run on a stream of their own and the work starts
    # as its operands land: the forward after X, each layer's backward after its own dY.  The widest dY goes first, so that
    # only the narrowest layer's backward is left when the last byte arrives.
    copy_stream = torch.cuda.Stream()
    order = sorted(range(len(layers)), key=lambda i: -layers[i]["n"])
    landed = [torch.cuda.Event() for _ in layers]
    x_landed = torch.cuda.Event()

    def step_e2e():
        main = torch.cuda.current_stream()
        with torch.cuda.stream(copy_stream):
            x_stage.copy_(x_pin, non_blocking=True)
            x_landed.record(copy_stream)
            for i in order:
                dys_stage[i].copy_(dys_pin[i], non_blocking=True)
                landed[i].record(copy_stream)
        main.wait_event(x_landed)
        x = x_stage.detach().requires_grad_(True)
        for l in layers:
            l["a"].grad = None
            l["b"].grad = None
        outs = [ag.lora_qlinear(x, l["payload"], Q4_K, l["n"], l["a"], l["b"], SCALING) for l in layers]
        for i in order:
            main.wait_event(landed[i])
            outs[i].backward(dys_stage[i])
        for (ha, hb), l in zip(grads_host, layers):
            ha.copy_(l["a"].grad, non_blocking=True)
            hb.copy_(l["b"].grad, non_blocking=True)
        torch.cuda.current_stream().synchronize()          # the host reads the step's result

    e2e_steps = max(3, min(args.steps, 10))
    for _ in range(2):
        step_e2e()
    barrier()
    e0.record()
    for _ in range(e2e_steps):
        step_e2e()
    e1.record()
    barrier()
    ms_e2e = e0.elapsed_time(e1)
    h2d = x_pin.numel() * 2 + sum(d.numel() * 2 for d in dys_pin)
    d2h = sum(a.numel() * 2 + b.numel() * 2 for a, b in grads_host)

    if dist is not None:
        t = torch.tensor([ms_total, ms_e2e], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total, ms_e2e = float(t[0]), float(t[1])

    if rank == 0:
        peaks, peak_src = load_peaks()
        ms_step = ms_total / args.steps
        value = world * m / (ms_step * 1e-3)
        flops = flops_per_step(m)
        peak_tf = float(peaks.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]))
        roof = None
        if kernel_ms:
            achieved = 2.0 * m * n_big * K_DIM / (kernel_ms * 1e-3) / 1e12
            roof = {"bound": "tensor", "kernel": "qgemm_kernel<Q4_K, forward> M=%d N=%d K=%d" % (m, n_big, K_DIM),
                    "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s", "frac": achieved / peak_tf,
                    "peak_source": f"{peak_src} burst cuBLAS bf16", "kernel_ms": kernel_ms,
                    # dram__bytes_read + dram__bytes_write of one launch, from an ncu capture of this kernel at the size named
                    # (profiles/); no figure is quoted for a size that was not captured
                    "traffic": DRAM_TRAFFIC_BYTES.get(m), "traffic_unit": "bytes/launch",
                    "algorithmic_bytes": 2.0 * m * (K_DIM + n_big) + n_big * K_DIM * 0.5625}
        line = {"metric": "quantized LoRA-linear fwd+bwd tokens/s", "value": value, "unit": "tokens/s", "n_gpus": world,
                "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_step, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config,
                "step_tflops": world * flops / (ms_step * 1e-3) / 1e12,
                "step_frac_of_tensor_peak": flops / (ms_step * 1e-3) / 1e12 / peak_tf,
                "roofline": roof, "clocks": clocks, "gpu_launches": launches,
                "e2e": {"value": world * m / (ms_e2e / e2e_steps * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                        "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e / e2e_steps,
                        "result": "adapter gradients dA, dB of the three layers (what the optimizer step reads); Y and dX stay on the device "
                                  "for the neighbouring layers"}}
        if world == 1 and not args.no_cpu_baseline:
            res = run_cpu(5, 2, budget_s=24.0, m_full=m)
            line["cpu_baseline"] = {"value": res["tokens_per_s"], "unit": "tokens/s", "cores": res["cores"], "kind": "port", "sample": res["sample"]}
    # ---- the MoE layer, in the same process: the path that shards over the GPUs ----
    moe = None
    if not args.no_moe:
        del x_dev, dys_dev, x_stage, dys_stage, x_pin, dys_pin
        torch.cuda.empty_cache()
        moe_steps = max(3, min(args.steps, 10))
        if world == 1:
            moe = {"one_gpu_16k_tokens": measure_moe("qwen16k", args, dev, dist, rank, world, moe_steps, args.warmup, cpu_baseline=not args.no_cpu_baseline),
                   "one_gpu_64k_tokens_skewed": measure_moe("skew64k", args, dev, dist, rank, world, moe_steps, args.warmup, cpu_baseline=False)}
        else:
            moe = {"expert_parallel_64k_tokens_skewed": measure_moe("skew64k", args, dev, dist, rank, world, moe_steps, args.warmup, cpu_baseline=False)}
    if rank == 0:
        if moe is not None:
            line["moe"] = moe
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
