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
# MoE workload: the 16384-token grouped configuration on one GPU and its 65536-token variant (skewed router,
# experts sharded over the ranks, NCCL all-to-all dispatch / combine) when launched on several.
# ---------------------------------------------------------------------------------------------
def run_moe(args) -> int:
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": "the MoE workload has no bounded CPU sample in this harness; use the dense workload"}))
        return 0
    import torch.distributed as dist

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29531")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from b2g import _lib, ep, ep_peer, gguf_quant, ops

    E, H, I, TOPK, R_LORA = 256, 2048, 512, 8, 16
    t_total = args.tokens if args.tokens != 32768 else (16384 if world == 1 else 65536)
    skew = world > 1 or t_total == 65536
    t_local = t_total // world
    e_local = E // world
    lo = rank * e_local
    gen = torch.Generator(device=dev).manual_seed(SEED + 1 + rank)

    def packed(shape, seed):
        out = []
        g = torch.Generator(device=dev).manual_seed(seed)
        for s0 in range(0, shape[0], 32):
            n = min(32, shape[0] - s0)
            out.append(gguf_quant.quantize_q4_k(torch.randn(n, *shape[1:], generator=g, device=dev) * 0.02))
        return torch.cat(out, 0).reshape(-1)

    gate_p, up_p, down_p = packed((e_local, I, H), 100 + rank), packed((e_local, I, H), 200 + rank), packed((e_local, H, I), 300 + rank)
    lora = {"gate_up_a": (torch.randn(e_local, R_LORA, H, generator=gen, device=dev) / 16).bfloat16().requires_grad_(True),
            "gate_up_b": (torch.randn(e_local, 2 * I, R_LORA, generator=gen, device=dev) * 0.01).bfloat16().requires_grad_(True),
            "down_a": (torch.randn(e_local, R_LORA, I, generator=gen, device=dev) / 16).bfloat16().requires_grad_(True),
            "down_b": (torch.randn(e_local, H, R_LORA, generator=gen, device=dev) * 0.01).bfloat16().requires_grad_(True)}
    hidden = torch.randn(t_local, H, generator=gen, device=dev).bfloat16()
    g_out = torch.randn(t_local, H, generator=gen, device=dev).bfloat16()
    logits = torch.randn(t_local, E, generator=gen, device=dev)
    if skew:
        bias = torch.randn(E, generator=torch.Generator(device=dev).manual_seed(SEED + 4), device=dev) * 0.5   # same on every rank
        logits = logits + bias

    use_peer = world > 1 and args.ep == "peer"
    xchg = ep_peer.PeerExchange(t_local * TOPK, H, E, device=dev) if use_peer else None

    def step():
        h = hidden.detach().requires_grad_(True)
        for v in lora.values():
            v.grad = None
        idx = ops.router_topk(logits, TOPK, None, False)
        wts = torch.softmax(logits.gather(1, idx), dim=-1)
        if use_peer:
            out = ep_peer.peer_moe_layer(xchg, h, idx, wts, gate_p, up_p, down_p, Q4_K, I, lora, SCALING)
        else:
            out = ep.cuda_moe_layer(h, idx, wts, gate_p, up_p, down_p, Q4_K, I, E, lora, SCALING)
        out.backward(g_out)
        return out, h.grad

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(max(3, args.warmup)):
        step()
    barrier()
    ops.check_status()
    _lib.COUNT_LAUNCHES, _lib.LAUNCHES = True, 0
    barrier()
    sampler.begin()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    torch.cuda.profiler.start()                   # `ncu --profile-from-start off` then sees only the timed steps (all threads)
    for _ in range(args.steps):
        step()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    e1.record()
    barrier()
    sampler.end()
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    launches = _lib.LAUNCHES
    _lib.COUNT_LAUNCHES = False
    if world == 1:
        sampler.extend(step, torch.cuda.synchronize)        # (a multi-rank step holds collectives: never run it on one rank alone)
    clocks = sampler.stop() if rank == 0 else {}
    ops.check_status()
    if rank == 0:
        peaks, peak_src = load_peaks()
        ms_step = float(ms) / args.steps
        rows = t_total * TOPK
        flops = 4.0 * rows * 3 * H * I + 6.0 * rows * R_LORA * ((H + 2 * I) + (I + H))
        peak_tf = float(peaks.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]))
        print(json.dumps({
            "metric": "quantized MoE (grouped Q4_K experts + LoRA) fwd+bwd tokens/s", "value": t_total / (ms_step * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong" if world > 1 or t_total == 65536 else "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "grouped MoE Q4_K LoRA, 256 experts top-8, hidden 2048, intermediate 512 (configuration %d of the benchmark specification)" % (4 if skew else 2),
                       "tokens_total": t_total, "experts_per_gpu": e_local, "skewed_router": skew,
                       "parallelism": (f"ep{world} (experts sharded, " + ("peer-store dispatch/combine over NVLink)" if use_peer else "NCCL all-to-all dispatch/combine)"))
                       if world > 1 else "1 GPU",
                       "l2": "routed rows 2 GiB, larger than L2"},
            "step_tflops": flops / (ms_step * 1e-3) / 1e12, "step_frac_of_tensor_peak_all_gpus": flops / (ms_step * 1e-3) / 1e12 / (peak_tf * world),
            "peak_source": peak_src, "clocks": clocks, "gpu_launches": launches}))
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
    ap.add_argument("--ep", default="peer", choices=["peer", "nccl"],
                    help="MoE workload at N>1: row exchange by peer stores over NVLink (default) or by NCCL all-to-all")
    ap.add_argument("--workload", default="dense", choices=["dense", "moe", "formats", "fixed", "lmhead"],
                    help="dense: the Q4_K attention-shape linears (default, replicas at N>1); moe: grouped Q4_K experts, expert-parallel at N>1; formats / fixed / lmhead: single-GPU side measurements (see run_side)")
    args = ap.parse_args()
    if args.workload == "moe":
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
                    # dram__bytes_read + dram__bytes_write of this kernel: 161.3 MB per launch in an ncu capture at M=16384;
                    # the traffic is activations in and out (the packed weight stays in L2), so it scales with M
                    "traffic": 161.3e6 * m / 16384, "traffic_unit": "bytes/launch"}
        line = {"metric": "quantized LoRA-linear fwd+bwd tokens/s", "value": value, "unit": "tokens/s", "n_gpus": world,
                "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_step, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config,
                "step_tflops": world * flops / (ms_step * 1e-3) / 1e12,
                "step_frac_of_tensor_peak": flops / (ms_step * 1e-3) / 1e12 / peak_tf,
                "roofline": roof, "clocks": clocks, "gpu_launches": launches,
                "e2e": {"value": world * m / (ms_e2e / e2e_steps * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                        "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e / e2e_steps}}
        if world == 1 and not args.no_cpu_baseline:
            res = run_cpu(3, 1, budget_s=24.0, m_full=m)
            line["cpu_baseline"] = {"value": res["tokens_per_s"], "unit": "tokens/s", "cores": res["cores"], "kind": "port", "sample": res["sample"]}
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
