#!/usr/bin/env python
"""Benchmark of the MoE expert-layer hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--tokens T] [--config cfg3|cfg2] [--impl reference]

One "step" is one pass of a MoE layer over a batch of T tokens: route -> bucket -> gather ->
grouped gate/up + SwiGLU -> grouped down -> weighted combine (+ shared expert).  The default
workload is the DeepSeek-V3-shape layer (hidden 7168, intermediate 2048, 256 routed experts + 1
shared, top-8, group-limited sigmoid routing, FP8-e4m3 weights with 128x128 fp32 block scales,
bf16 activations); `--config cfg2` is the Qwen3-30B-A3B-shape layer (hidden 2048, intermediate
768, 128 experts, top-8, softmax routing, bf16 weights, Zipf(1.1) expert load).  Weights are random
(seeded, generated on the device), activations synthetic ~N(0,1).

Prints ONE JSON line.  `value` is tokens/s with inputs and outputs resident in HBM; `e2e` is the
same pass through the host-buffer entry point of the C ABI (pinned host -> device copy of the
activations and device -> host read of the result inside the timed region).  `check` compares the
routing of the whole timed batch and the outputs of a few of its tokens with the CPU oracle,
outside the timed region.  `--impl reference` times the CPU restatement of the reference's torch
expert path on the host cores on a bounded sample of the same workload.

Timing: after at least a second of untimed passes (so the GPU is in its sustained power state)
the block of K steps is timed repeatedly until half a second is covered; `ms_per_step` is the
median block, `blocks_ms` lists them all; SM clock and throttle reasons are sampled every 10 ms
DURING those blocks, and the per-stage profile is taken back to back right behind them.
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

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "expert-kit_b200"))

import torch  # noqa: E402

UNIT = "tokens/s"
FALLBACK_HBM_GBS = 6650.0
FALLBACK_TFLOPS = 1590.0
SEED = 3000

# DRAM traffic of the dominant kernel per expert slot that received rows, from ncu captures of a
# profiler-sized case (dram__bytes_read.sum + dram__bytes_write.sum per launch / active slots).  Keyed by
# (kernel, tile layout version): a library whose layout differs from the captured one reports null.
NCU_TRAFFIC = {
    ("ffn_tc_kernel<fp8, gate/up + SwiGLU>", 5): {
        "bytes_per_active_slot": 976.81e6 / 33,
        "source": "profiles/ffn_tc_fp8_cfg3_32experts_T32.md (33 slots, T=32: 973.33 MB read + 3.48 MB written)"},
}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            j = json.load(open(p))
            return dict(hbm=float(j["hbm_gbs"]), tf=float(j["bf16_tflops"]),
                        tf_sus=float(j.get("bf16_tflops_sustained", j["bf16_tflops"])), src="measured")
        except Exception:
            pass
    return dict(hbm=FALLBACK_HBM_GBS, tf=FALLBACK_TFLOPS, tf_sus=1400.0, src="fallback")


# ---- clocks ---------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock, power and throttle reasons of one GPU every 10 ms through NVML (reading
    only; nothing is ever set), with a host timestamp per sample, so that the samples falling
    inside a timed window can be picked out afterwards.  An `nvidia-smi -lms` child is the
    fallback when the NVML binding is missing (then the whole run is summarised)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int, period_s: float = 0.01):
        self.samples = []          # (t, sm_mhz, reasons bitmask, watts)
        self.max_mhz = None
        self.p = None
        self._stop = threading.Event()
        self._thread = None
        self.names = {}
        if os.environ.get("EK_BENCH_NO_CLOCKS"):
            return
        try:
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = gpu_index
            if visible:
                parts = visible.split(",")
                if gpu_index < len(parts) and parts[gpu_index].strip().isdigit():
                    phys = int(parts[gpu_index])
            h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
            self.names = {"hw_slowdown": getattr(pynvml, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
                          "hw_thermal_slowdown": getattr(pynvml, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
                          "sw_thermal_slowdown": getattr(pynvml, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
                          "sw_power_cap": getattr(pynvml, "nvmlClocksThrottleReasonSwPowerCap", 0x4)}

            def loop():
                while not self._stop.is_set():
                    try:
                        mhz = float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM))
                        r = int(pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(h))
                        try:
                            w = pynvml.nvmlDeviceGetPowerUsage(h) / 1000.0
                        except Exception:
                            w = None
                        self.samples.append((time.perf_counter(), mhz, r, w))
                    except Exception:
                        pass
                    self._stop.wait(period_s)

            self._thread = threading.Thread(target=loop, daemon=True)
            self._thread.start()
            return
        except Exception:
            self._thread = None
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                       "-i", str(gpu_index), "-lms", "100"], stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.p = None

    def window(self, t0: float, t1: float):
        """Summary of the samples taken between two host timestamps (NVML path)."""
        if self._thread is None:
            return None
        s = [x for x in self.samples if t0 <= x[0] <= t1]
        if not s:
            return None
        reasons = sorted(n for n, bit in self.names.items() if any(x[2] & bit for x in s))
        watts = [x[3] for x in s if x[3] is not None]
        return {"sm_mhz": statistics.median(x[1] for x in s), "sm_mhz_min": min(x[1] for x in s),
                "sm_max_mhz": self.max_mhz, "reasons": reasons, "samples": len(s),
                "power_w": statistics.median(watts) if watts else None,
                "source": "nvml, 10 ms period, samples inside the timed blocks only"}

    def stop(self):
        if self._thread is not None:
            self._stop.set()
            self._thread.join(timeout=2)
            return None
        if self.p is None:
            return None
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except Exception:
            self.p.kill()
        self.f.flush()
        self.f.seek(0)
        sm, mx, reasons = [], [], set()
        for line in self.f.read().splitlines():
            c = [x.strip() for x in line.split(",")]
            if len(c) < 9:
                continue
            try:
                sm.append(float(c[1]))
                mx.append(float(c[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), c[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        try:
            os.unlink(self.f.name)
        except OSError:
            pass
        if not sm:
            return None
        busy = [v for v in sm if v > 0.5 * max(sm)]
        return {"sm_mhz": statistics.median(busy or sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm), "source": "nvidia-smi, 100 ms period, whole run (NVML binding missing)"}


# ---- workloads --------------------------------------------------------------------------------
def shape_of(name: str):
    from ek_b200 import synth
    return {"cfg3": synth.DSV3, "cfg2": synth.QWEN3}[name]


def compute_dtype(S) -> str:
    """Operand type of the tensor-core contractions (fp32 accumulation): quantised weights are converted
    exactly to f16 and meet f16 activations; bf16 weights meet bf16 activations.  Inputs and outputs
    of the layer are bf16 either way."""
    return "f16" if S.quant != 0 else "bf16"


def metric_of(cfg_name: str) -> str:
    return {"cfg3": "MoE expert-layer tokens/s (DSV3 FP8-W/bf16-A)",
            "cfg2": "MoE expert-layer tokens/s (Qwen3-30B-A3B shape, bf16 W/A)"}[cfg_name]


def algorithmic(S, T: int, active: int, rows_routed: int, n_exp: int, T_shared: int):
    """Algorithmic bytes and flops of one layer pass and of its gate/up launch.  `active` = routed
    experts that received a row, `rows_routed` = their rows, `T_shared` = tokens the shared expert
    sees on this GPU."""
    H, I = S.hidden, S.intermediate
    bw = 2 if S.quant == 0 else 1
    nb = (I // 128) * (H // 128)
    sc = 0 if S.quant == 0 else 12 * nb
    slots = active + (S.n_shared if T_shared > 0 else 0)
    rows = rows_routed + S.n_shared * T_shared
    bytes_layer = slots * (3 * H * I * bw + sc) + 2 * H * n_exp + 4 * T * H
    flops_layer = 2 * T * H * n_exp + 6 * H * I * rows
    gu_bytes = slots * (2 * H * I * bw + (0 if S.quant == 0 else 8 * nb)) + rows * H * 2 + rows * I * 2
    gu_flops = 4 * H * I * rows
    return bytes_layer, flops_layer, gu_bytes, gu_flops


def workload_config(S, cfg_name: str, T: int, n_gpus: int, n_exp: int, layers: int = 1):
    if cfg_name == "cfg3":
        w = "cfg3 DeepSeek-V3-shape MoE layer, W8A16 (fp8 e4m3 + 128x128 fp32 block scales)"
        routing = "sigmoid, 8 groups, top-4 groups, renormalised, x2.5"
    else:
        w = "cfg2 Qwen3-30B-A3B-shape MoE layer, bf16 weights, Zipf(1.1)-skewed expert load"
        routing = "softmax, renormalised top-8, bf16 routing weights"
    w += f", global batch T={T} tokens"
    if layers > 1:
        w += f" x {layers} layers per step (cfg5-style expert stack)"
    if n_exp != S.n_experts:
        w += f" [REDUCED to {n_exp} routed experts: profiling case, not the benchmark]"
    weights_gb = (n_exp + S.n_shared) * 3 * S.hidden * S.intermediate * (2 if S.quant == 0 else 1) / 1e9
    return {"workload": w, "hidden": S.hidden, "intermediate": S.intermediate, "experts": n_exp,
            "shared_experts": S.n_shared, "top_k": S.top_k, "routing": routing, "global_tokens": T,
            "tokens_per_gpu": T // n_gpus,
            "parallelism": "single GPU" if n_gpus == 1 else
            f"ep{n_gpus}: {n_exp // n_gpus} routed experts per GPU, shared expert and router replicated; tokens "
            "stored into every rank's memory and fp32 partial sums loaded from every rank's memory by the library's "
            "own kernels over NVLink (CUDA IPC mappings; NCCL all-gather + reduce-scatter if the mappings cannot be "
            "made), NCCL all-to-all dispatch/combine above 2048 tokens; global batch fixed (strong scaling)",
            "l2": f"weights streamed per step ({weights_gb:.1f} GB per layer) exceed the 126 MB L2; four input batches "
                  "used in rotation; no flush needed"}


def oracle_config(S, n_exp: int):
    """The oracle's description of the same layer (checker only)."""
    from oracle import ek_oracle as O
    return O.MoEConfig(hidden=S.hidden, intermediate=S.intermediate, n_experts=n_exp, top_k=S.top_k,
                       scoring=S.scoring, n_group=S.n_group, topk_group=S.topk_group, norm_topk_prob=True,
                       routed_scaling=S.routed_scaling, n_shared=S.n_shared, bf16_combine=S.bf16_combine,
                       quant={0: "bf16", 1: "fp8", 2: "int8"}[S.quant])


def oracle_check(S, n_exp: int, dev, x_dev, y_dev, routing, n_tokens: int = 4):
    """Outside the timed region: routing of ALL tokens of one timed batch and the outputs of a few
    of them against the CPU oracle.  `routing` holds the host tensors the backend reported (ids,
    weights and, at N = 1, logits / counts / offsets / perm).  The experts the sampled tokens use
    are generated again from their seeds (on any rank), copied to the host and evaluated there."""
    from ek_b200 import synth
    from oracle import sampled as OS
    cfg = oracle_config(S, n_exp)
    wg, _ = synth.make_router(S, dev, SEED, 0, n_exp)
    bias = torch.zeros(n_exp) if S.scoring == 1 else None
    xc = x_dev.cpu()
    r = OS.check_routing(cfg, xc, wg.cpu(), bias, routing)

    def fetch(e):
        return OS.expert_from_named(synth.make_expert(S, dev, SEED, 0, e))

    o = OS.check_outputs_sampled(cfg, xc, y_dev.cpu(), r, fetch, n_tokens)
    mean_bound = 1e-3 * max(1.0, o.get("mean_ref", 0.0) / 0.1)
    ok = (r.get("exact_given_logits", True) and r.get("bucket_exact", True) and r.get("differ_unexplained", 0) == 0
          and r.get("differ_not_a_tie_swap", 0) == 0 and r["ids_differ"] <= max(1, r["tokens"] // 100)
          and o.get("tokens_checked", 0) > 0 and o["max_rel"] <= 2e-2 and o["mean_abs"] <= mean_bound)
    out = {"ok": bool(ok), "ids_equal": r["ids_equal"], "tokens_routed": r["tokens"], "ids_differ": r["ids_differ"],
           "exact_given_logits": r.get("exact_given_logits"), "bucket_exact": r.get("bucket_exact"),
           "differ_unexplained": r.get("differ_unexplained"), "weights_max_rel": r.get("weights_max_rel"),
           "tokens_checked": o.get("tokens_checked", 0), "experts_evaluated": o.get("experts_evaluated"),
           "max_rel": o.get("max_rel"), "mean_abs": o.get("mean_abs"), "mean_ref": o.get("mean_ref"),
           "bounds": {"max_rel": 2e-2, "mean_abs": mean_bound},
           "oracle": "CPU restatement of the reference's torch expert path (oracle/ek_oracle.py), outside the timed region"}
    return out


# ---- timing helpers -----------------------------------------------------------------------------
def condition(step, seconds: float, sync):
    """Untimed passes for at least `seconds`: warm-up and the GPU's sustained power state."""
    t_end = time.perf_counter() + seconds
    n = 0
    while time.perf_counter() < t_end:
        for _ in range(8):
            step(n)
            n += 1
        sync()
    return n


def timed_blocks(step, K: int, sync, reduce_max=None, min_seconds: float = 0.5, min_blocks: int = 3,
                 max_blocks: int = 400):
    """Times the block of exactly K steps repeatedly (CUDA events on the launching stream, a
    synchronisation on both sides of every block).  Returns (per-block ms list, t0, t1)."""
    blocks = []
    sync()
    t0 = time.perf_counter()
    total = 0.0
    while len(blocks) < min_blocks or (total < min_seconds * 1e3 and len(blocks) < max_blocks):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(K):
            step(i)
        e1.record()
        sync()
        ms = e0.elapsed_time(e1)
        if reduce_max is not None:
            ms = reduce_max(ms)
        blocks.append(ms)
        total += ms
    return blocks, t0, time.perf_counter()


def stage_profile(be, step, sync, n_pass: int = 48):
    """Mean per-stage device time over `n_pass` passes issued back to back (one synchronisation at
    the end: the GPU stays in the state the timed blocks ran in)."""
    be.stage_timing(True)
    for i in range(n_pass):
        step(i)
    sync()
    st = be.stage_times()
    be.stage_timing(False)
    return st


# ---- CPU baseline (oracle port of the reference's torch expert path) -------------------------
def cpu_baseline(S, T: int, n_exp: int, budget_s: float = 15.0, seed: int = 5, scan: bool = True):
    """Scope (ii): route + bucket + per-expert bf16 FFN loop + weighted combine + shared expert on
    the host cores, on a sample of distinct experts (weights dequantised once at load, as the
    reference's load_module would hold them), the expert loop scaled to the number of experts the
    routing actually activates.  Scope (i), with `scan`: the expert FFN alone over a batch scan, the
    measurement ek-benchmark makes (ek-benchmark/src/bench.rs:75-131)."""
    from oracle import ek_oracle as O
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    cfg = oracle_config(S, n_exp)
    H, I, K = S.hidden, S.intermediate, S.top_k
    g = torch.Generator().manual_seed(seed)
    wg = (torch.randn(n_exp, H, generator=g) * 0.02).to(torch.bfloat16)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    t0 = time.perf_counter()
    logits, ids, w = O.route(cfg, x, wg, torch.zeros(n_exp) if S.scoring == 1 else None)
    counts, offsets, perm = O.bucket(ids, n_exp)
    t_route = time.perf_counter() - t0
    active = int((counts > 0).sum())
    n_sample = 8
    experts = [[torch.randn(s, generator=g).mul_(0.02).to(torch.bfloat16) for s in ((I, H), (I, H), (H, I))]
               for _ in range(n_sample)]
    rows_per = max(1, round(T * K / max(active, 1)))
    xe = x[:rows_per] if rows_per <= T else x.repeat((rows_per + T - 1) // T, 1)[:rows_per]
    O.expert_ffn(xe, *experts[0])   # warm-up
    n_calls, t_ffn = 0, 0.0
    while t_ffn < budget_s * 0.5 and n_calls < 16384:    # about half the budget in the expert loop
        ws = experts[n_calls % n_sample]
        t0 = time.perf_counter()
        O.expert_ffn(xe, *ws)
        t_ffn += time.perf_counter() - t0
        n_calls += 1
    per_call = t_ffn / n_calls
    t_shared = 0.0
    if S.n_shared > 0:
        t0 = time.perf_counter()
        O.expert_ffn(x, *experts[0])    # shared expert: all T rows
        t_shared = time.perf_counter() - t0
    outs = torch.zeros(T, K, H, dtype=torch.bfloat16)
    t0 = time.perf_counter()
    O.combine(outs, w, S.bf16_combine)
    t_comb = time.perf_counter() - t0
    step = t_route + active * per_call + t_shared + t_comb
    out = dict(value=T / step, unit=UNIT, cores=cores, kind="port",
               sample=(f"router+bucket, {n_calls} single-expert FFN calls of {rows_per} rows on {n_sample} distinct "
                       f"bf16 experts (scaled to the {active} active experts), shared expert, combine; T={T}; "
                       f"{per_call * 1e3:.2f} ms per expert call"),
               ms_per_step=step * 1e3)
    if scan:
        # scope (i): forward of one expert only, per batch size, mean over a few calls on distinct experts
        rows = {}
        for b in (1, 8, 32, 256):
            xb = torch.randn(b, H, generator=g).to(torch.bfloat16)
            O.expert_ffn(xb, *experts[0])
            ts = []
            while sum(ts) < 0.5 and len(ts) < 2048:          # half a second per batch size
                t0 = time.perf_counter()
                O.expert_ffn(xb, *experts[len(ts) % n_sample])
                ts.append(time.perf_counter() - t0)
            m = statistics.mean(ts)
            rows[str(b)] = {"us_per_call": m * 1e6, "rows_per_s": b / m}
        out["expert_ffn_only"] = {"scope": "one expert's forward alone per batch size, as ek-benchmark's batch scan",
                                  "batch": rows}
    return out


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    S = shape_of(args.config)
    T = args.tokens
    vals = []
    base = None
    for i in range(args.warmup + args.steps):
        base = cpu_baseline(S, T, args.experts or S.n_experts,
                            budget_s=max(2.0, 30.0 / max(1, args.warmup + args.steps)), seed=5 + i, scan=False)
        if i >= args.warmup:
            vals.append(base)
    v = statistics.mean(b["value"] for b in vals)
    ms = statistics.mean(b["ms_per_step"] for b in vals)
    line = {"impl": "reference", "metric": metric_of(args.config), "value": v, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(S, args.config, T, args.gpus, args.experts or S.n_experts),
            "cpu_baseline": {"value": v, "unit": UNIT, "cores": base["cores"], "kind": "port", "sample": base["sample"]},
            "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def roofline_of(S, stage, gu_bytes, gu_flops, active_slots, P, layout_version, where=""):
    gu_s = max(stage["gateup"], 1e-6) / 1e3
    t_hbm, t_tc = gu_bytes / (P["hbm"] * 1e9), gu_flops / (P["tf"] * 1e12)
    if t_hbm >= t_tc:
        roof = {"bound": "hbm", "achieved": gu_bytes / gu_s / 1e9, "peak": P["hbm"], "unit": "GB/s"}
    else:
        roof = {"bound": "tensor", "achieved": gu_flops / gu_s / 1e12, "peak": P["tf"], "unit": "TFLOP/s"}
    roof["frac"] = roof["achieved"] / roof["peak"]
    kname = {0: "ffn_tc_kernel<bf16, gate/up + SwiGLU>", 1: "ffn_tc_kernel<fp8, gate/up + SwiGLU>",
             2: "ffn_tc_kernel<int8, gate/up + SwiGLU>"}[S.quant]
    cap = NCU_TRAFFIC.get((kname, layout_version))
    roof["traffic"] = int(active_slots * cap["bytes_per_active_slot"]) if cap else None
    roof["traffic_source"] = (cap["source"] + ", scaled by the active expert slots") if cap else \
        "no ncu capture of this kernel / tile layout version on record"
    roof["kernel"] = kname + where
    roof["peak_source"] = P["src"]
    roof["launch_ms"] = stage["gateup"]
    roof["algorithmic_bytes"] = gu_bytes
    roof["algorithmic_flops"] = gu_flops
    return roof


def layer_run(S, be, dev, T, n_exp, steps, sync, u, want_stage=True, cond_s=0.3, min_s=0.2):
    """tokens/s and layer-roofline fraction of one batch size on an existing backend (sweep rows)."""
    from ek_b200 import synth
    xs = [synth.make_tokens(S, dev, SEED + 11 + i, T, u) for i in range(4)]
    y = torch.empty(T, S.hidden, dtype=torch.bfloat16, device=dev)

    def step(i):
        be.moe_forward_fused_async(0, xs[i % 4], y)

    condition(step, cond_s, sync)
    blocks, _, _ = timed_blocks(step, steps, sync, min_seconds=min_s)
    ms_step = statistics.median(blocks) / steps
    stage = stage_profile(be, step, sync, 24) if want_stage else None
    counts = be.expert_counts(0)
    a = int((counts > 0).sum())
    P = peaks()
    bl, fl, _, _ = algorithmic(S, T, a, int(counts.sum()), n_exp, T)
    rs = max(bl / (P["hbm"] * 1e9), fl / (P["tf_sus"] * 1e12))
    out = {"tokens_per_s": T / (ms_step / 1e3), "ms_per_step": ms_step, "active_experts": a,
           "layer_roofline_frac": (rs * 1e3) / ms_step,
           "bound": "hbm" if bl / (P["hbm"] * 1e9) >= fl / (P["tf_sus"] * 1e12) else "tensor"}
    if stage:
        out["stage_ms"] = {k_: round(v, 4) for k_, v in stage.items()}
    return out


# ---- N > 1: expert parallel -----------------------------------------------------------------------
def main_ep(args, rank: int, world: int, local: int):
    """The layer's experts are sharded over the ranks (expert parallel); the global batch of
    --tokens tokens is split evenly over the ranks."""
    import datetime
    import torch.distributed as dist
    import ek_b200
    from ek_b200 import synth, _lib as L
    # NCCL's own log must not reach stdout (one JSON line); a level the caller set is kept
    if "NCCL_DEBUG" in os.environ and "NCCL_DEBUG_FILE" not in os.environ:
        os.environ["NCCL_DEBUG_FILE"] = "/dev/stderr"
    # a short collective timeout: a rank that fails must not keep the others (and the GPUs) waiting
    dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=120))
    S = shape_of(args.config)
    T = args.tokens
    if T % world:
        raise SystemExit("--tokens must be divisible by the number of GPUs")
    Tl = T // world
    n_exp = args.experts or S.n_experts
    NL = args.layers
    dev = torch.device("cuda", local)
    be, dirs = synth.build_backend(S, max(T, 256), SEED, dev, ep_rank=rank, ep_size=world, n_layers=NL, n_experts=n_exp)
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(stream)
    be.set_stream(stream.cuda_stream)
    moe_one = ek_b200.ExpertParallelMoE(ek_b200.BackendStages(be), mode=args.ep_mode)

    def forward(x):
        y = None
        for layer in range(NL):
            y = moe_one.forward(layer, x)
        return y

    # rank r's tokens: rows [r*Tl, (r+1)*Tl) of the global batch i
    xs = [synth.make_tokens(S, dev, SEED + 11 + i, T, dirs[0])[rank * Tl:(rank + 1) * Tl].contiguous() for i in range(4)]

    def step(i):
        forward(xs[i % 4])

    def sync():
        be.sync()
        torch.cuda.synchronize()

    def reduce_max(ms):
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for i in range(max(args.warmup, 3)):
        step(i)
    sync()
    # conditioning: the same number of passes on every rank (forward is collective)
    n_cond = int(1000.0 / 0.4 / NL) if NL < 8 else 20
    for i in range(n_cond):
        step(i)
    sync()
    sampler = ClockSampler(local) if rank == 0 else None
    dist.barrier()
    torch.cuda.synchronize()
    l0 = be.kernel_launches()
    # the number of blocks must be the same on every rank: fixed from a first block's duration
    first, _, _ = timed_blocks(step, args.steps, sync, reduce_max, min_seconds=0.0, min_blocks=1)
    n_blocks = max(3, min(200, int(500.0 / max(first[0], 1e-3)) + 1))
    dist.barrier()
    l0 = be.kernel_launches()
    blocks, t0, t1 = timed_blocks(step, args.steps, sync, reduce_max, min_seconds=0.0, min_blocks=n_blocks, max_blocks=n_blocks)
    launches = (be.kernel_launches() - l0) // n_blocks
    clocks = sampler.window(t0, t1) if sampler else None
    ms_step = statistics.median(blocks) / args.steps
    value = T / (ms_step / 1e3)
    stage = stage_profile(be, step, sync, 48 if NL == 1 else NL)
    if sampler:
        fb = sampler.stop()
        clocks = clocks or fb
    el = n_exp // world
    mine = be.expert_counts(0)[rank * el:(rank + 1) * el]     # peer/gather: this rank routed the whole global batch
    if moe_one.last_counts_all is not None:
        mine = moe_one.last_counts_all[:, rank * el:(rank + 1) * el].sum(0)
    active = int((mine > 0).sum())
    P = peaks()
    bytes_rank, flops_rank, gu_bytes, gu_flops = algorithmic(S, Tl, active, int(mine.sum()), n_exp, Tl)
    roof = roofline_of(S, stage, gu_bytes, gu_flops, active + S.n_shared, P, L.EK_TILE_LAYOUT_VERSION,
                       " on rank 0's experts")
    roof_s = NL * max(bytes_rank / (P["hbm"] * 1e9), flops_rank / (P["tf_sus"] * 1e12))   # per step
    nvlink_bytes = (world - 1) * Tl * S.hidden * 2 + (world - 1) * Tl * S.hidden * 4
    layer = {"roofline_tokens_per_s": T / roof_s, "frac": roof_s * 1e3 / ms_step, "bound": "hbm",
             "layers": NL, "bytes_per_gpu_per_layer": bytes_rank, "flops_per_gpu_per_layer": flops_rank,
             "active_experts_rank0": active, "nvlink_bytes_per_gpu_per_layer": int(nvlink_bytes),
             "stage_ms_rank0": {k_: round(v, 4) for k_, v in stage.items()},
             "stage_sum_ms": round(sum(stage.values()), 4)}

    # end to end: host batch in, host result out, through the public Python API of this package
    xh = [x.cpu().pin_memory() for x in xs]
    yh = torch.empty(Tl, S.hidden, dtype=torch.bfloat16).pin_memory()
    xd = torch.empty(Tl, S.hidden, dtype=torch.bfloat16, device=dev)
    e2e_steps = max(3, min(args.steps, 10))

    def e2e_step(i):
        xd.copy_(xh[i % 4], non_blocking=True)
        y = forward(xd)
        yh.copy_(y, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    e2e_step(0)
    dist.barrier()
    torch.cuda.synchronize()
    e2e_blocks = []
    for _ in range(5):
        dist.barrier()
        t0 = time.perf_counter()
        for i in range(e2e_steps):
            e2e_step(i)
        torch.cuda.synchronize()
        e2e_blocks.append(reduce_max((time.perf_counter() - t0) * 1e3))
    e2e_ms = statistics.median(e2e_blocks) / e2e_steps
    e2e = {"value": T / (e2e_ms / 1e3), "unit": UNIT, "h2d_bytes_per_step": T * S.hidden * 2,
           "d2h_bytes_per_step": T * S.hidden * 2, "steps": e2e_steps, "ms_per_step": e2e_ms}

    # check of rank 0's slice of one timed batch against the oracle (every rank takes part in the pass)
    check = None
    if not args.no_check:
        y = moe_one.forward(0, xs[0])
        sync()
        routing = None
        if rank == 0:
            mode = moe_one.last_mode
            if mode in ("peer", "gather"):      # this rank routed all T tokens; its own are the first Tl
                ids, w = be.last_routing(T)
                routing = dict(ids=ids[:Tl], weights=w[:Tl])
            else:
                ids, w = be.last_routing(Tl)
                routing = dict(ids=ids, weights=w)
        dist.barrier()
        if rank == 0:
            try:
                check = oracle_check(S, n_exp, dev, xs[0], y, routing, 3)
                check["scheme"] = moe_one.last_mode
                check["note"] = "rank 0's tokens; their experts live on all ranks and were generated again from the seeds"
            except Exception as ex:   # noqa: BLE001
                check = {"ok": False, "error": repr(ex)}
    if rank == 0:
        line = {"metric": metric_of(args.config), "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": compute_dtype(S), "data": "synthetic",
                "config": workload_config(S, args.config, T, world, n_exp, NL),
                "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks, "roofline": roof,
                "layer_roofline": layer, "cpu_baseline": None, "check": check,
                "blocks_ms": [round(b / args.steps, 5) for b in blocks], "conditioning_passes": n_cond,
                "ms_x_mhz": (ms_step * clocks["sm_mhz"]) if clocks else None,
                "exchange": moe_one.last_mode}
        print(json.dumps(line))
    dist.barrier()
    moe_one.close()
    be.close()
    dist.barrier()
    dist.destroy_process_group()


# ---- N = 1 ----------------------------------------------------------------------------------------
def main_single(args, local: int):
    from ek_b200 import synth, _lib as L
    S = shape_of(args.config)
    T = args.tokens
    n_exp = args.experts or S.n_experts
    sweep = [int(t) for t in args.sweep.split(",") if t]
    if args.extras and not sweep:
        sweep = [1, 32, 1024, 4096] if args.config == "cfg3" else [1, 16, 64]
    dev = torch.device("cuda", local)
    # the continuous-batching stream: 2000 steps when asked for, a 300-step sample in the default run
    if args.stream == 0 and args.extras and args.config == "cfg3" and n_exp == S.n_experts:
        args.stream = 300
    T_max = max([T] + sweep + ([2400] if args.stream > 0 else []))
    be, dirs = synth.build_backend(S, T_max, SEED, dev, n_experts=n_exp)
    u = dirs[0]
    # the library launches on this stream, so torch's events bracket exactly its kernels
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(stream)
    be.set_stream(stream.cuda_stream)
    xs = [synth.make_tokens(S, dev, SEED + 11 + i, T, u) for i in range(4)]
    y = torch.empty(T, S.hidden, dtype=torch.bfloat16, device=dev)

    def step(i):
        be.moe_forward_fused_async(0, xs[i % 4], y)

    def sync():
        be.sync()
        torch.cuda.synchronize()

    for i in range(max(args.warmup, 3)):
        step(i)
    sync()
    sampler = ClockSampler(local)
    n_cond = 0 if args.quick else condition(step, 1.0, sync)
    l0 = be.kernel_launches()
    if args.quick:
        blocks, t0, t1 = timed_blocks(step, args.steps, sync, min_seconds=0.0, min_blocks=1, max_blocks=1)
    else:
        blocks, t0, t1 = timed_blocks(step, args.steps, sync)
    launches = (be.kernel_launches() - l0) // len(blocks)
    stage = stage_profile(be, step, sync, 4 if args.quick else 48)   # back to back with the timed blocks
    t2 = time.perf_counter()
    clocks = sampler.window(t0, t1)
    clocks_stage = sampler.window(t1, t2)
    ms_step = statistics.median(blocks) / args.steps
    value = T / (ms_step / 1e3)

    counts = be.expert_counts(0)
    active = int((counts > 0).sum())
    P = peaks()
    bytes_layer, flops_layer, gu_bytes, gu_flops = algorithmic(S, T, active, int(counts.sum()), n_exp, T)
    roof = roofline_of(S, stage, gu_bytes, gu_flops, active + S.n_shared, P, L.EK_TILE_LAYOUT_VERSION)
    if clocks_stage:
        roof["sm_mhz_during_stage_profile"] = clocks_stage["sm_mhz"]
    t_b, t_f = bytes_layer / (P["hbm"] * 1e9), flops_layer / (P["tf_sus"] * 1e12)
    layer_roof_s = max(t_b, t_f)
    layer = {"roofline_tokens_per_s": T / layer_roof_s, "frac": layer_roof_s * 1e3 / ms_step,
             "bound": "hbm" if t_b >= t_f else "tensor", "bytes": bytes_layer, "flops": flops_layer,
             "active_experts": active, "stage_ms": {k_: round(v, 4) for k_, v in stage.items()},
             "stage_sum_ms": round(sum(stage.values()), 4),
             "stage_sum_over_step": round(sum(stage.values()) / ms_step, 4)}

    # end to end through the host-buffer entry point of the C ABI
    xh = [x.cpu().pin_memory() for x in xs]
    yh = torch.empty(T, S.hidden, dtype=torch.bfloat16).pin_memory()
    e2e_steps = max(3, min(args.steps, 10))
    fused = be._lib.ek_moe_forward_fused

    def e2e_step(i):
        be._check(fused(be._h, 0, xh[i % 4].data_ptr(), T, yh.data_ptr(), None))

    for i in range(1 if args.quick else 3):
        e2e_step(i)
    e2e_blocks, tot = [], 0.0
    while len(e2e_blocks) < (1 if args.quick else 3) or (not args.quick and tot < 0.3 and len(e2e_blocks) < 200):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for i in range(e2e_steps):
            e2e_step(i)
        torch.cuda.synchronize()
        e2e_blocks.append(time.perf_counter() - t0)
        tot += e2e_blocks[-1]
    e2e_ms = statistics.median(e2e_blocks) / e2e_steps * 1e3
    e2e = {"value": T / (e2e_ms / 1e3), "unit": UNIT, "h2d_bytes_per_step": T * S.hidden * 2,
           "d2h_bytes_per_step": T * S.hidden * 2, "steps": e2e_steps, "ms_per_step": e2e_ms}

    check = None
    if not args.no_check:
        try:
            yc, art = be.moe_forward_fused(0, xs[0], debug=True)
            check = oracle_check(S, n_exp, dev, xs[0], yc, art, 4)
        except Exception as ex:   # noqa: BLE001
            check = {"ok": False, "error": repr(ex)}

    sweep_out = {}
    for Tn in sweep:
        sweep_out[str(Tn)] = layer_run(S, be, dev, Tn, n_exp, max(3, args.steps // 2), sync, u)

    worker_out = worker_path(args, S, be, dev, T, u) if args.worker_threads > 0 else None
    stream_out = stream_run(args, S, be, dev, n_exp) if args.stream > 0 else None
    be.close()
    del be
    torch.cuda.empty_cache()

    extra = {}
    if args.extras and args.config == "cfg3" and n_exp == S.n_experts:
        extra = run_extras(args, dev, sync)

    base = None
    if not args.no_cpu_baseline:
        b = cpu_baseline(S, T, n_exp)
        base = {k_: b[k_] for k_ in ("value", "unit", "cores", "kind", "sample", "expert_ffn_only") if k_ in b}
        base["scope"] = "route + bucket + expert FFNs + weighted combine + shared expert"
    fb = sampler.stop()
    line = {"metric": metric_of(args.config), "value": value, "unit": UNIT, "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": compute_dtype(S), "data": "synthetic",
            "config": workload_config(S, args.config, T, 1, n_exp),
            "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks or fb, "roofline": roof,
            "layer_roofline": layer, "cpu_baseline": base, "check": check,
            "blocks_ms": [round(b / args.steps, 5) for b in blocks], "conditioning_passes": n_cond,
            "ms_x_mhz": (ms_step * clocks["sm_mhz"]) if clocks else None}
    if sweep_out:
        line["sweep"] = sweep_out
    if stream_out:
        line["stream"] = stream_out
    if worker_out:
        line["worker_path"] = worker_out
    if extra:
        line["extra"] = extra
    print(json.dumps(line))


def run_extras(args, dev, sync_unused):
    """Configurations beside the headline one, recorded in the same line: the Qwen3-30B-A3B-shape
    layer (bf16 weights) at decode batch sizes, and the INT8 form of the headline layer on a reduced
    expert count."""
    from ek_b200 import synth
    out = {}
    for name, S, n_exp, Ts in (("cfg2_qwen3_bf16", synth.QWEN3, synth.QWEN3.n_experts, (1, 16, 64, 256)),):
        try:
            be, dirs = synth.build_backend(S, max(Ts), SEED, dev, n_experts=n_exp)
            stream = torch.cuda.current_stream(dev)
            be.set_stream(stream.cuda_stream)

            def sync():
                be.sync()
                torch.cuda.synchronize()
            rows = {}
            for Tn in Ts:
                rows[str(Tn)] = layer_run(S, be, dev, Tn, n_exp, max(3, args.steps // 2), sync, dirs[0])
            out[name] = {"config": workload_config(S, "cfg2", max(Ts), 1, n_exp)["workload"], "tokens": rows}
            be.close()
            del be
            torch.cuda.empty_cache()
        except Exception as ex:   # noqa: BLE001
            out[name] = {"error": repr(ex)}
    try:
        import copy
        S8 = copy.copy(synth.DSV3)
        S8.quant, S8.name = 2, "dsv3i8"
        n_exp = 64
        S8.n_group, S8.topk_group = 8, 4
        be, dirs = synth.build_backend(S8, 256, SEED, dev, n_experts=n_exp)
        be.set_stream(torch.cuda.current_stream(dev).cuda_stream)

        def sync8():
            be.sync()
            torch.cuda.synchronize()
        # 64 tokens on 64 experts load an expert like the headline's 256 tokens on 256 experts (8 rows each)
        rows = {str(Tn): layer_run(S8, be, dev, Tn, n_exp, max(3, args.steps // 2), sync8, None) for Tn in (64, 256)}
        out["int8_dsv3_shape_64_experts"] = {"config": "DeepSeek-V3 layer dimensions, INT8 weights + block scales, 64 routed "
                                             "experts + 1 shared (2.9 GB of weights)", "tokens": rows}
        be.close()
        del be
        torch.cuda.empty_cache()
    except Exception as ex:   # noqa: BLE001
        out["int8_dsv3_shape_64_experts"] = {"error": repr(ex)}
    try:
        out["registration_fp8_host_tensors"] = registration_run(dev)
    except Exception as ex:   # noqa: BLE001
        out["registration_fp8_host_tensors"] = {"error": repr(ex)}
    return out


def registration_run(dev, n_exp: int = 64):
    """Loader throughput: `n_exp` DeepSeek-V3-shape fp8 experts (44 MB each) registered from pageable
    host memory by 1, 8 and 64 threads at once - the reference loads 64 experts concurrently
    (ek-computation/src/worker/state.rs:178-197)."""
    from concurrent.futures import ThreadPoolExecutor
    from ek_b200 import synth, Backend
    S = synth.DSV3
    be = Backend(S.backend_config(256, dev.index, 0, 1, 1, n_exp))
    host = [{k_: v.cpu() for k_, v in synth.make_expert(S, dev, SEED + 7, 0, e).items()} for e in range(8)]
    nbytes = sum(v.numel() * v.element_size() for v in host[0].values())
    res = {}
    for nthr in (64, 1, 8, 64):        # the first round is untimed: it allocates the loader lanes' staging
        for e in range(n_exp):
            be.evict(be.expert_id(0, e))
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        with ThreadPoolExecutor(nthr) as ex:
            list(ex.map(lambda e: be.register_expert(be.expert_id(0, e), host[e % 8]), range(n_exp)))
        dt = time.perf_counter() - t0
        res[str(nthr)] = {"experts_per_s": n_exp / dt, "GB_per_s": n_exp * nbytes / dt / 1e9}
    be.close()
    del be
    torch.cuda.empty_cache()
    return {"experts": n_exp, "bytes_per_expert": nbytes, "source": "pageable host tensors", "threads": res}


def worker_path(args, S, be, dev, T, u):
    """The reference's own seam: one single-expert call per distinct expert of the batch, issued from
    N host threads as its worker does per RPC (host buffers in and out); the library serves whatever
    is queued as one grouped launch."""
    from ek_b200 import synth
    xw = synth.make_tokens(S, dev, SEED + 77, T, u)
    _, art = be.moe_forward_fused(0, xw, debug=True)
    ids = art["ids"].cpu()
    xh = xw.cpu()
    per_expert = {}
    for e in torch.unique(ids).tolist():
        rows = (ids == e).any(dim=1).nonzero().flatten()
        xe = xh[rows].contiguous().pin_memory()
        # (id, x pointer, rows, y pointer) prepared once: the timed loop is the C call alone, so
        # the interpreter lock is free while a call waits and the threads really overlap
        per_expert[e] = (be.expert_id(0, e).encode(), xe, xe.shape[0], torch.empty_like(xe).pin_memory())
    experts = sorted(per_expert)
    fwd, handle = be._lib.ek_expert_forward, be._h
    nthr = args.worker_threads
    c0, b0 = be.worker_batch_stats()
    reps = max(3, args.steps // 4)
    go = threading.Barrier(nthr + 1)

    def run(tid):
        mine = experts[tid::nthr]
        for _ in range(reps + 1):
            go.wait()
            for e in mine:
                eid, xe, n_e, ye = per_expert[e]
                if fwd(handle, eid, xe.data_ptr(), n_e, ye.data_ptr()) != 0:
                    raise RuntimeError(be._lib.ek_last_error(handle).decode())
            go.wait()

    ths = [threading.Thread(target=run, args=(i,)) for i in range(nthr)]
    for t_ in ths:
        t_.start()
    go.wait(); go.wait()                      # warm-up round
    t0 = time.perf_counter()
    for _ in range(reps):
        go.wait(); go.wait()
    dt = (time.perf_counter() - t0) / reps
    for t_ in ths:
        t_.join()
    c1, b1 = be.worker_batch_stats()
    return {"threads": nthr, "calls_per_step": len(experts), "ms_per_step": dt * 1e3,
            "tokens_per_s": T / dt, "calls": c1 - c0, "grouped_passes": b1 - b0,
            "note": "single-expert calls with host buffers from N threads (wall clock, expert FFN only)"}


def stream_run(args, S, be, dev, n_exp):
    """Continuous-batching stream through the controller-level entry point: per step a Poisson(96)
    number of decode tokens plus, every 10th step, one prefill chunk of 512-2048 tokens; Zipf(1.2)
    expert load with the hot set rotated every 200 steps; every expert receives at least one row."""
    K = S.top_k
    gs = torch.Generator().manual_seed(4)
    gd = torch.Generator(device=dev).manual_seed(5)
    zipf_p = (torch.arange(1, n_exp + 1, dtype=torch.float32, device=dev) ** -1.2)

    def zipf_ids_dev(Ts, rot):
        ids = torch.multinomial(zipf_p.expand(Ts, n_exp), K, replacement=False, generator=gd)
        ids = (ids + rot) % n_exp
        for _ in range(4):
            present = torch.zeros(n_exp, dtype=torch.bool, device=dev)
            present[ids.reshape(-1)] = True
            missing = (~present).nonzero().flatten()
            if missing.numel() == 0:
                break
            pos = torch.arange(missing.numel(), device=dev)
            ids[pos % Ts, pos // Ts] = missing          # slot 0 of every token first, then slot 1, ...
        return ids.to(torch.int32).contiguous()

    steps = []
    for i in range(args.stream):
        Ts = int(torch.poisson(torch.tensor(96.0), generator=gs).item()) + 1
        if i % 10 == 9:
            Ts += int(torch.randint(512, 2049, (1,), generator=gs).item())
        Ts = max(Ts, n_exp // K + 1)
        steps.append((Ts, zipf_ids_dev(Ts, (i // 200) * 37)))
    Tmax = max(t for t, _ in steps)
    if Tmax > be.cfg.max_tokens:
        return {"skipped": f"largest step has {Tmax} tokens; the workspace holds {be.cfg.max_tokens}"}
    g = torch.Generator(device=dev).manual_seed(6)
    xb = torch.randn(Tmax, S.hidden, generator=g, device=dev).to(torch.bfloat16)
    ob = torch.empty(Tmax * K * S.hidden, dtype=torch.bfloat16, device=dev)

    def run_stream():
        for Ts, ids in steps:
            be._check(be._lib.ek_moe_forward(be._h, 0, xb.data_ptr(), Ts, ids.data_ptr(), K, ob.data_ptr()))

    run_stream()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    run_stream()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    tok = sum(t for t, _ in steps)
    return {"steps": args.stream, "tokens": tok, "seconds": dt, "tokens_per_s": tok / dt,
            "ms_per_step": dt / args.stream * 1e3}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--tokens", type=int, default=256)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--config", default="cfg3", choices=["cfg3", "cfg2"],
                    help="cfg3: DeepSeek-V3-shape layer, fp8 weights (the headline workload); cfg2: Qwen3-30B-A3B-shape "
                         "layer, bf16 weights, Zipf(1.1) expert load")
    ap.add_argument("--sweep", default="", help="comma-separated extra token counts reported under 'sweep'")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-check", action="store_true", help="skip the oracle check of the timed batch")
    ap.add_argument("--quick", action="store_true",
                    help="N = 1, for profiler captures: W warm-up passes, ONE block of K steps, a short stage profile; no "
                         "conditioning, no end-to-end loop, no check, no extras, no CPU baseline (not a benchmark number)")
    ap.add_argument("--no-extras", dest="extras", action="store_false",
                    help="N = 1: leave out the default sweep and the cfg2 / INT8 rows under 'extra'")
    ap.add_argument("--stream", type=int, default=0,
                    help="also run a continuous-batching stream of this many steps (the default run takes a 300-step sample; 2000 = the full configuration) (decode ~Poisson(96) tokens, a "
                         "512-2048 token prefill chunk every 10th step, Zipf(1.2) expert load rotated every 200 steps, "
                         "every expert >= 1 row) through the controller-level entry point; reported under 'stream'")
    ap.add_argument("--worker-threads", type=int, default=0,
                    help="also drive the worker-level seam: one single-expert call per distinct expert of the batch "
                         "from this many host threads; reported under 'worker_path'")
    ap.add_argument("--layers", type=int, default=1,
                    help="N > 1: MoE layers per step (58 = the full DeepSeek-V3 expert stack; each layer has its own weights)")
    ap.add_argument("--ep-mode", default="auto", choices=["auto", "gather", "a2a", "peer"],
                    help="exchange scheme at N > 1 (auto: peer-memory kernels up to 2048 global tokens, NCCL all-gather / "
                         "reduce-scatter if peer mappings fail, all-to-all above)")
    ap.add_argument("--experts", type=int, default=0,
                    help="routed experts (default: the configuration's own count; smaller values give profiler-sized cases)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl != "reference" else args.warmup
    if args.quick:
        args.no_check = args.no_cpu_baseline = True
        args.extras = False
    if args.impl == "reference":
        return run_reference(args)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    torch.cuda.set_device(local)
    if world > 1:
        return main_ep(args, rank, world, local)
    return main_single(args, local)


if __name__ == "__main__":
    main()
