#!/usr/bin/env python
"""Benchmark of the MoE expert-layer hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--tokens T] [--impl reference]

One "step" is one pass of a DeepSeek-V3-shape MoE layer (hidden 7168, intermediate 2048, 256
routed experts + 1 shared, top-8, group-limited sigmoid routing, FP8-e4m3 weights with
128x128 fp32 block scales, bf16 activations) over a batch of T tokens: route -> bucket ->
gather -> grouped gate/up + SwiGLU -> grouped down -> weighted combine + shared expert.
Weights are random (seeded, generated on the device) and the activations synthetic ~N(0,1).

Prints ONE JSON line.  `value` is tokens/s with inputs and outputs resident in HBM; `e2e` is
the same pass through the host-buffer entry point of the C ABI (pinned host -> device copy of
the activations and device -> host read of the result inside the timed region).
`--impl reference` times the CPU restatement of the reference's torch expert path on the host
cores on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "expert-kit_b200"))

import torch  # noqa: E402

METRIC = "MoE expert-layer tokens/s (DSV3 FP8-W/bf16-A)"
UNIT = "tokens/s"
H, I, E, K, NSHARED = 7168, 2048, 256, 8, 1
LAYERS_NOTE = ""
FALLBACK_HBM_GBS = 6650.0
FALLBACK_TFLOPS = 1590.0


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
    """Samples SM clock and throttle reasons of one GPU while the benchmark runs: a background
    thread reading NVML every 200 ms (reading only; nothing is ever set).  An `nvidia-smi -lms`
    child is the fallback when the NVML binding is missing."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        import threading
        self.sm, self.reasons, self.max_mhz = [], set(), None
        self.p = None
        self._stop = threading.Event()
        self._thread = None
        if os.environ.get("EK_BENCH_NO_CLOCKS"):
            return
        try:
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = int(visible.split(",")[gpu_index]) if visible and visible.split(",")[gpu_index].isdigit() else gpu_index
            h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
            names = {"hw_slowdown": getattr(pynvml, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
                     "hw_thermal_slowdown": getattr(pynvml, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
                     "sw_thermal_slowdown": getattr(pynvml, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
                     "sw_power_cap": getattr(pynvml, "nvmlClocksThrottleReasonSwPowerCap", 0x4)}

            def loop():
                while not self._stop.is_set():
                    try:
                        self.sm.append(float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)))
                        r = pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                        for n, bit in names.items():
                            if r & bit:
                                self.reasons.add(n)
                    except Exception:
                        pass
                    self._stop.wait(0.2)

            self._thread = threading.Thread(target=loop, daemon=True)
            self._thread.start()
            return
        except Exception:
            self._thread = None
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                       "-i", str(gpu_index), "-lms", "500"], stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.p = None

    def stop(self):
        if self._thread is not None:
            self._stop.set()
            self._thread.join(timeout=2)
            if not self.sm:
                return None
            busy = [v for v in self.sm if v > 0.5 * max(self.sm)]
            return {"sm_mhz": statistics.median(busy or self.sm), "sm_max_mhz": self.max_mhz,
                    "reasons": sorted(self.reasons), "samples": len(self.sm), "source": "nvml"}
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
                "samples": len(sm), "source": "nvidia-smi"}


# ---- synthetic layer on the device ----------------------------------------------------------
def quantize_fp8_block_dev(w: torch.Tensor):
    r, c = w.shape
    b = w.view(r // 128, 128, c // 128, 128)
    amax = b.abs().amax(dim=(1, 3)).clamp_min(1e-12)
    s = (amax / 448.0).float()
    q = (b / s[:, None, :, None]).to(torch.float8_e4m3fn).view(r, c)
    return q.contiguous(), s.contiguous()


def build_backend(T_max: int, rank: int = 0, seed: int = 3000, n_experts: int = E, ep_rank: int = 0,
                  ep_size: int = 1, n_layers: int = 1):
    """Registers the router, the shared expert and the routed experts this rank owns
    (all of them at ep_size 1).  The router weight is the same on every rank."""
    import ek_b200
    from ek_b200.backend import expert_tensors
    dev = torch.device("cuda", torch.cuda.current_device())
    cfg = ek_b200.BackendConfig(hidden=H, intermediate=I, n_experts=n_experts, top_k=K, scoring=1, n_group=8,
                                topk_group=4, norm_topk_prob=True, routed_scaling=2.5, n_shared_experts=NSHARED,
                                bf16_combine=False, quant=1, max_tokens=T_max, max_layers=n_layers,
                                device=dev.index, ep_rank=ep_rank, ep_size=ep_size, model_name="dsv3")
    be = ek_b200.Backend(cfg)
    el = n_experts // ep_size
    for layer in range(n_layers):
        g = torch.Generator(device=dev).manual_seed(seed + 1000 * layer)
        wg = (torch.randn(n_experts, H, generator=g, device=dev) * 0.02).to(torch.bfloat16)
        be.register_router(layer, wg, torch.zeros(n_experts, device=dev))
        g = torch.Generator(device=dev).manual_seed(seed + 1000 * layer + 1 + rank)
        for e in list(range(ep_rank * el, (ep_rank + 1) * el)) + ["shared"]:
            mats = []
            for shape in ((I, H), (I, H), (H, I)):
                w = torch.randn(shape, generator=g, device=dev) * 0.02
                mats.append(quantize_fp8_block_dev(w))
            (up, us), (gate, gs), (down, ds) = mats
            if e == "shared":
                be.register_expert(be.shared_id(layer), expert_tensors(layer, None, up, gate, down, us, gs, ds, shared=True))
            else:
                be.register_expert(be.expert_id(layer, e), expert_tensors(layer, e, up, gate, down, us, gs, ds))
    return be, dev


def algorithmic(T: int, active: int, n_exp: int = E):
    sc = 12 * (I // 128) * (H // 128)
    per = 3 * H * I + sc
    bytes_layer = (active + NSHARED) * per + 2 * H * n_exp + 4 * T * H
    flops_layer = 2 * T * H * n_exp + 6 * H * I * T * K + 6 * H * I * NSHARED * T
    rows = T * K + NSHARED * T
    gu_bytes = (active + NSHARED) * (2 * H * I + 8 * (I // 128) * (H // 128)) + rows * H * 2 + rows * I * 2
    gu_flops = 4 * H * I * rows
    return bytes_layer, flops_layer, gu_bytes, gu_flops


# ---- CPU baseline (oracle port of the reference's torch expert path) -------------------------
def cpu_baseline(T: int, budget_s: float = 15.0, seed: int = 5):
    """Times route + bucket + per-expert bf16 FFN loop + weighted combine + shared expert on the
    host cores, on a sample of distinct experts (weights dequantised once at load, as the
    reference's load_module would hold them), and scales the expert loop to the number of
    experts the routing actually activates."""
    from oracle import ek_oracle as O
    from oracle import configs as OC
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    cfg = OC.config(3)
    g = torch.Generator().manual_seed(seed)
    wg = (torch.randn(E, H, generator=g) * 0.02).to(torch.bfloat16)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    t0 = time.perf_counter()
    logits, ids, w = O.route(cfg, x, wg, torch.zeros(E))
    counts, offsets, perm = O.bucket(ids, E)
    t_route = time.perf_counter() - t0
    active = int((counts > 0).sum())
    n_sample = 4
    experts = []
    for _ in range(n_sample):
        ws = [torch.randn(s, generator=g).mul_(0.02).to(torch.bfloat16) for s in ((I, H), (I, H), (H, I))]
        experts.append(ws)
    rows_per = max(1, round(T * K / max(active, 1)))
    xe = x[:rows_per] if rows_per <= T else x.repeat((rows_per + T - 1) // T, 1)[:rows_per]
    O.expert_ffn(xe, *experts[0])   # warm-up
    n_calls, t_ffn = 0, 0.0
    while t_ffn < budget_s * 0.6 and n_calls < 64:
        ws = experts[n_calls % n_sample]
        t0 = time.perf_counter()
        O.expert_ffn(xe, *ws)
        t_ffn += time.perf_counter() - t0
        n_calls += 1
    per_call = t_ffn / n_calls
    t0 = time.perf_counter()
    O.expert_ffn(x, *experts[0])    # shared expert: all T rows
    t_shared = time.perf_counter() - t0
    outs = torch.zeros(T, K, H, dtype=torch.bfloat16)
    t0 = time.perf_counter()
    O.combine(outs, w, False)
    t_comb = time.perf_counter() - t0
    step = t_route + active * per_call + t_shared + t_comb
    return dict(value=T / step, unit=UNIT, cores=cores, kind="port",
                sample=(f"router+bucket, {n_calls} single-expert FFN calls of {rows_per} rows on {n_sample} distinct "
                        f"bf16 experts (scaled to the {active} active experts), shared expert, combine; T={T}; "
                        f"{per_call * 1e3:.2f} ms per expert call"),
                ms_per_step=step * 1e3)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    T = args.tokens
    vals = []
    base = None
    for i in range(args.warmup + args.steps):
        base = cpu_baseline(T, budget_s=max(2.0, 30.0 / max(1, args.warmup + args.steps)), seed=5 + i)
        if i >= args.warmup:
            vals.append(base)
    v = statistics.mean(b["value"] for b in vals)
    ms = statistics.mean(b["ms_per_step"] for b in vals)
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak" if args.gpus == 1 else "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": workload_config(T, args.gpus),
            "cpu_baseline": {"value": v, "unit": UNIT, "cores": base["cores"], "kind": "port", "sample": base["sample"]},
            "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def workload_config(T: int, n_gpus: int, n_exp: int = E):
    return {"workload": f"cfg3 DeepSeek-V3-shape MoE layer, W8A16 (fp8 e4m3 + 128x128 fp32 block scales), global batch T={T} tokens"
                        + LAYERS_NOTE
                        + ("" if n_exp == E else f" [REDUCED to {n_exp} routed experts: profiling case, not the benchmark]"),
            "hidden": H, "intermediate": I, "experts": n_exp, "shared_experts": NSHARED, "top_k": K,
            "routing": "sigmoid, 8 groups, top-4 groups, renormalised, x2.5", "global_tokens": T,
            "tokens_per_gpu": T // n_gpus,
            "parallelism": "single GPU" if n_gpus == 1 else
            f"ep{n_gpus}: {n_exp // n_gpus} routed experts per GPU, shared expert and router replicated, "
            "decode-sized batches: tokens stored into every rank's memory and fp32 partial sums loaded from every "
            "rank's memory by the library's own kernels over NVLink (CUDA IPC mappings; NCCL all-gather + "
            "reduce-scatter if the mappings cannot be made), NCCL all-to-all dispatch/combine above 2048 tokens; "
            "global batch fixed (strong scaling)",
            "l2": "weights streamed per step (11.3 GB) exceed the 126 MB L2; no flush needed"}



def main_ep(args, rank: int, world: int, local: int):
    """N > 1: the layer's experts are sharded over the ranks (expert parallel); the global batch of
    --tokens tokens is split evenly over the ranks; dispatch and combine are NCCL all-to-alls."""
    import torch.distributed as dist
    import ek_b200
    import datetime
    os.environ["NCCL_DEBUG"] = os.environ.get("EK_BENCH_NCCL_DEBUG", "WARN")   # keep stdout to the one JSON line
    # a short collective timeout: a rank that fails must not keep the others (and the GPUs) waiting
    dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=90))
    T = args.tokens
    if T % world:
        raise SystemExit("--tokens must be divisible by the number of GPUs")
    Tl = T // world
    n_exp = args.experts
    NL = args.layers
    be, dev = build_backend(max(T, 256), rank, n_experts=n_exp, ep_rank=rank, ep_size=world, n_layers=NL)
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(stream)
    be.set_stream(stream.cuda_stream)
    moe_one = ek_b200.ExpertParallelMoE(ek_b200.BackendStages(be), mode=args.ep_mode)

    class _Stack:
        """One step = every layer of the stack on its own seeded hidden states (the attention
        blocks between the MoE layers are not part of this path)."""
        last_counts_all = None

        def forward(self, _layer, x):
            y = None
            for layer in range(NL):
                y = moe_one.forward(layer, x)
            self.last_counts_all = moe_one.last_counts_all
            return y

    moe = _Stack() if NL > 1 else moe_one
    g = torch.Generator(device=dev).manual_seed(17 + rank)
    xs = [torch.randn(Tl, H, generator=g, device=dev).to(torch.bfloat16) for _ in range(4)]
    for i in range(args.warmup):
        moe.forward(0, xs[i % 4])
    be.sync()
    sampler = ClockSampler(local) if rank == 0 else None
    dist.barrier()
    torch.cuda.synchronize()
    l0 = be.kernel_launches()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        moe.forward(0, xs[i % 4])
    e1.record()
    be.sync()
    torch.cuda.synchronize()
    launches = be.kernel_launches() - l0
    t = torch.tensor([e0.elapsed_time(e1)], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dist.barrier()
    ms = float(t.item())
    ms_step = ms / args.steps
    value = T * args.steps / (ms / 1e3)

    # dominant kernel on this rank: gate/up over the local experts
    be.stage_timing(True)
    samples = {}
    for i in range(max(5, min(args.steps, 20))):
        moe.forward(0, xs[i % 4])
        be.sync()
        for k_, v in be.stage_times().items():
            samples.setdefault(k_, []).append(v)
    be.stage_timing(False)
    stage = {k_: statistics.median(v) for k_, v in samples.items()}
    el = n_exp // world
    if moe.last_counts_all is not None and args.ep_mode == "a2a":
        mine = moe.last_counts_all[:, rank * el:(rank + 1) * el].sum(0)
    else:   # gather scheme: this rank routed the whole global batch itself
        mine = be.expert_counts(0)[rank * el:(rank + 1) * el]
    active = int((mine > 0).sum())
    rows = int(mine.sum()) + NSHARED * Tl
    # keep every GPU under the same load for about half a second so that the clock sampler sees it;
    # the iteration count is the same on all ranks (forward is a collective)
    for _ in range(int(600.0 / max(ms_step, 0.05)) + 1):
        moe.forward(0, xs[0])
    be.sync()
    clocks = sampler.stop() if sampler else None
    P = peaks()
    gu_bytes = (active + NSHARED) * (2 * H * I + 8 * (I // 128) * (H // 128)) + rows * H * 2 + rows * I * 2
    gu_flops = 4 * H * I * rows
    gu_s = max(stage["gateup"], 1e-6) / 1e3
    roof = {"bound": "hbm", "achieved": gu_bytes / gu_s / 1e9, "peak": P["hbm"], "unit": "GB/s"}
    roof["frac"] = roof["achieved"] / roof["peak"]
    roof["traffic"] = int((active + NSHARED) * 976.77e6 / 33)
    roof["kernel"] = "ffn_tc_kernel<fp8, gate/up + SwiGLU> on rank 0's experts"
    roof["peak_source"] = P["src"]
    roof["launch_ms"] = stage["gateup"]
    roof["algorithmic_bytes"] = gu_bytes
    # per-GPU roofline of the sharded layer: each rank streams its own experts once
    sc = 12 * (I // 128) * (H // 128)
    bytes_rank = (active + NSHARED) * (3 * H * I + sc) + 2 * H * n_exp + 4 * Tl * H
    flops_rank = 2 * Tl * H * n_exp + 6 * H * I * (rows)
    roof_s = NL * max(bytes_rank / (P["hbm"] * 1e9), flops_rank / (P["tf_sus"] * 1e12))   # per step
    nvlink_bytes = 2 * Tl * K * H * 2 * (1 - 1 / world)
    layer = {"roofline_tokens_per_s": T / roof_s, "frac": roof_s * 1e3 / ms_step, "bound": "hbm",
             "layers": NL, "bytes_per_gpu_per_layer": bytes_rank, "flops_per_gpu_per_layer": flops_rank, "active_experts_rank0": active,
             "nvlink_bytes_per_gpu_per_step": int(nvlink_bytes), "stage_ms_rank0": stage}

    # end to end: host batch in, host result out, through the public Python API of this package
    xh = [x.cpu().pin_memory() for x in xs]
    yh = torch.empty(Tl, H, dtype=torch.bfloat16).pin_memory()
    xd = torch.empty(Tl, H, dtype=torch.bfloat16, device=dev)
    e2e_steps = max(3, min(args.steps, 10))

    def e2e_step(i):
        xd.copy_(xh[i % 4], non_blocking=True)
        y = moe.forward(0, xd)
        yh.copy_(y, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    e2e_step(0)
    dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        e2e_step(i)
    torch.cuda.synchronize()
    tt = torch.tensor([time.perf_counter() - t0], device=dev)
    dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    e2e = {"value": T * e2e_steps / float(tt.item()), "unit": UNIT, "h2d_bytes_per_step": T * H * 2,
           "d2h_bytes_per_step": T * H * 2, "steps": e2e_steps}
    if rank == 0:
        # the CPU baseline is timed at N = 1 only: here the other ranks' host threads (NCCL proxies,
        # the ranks waiting in destroy_process_group) share the cores and would distort it
        base = None
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": workload_config(T, world, n_exp),
                "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks, "roofline": roof,
                "layer_roofline": layer, "cpu_baseline": base}
        print(json.dumps(line))
    moe_one.close()
    be.close()
    dist.barrier()
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--tokens", type=int, default=256)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--sweep", default="", help="comma-separated extra token counts reported under 'sweep'")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--stream", type=int, default=0,
                    help="also run a continuous-batching stream of this many steps (decode ~Poisson(96) tokens, a "
                         "512-2048 token prefill chunk every 10th step, Zipf(1.2) expert load rotated every 200 steps, "
                         "every expert >= 1 row) through the controller-level entry point; reported under 'stream'")
    ap.add_argument("--worker-threads", type=int, default=0,
                    help="also drive the worker-level seam: one single-expert call per distinct expert of the batch "
                         "from this many host threads; reported under 'worker_path'")
    ap.add_argument("--layers", type=int, default=1,
                    help="MoE layers per step (58 = the full DeepSeek-V3 expert stack; each layer has its own weights)")
    ap.add_argument("--ep-mode", default="auto", choices=["auto", "gather", "a2a", "peer"],
                    help="exchange scheme at N > 1 (auto: all-gather/reduce-scatter up to 2048 global tokens; peer: the same "
                         "scheme with the library's own kernels over peer memory instead of NCCL collectives)")
    ap.add_argument("--experts", type=int, default=E,
                    help="routed experts (default: the full 256; smaller values give profiler-sized cases)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl != "reference" else args.warmup
    global LAYERS_NOTE
    if args.layers > 1:
        LAYERS_NOTE = f" x {args.layers} layers per step (cfg5-style expert stack)"
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
    dist = None

    T = args.tokens
    sweep = [int(t) for t in args.sweep.split(",") if t]
    n_exp = args.experts
    be, dev = build_backend(max([T] + sweep + ([2400] if args.stream > 0 else [])), rank, n_experts=n_exp)
    # the library launches on this stream, so torch's events bracket exactly its kernels
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(stream)
    be.set_stream(stream.cuda_stream)
    g = torch.Generator(device=dev).manual_seed(17 + rank)

    def timed(Tn: int, steps: int, warmup: int):
        xs = [torch.randn(Tn, H, generator=g, device=dev).to(torch.bfloat16) for _ in range(4)]
        y = torch.empty(Tn, H, dtype=torch.bfloat16, device=dev)
        for i in range(warmup):
            be.moe_forward_fused_async(0, xs[i % 4], y)
        be.sync()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        l0 = be.kernel_launches()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            be.moe_forward_fused_async(0, xs[i % 4], y)
        e1.record()
        be.sync()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        launches = be.kernel_launches() - l0
        if dist is not None:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dist.barrier()
            ms = float(t.item())
        return ms, launches, xs

    sampler = ClockSampler(local) if rank == 0 else None
    ms, launches, xs = timed(T, args.steps, args.warmup)
    ms_step = ms / args.steps
    value = world * T * args.steps / (ms / 1e3)

    # dominant kernel: per-launch duration from CUDA events on the launching stream
    def stage_profile(Tn, xs_n, n_prof):
        """Median per-stage device time (CUDA events on the launching stream) over n_prof passes."""
        be.stage_timing(True)
        yy = torch.empty(Tn, H, dtype=torch.bfloat16, device=dev)
        samples = {}
        for i in range(n_prof):
            be.moe_forward_fused_async(0, xs_n[i % 4], yy)
            be.sync()
            for k_, v in be.stage_times().items():
                samples.setdefault(k_, []).append(v)
        be.stage_timing(False)
        return {k_: statistics.median(v) for k_, v in samples.items()}

    y = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
    stage = stage_profile(T, xs, max(5, min(args.steps, 20)))
    if sampler:
        # keep the GPU under the same load until the sampler has seen it for half a second
        t_end = time.perf_counter() + 0.6
        while time.perf_counter() < t_end:
            be.moe_forward_fused_async(0, xs[0], y)
            be.sync()
    clocks = sampler.stop() if sampler else None
    counts = be.expert_counts(0)
    active = int((counts > 0).sum())
    P = peaks()
    bytes_layer, flops_layer, gu_bytes, gu_flops = algorithmic(T, active, n_exp)
    gu_s = stage["gateup"] / 1e3
    t_hbm, t_tc = gu_bytes / (P["hbm"] * 1e9), gu_flops / (P["tf"] * 1e12)
    if t_hbm >= t_tc:
        roof = {"bound": "hbm", "achieved": gu_bytes / gu_s / 1e9, "peak": P["hbm"], "unit": "GB/s"}
    else:
        roof = {"bound": "tensor", "achieved": gu_flops / gu_s / 1e12, "peak": P["tf"], "unit": "TFLOP/s"}
    roof["frac"] = roof["achieved"] / roof["peak"]
    # DRAM bytes of one launch, scaled by active experts from the ncu capture of the same kernel on
    # a 33-expert case (973.30 MB read + 3.47 MB written; profiles/ffn_tc_fp8_cfg3_32experts_T32.md)
    roof["traffic"] = int((active + NSHARED) * 976.77e6 / 33)
    roof["kernel"] = "ffn_tc_kernel<fp8, gate/up + SwiGLU>"
    roof["peak_source"] = P["src"]
    roof["launch_ms"] = stage["gateup"]
    roof["algorithmic_bytes"] = gu_bytes
    layer_roof_s = max(bytes_layer / (P["hbm"] * 1e9), flops_layer / (P["tf_sus"] * 1e12))
    layer = {"roofline_tokens_per_s": T / layer_roof_s, "frac": (T / (ms_step / 1e3)) / (T / layer_roof_s),
             "bound": "hbm" if bytes_layer / (P["hbm"] * 1e9) >= flops_layer / (P["tf_sus"] * 1e12) else "tensor",
             "bytes": bytes_layer, "flops": flops_layer, "active_experts": active, "stage_ms": stage}

    # end to end through the host-buffer entry point of the C ABI
    xh = [x.cpu().pin_memory() for x in xs]
    yh = torch.empty(T, H, dtype=torch.bfloat16).pin_memory()
    e2e_steps = max(3, min(args.steps, 10))
    for i in range(2):
        be._check(be._lib.ek_moe_forward_fused(be._h, 0, xh[i].data_ptr(), T, yh.data_ptr(), None))
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        be._check(be._lib.ek_moe_forward_fused(be._h, 0, xh[i % 4].data_ptr(), T, yh.data_ptr(), None))
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    if dist is not None:
        t = torch.tensor([e2e_s], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e = {"value": world * T * e2e_steps / e2e_s, "unit": UNIT, "h2d_bytes_per_step": T * H * 2,
           "d2h_bytes_per_step": T * H * 2, "steps": e2e_steps}

    sweep_out = {}
    for Tn in sweep:
        ms_n, _, xs_n = timed(Tn, max(3, args.steps // 2), 3)
        st = ms_n / max(3, args.steps // 2)
        stage_n = stage_profile(Tn, xs_n, 5)
        c = be.expert_counts(0)
        a = int((c > 0).sum())
        bl, fl, _, _ = algorithmic(Tn, a, n_exp)
        rs = max(bl / (P["hbm"] * 1e9), fl / (P["tf_sus"] * 1e12))
        sweep_out[str(Tn)] = {"tokens_per_s": world * Tn / (st / 1e3), "ms_per_step": st, "active_experts": a,
                              "layer_roofline_frac": (rs * 1e3) / st,
                              "stage_ms": {k_: round(v, 4) for k_, v in stage_n.items()}}

    worker_out = None
    if args.worker_threads > 0:
        # The reference's own seam: one single-expert call per distinct expert of the batch, issued
        # from N host threads as its worker does per RPC (host buffers in and out); the library
        # serves whatever is queued as one grouped launch.
        import threading
        xw = torch.randn(T, H, generator=g, device=dev).to(torch.bfloat16)
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
        worker_out = {"threads": nthr, "calls_per_step": len(experts), "ms_per_step": dt * 1e3,
                      "tokens_per_s": T / dt, "calls": c1 - c0, "grouped_passes": b1 - b0,
                      "note": "single-expert calls with host buffers from N threads (wall clock, expert FFN only)"}

    stream_out = None
    if args.stream > 0:
        gs = torch.Generator().manual_seed(4)
        gd = torch.Generator(device=dev).manual_seed(5)
        zipf_p = (torch.arange(1, n_exp + 1, dtype=torch.float32, device=dev) ** -1.2)

        def zipf_ids_dev(Ts, rot):
            """k distinct experts per token from a Zipf(1.2) law over a rotated ranking; experts left
            without a row take over the first (hottest) slot of distinct tokens."""
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
        xb = torch.randn(Tmax, H, generator=g, device=dev).to(torch.bfloat16)
        ob = torch.empty(Tmax * K * H, dtype=torch.bfloat16, device=dev)
        import ctypes as C

        def run_stream():
            for Ts, ids in steps:
                be._check(be._lib.ek_moe_forward(be._h, 0, xb.data_ptr(), Ts, ids.data_ptr(), K, ob.data_ptr()))

        if Tmax <= be.cfg.max_tokens:
            run_stream()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            run_stream()
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            tok = sum(t for t, _ in steps)
            stream_out = {"steps": args.stream, "tokens": tok, "seconds": dt, "tokens_per_s": tok / dt,
                          "ms_per_step": dt / args.stream * 1e3}
        else:
            stream_out = {"skipped": f"largest step has {Tmax} tokens; rerun with --sweep {Tmax} to size the workspace"}

    if rank == 0:
        base = None
        if not args.no_cpu_baseline:
            b = cpu_baseline(T)
            base = {k_: b[k_] for k_ in ("value", "unit", "cores", "kind", "sample")}
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": workload_config(T, world, n_exp),
                "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks, "roofline": roof,
                "layer_roofline": layer, "cpu_baseline": base}
        if sweep_out:
            line["sweep"] = sweep_out
        if stream_out:
            line["stream"] = stream_out
        if worker_out:
            line["worker_path"] = worker_out
        print(json.dumps(line))
    be.close()
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
