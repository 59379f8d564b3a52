"""MoE-layer throughput benchmark for the B200 MoE expert hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

A step is one pass of the MoE layer (router top-K -> token grouping -> MXFP8
activation quantisation -> grouped gate/up contraction + SwiGLU -> grouped down
contraction + affinity -> combine) over one batch of seeded synthetic tokens.
Rank 0 prints one JSON line.  ``value`` is tokens/s with inputs resident in HBM;
``e2e`` is the same metric through the public API with host buffers (pinned
host -> device copy of the tokens and device -> host copy of the result inside
the timed region).  ``--impl reference`` times the reference's CPU algorithm
(the oracle restatement) on this host's cores instead.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# benchmark configurations that fit one GPU (mixtral_prefill is the headline case)
WORKLOADS = {
    "mixtral_prefill": dict(kind="prefill", T=4096, H=4096, I=14336, E=8, K=2, B=512, zipf=None),
    "mixtral_decode": dict(kind="decode", T=64, H=4096, I=14336, E=8, K=2, B=128, zipf=None),
    "finegrained_prefill": dict(kind="prefill", T=8192, H=7168, I=2048, E=256, K=8, B=128, zipf=1.2),
    "ep_prefill": dict(kind="prefill", T=32768, H=4096, I=1536, E=128, K=8, B=256, zipf=None),
    "tiny_prefill": dict(kind="prefill", T=256, H=512, I=1024, E=4, K=2, B=128, zipf=None),
}


# DRAM bytes (read + write) per launch of the dominant kernel, from the ncu captures summarised under
# profiles/ (one capture per workload; null where none was taken).
NCU_TRAFFIC_BYTES = {
    "mixtral_prefill": (1.004123e9 + 118.779392e6) + (0.486658e9 + 10.018304e6),  # CTA-pair + left-over launch
    "mixtral_decode": 971.416576e6 + 18.775808e6,
}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"],
                    bf16_tflops_sustained=p.get("bf16_tflops_sustained", p["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples the SM clock and throttle reasons through NVML every few milliseconds while a region runs
    (read-only queries; falls back to one nvidia-smi query if NVML is unavailable)."""

    REASONS = (("hw_slowdown", 0x8), ("hw_thermal_slowdown", 0x40), ("sw_thermal_slowdown", 0x20),
               ("sw_power_cap", 0x4))

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self.thread = None
        self.handle = None
        try:
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = int(visible.split(",")[gpu_index]) if visible and visible.split(",")[gpu_index].isdigit() else gpu_index
            self.nv = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.handle = None

    def _loop(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(float(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)))
                mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle))
                for name, bit in self.REASONS:
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.003)

    def start(self):
        if self.handle is not None:
            self.thread = threading.Thread(target=self._loop, daemon=True)
            self.thread.start()

    def stop(self):
        if self.thread is not None:
            self._stop.set()
            self.thread.join(timeout=2)
            sm = self.samples
            return {"sm_mhz": statistics.median(sm) if sm else None, "sm_min_mhz": min(sm) if sm else None,
                    "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(sm),
                    "source": "NVML, 3 ms period, over the timed regions"}
        try:
            out = subprocess.run(["nvidia-smi", f"--id={self.gpu}", "--query-gpu=clocks.sm,clocks.max.sm",
                                  "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=10).stdout
            cur, mx = (float(v) for v in out.strip().split(","))
            return {"sm_mhz": cur, "sm_max_mhz": mx, "reasons": [], "samples": 1, "source": "nvidia-smi after the run"}
        except Exception:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["clock query unavailable"], "samples": 0}


W_FORMATS = {"e4m3": 0, "e5m2": 1, "e2m1": 5}


def algorithmic_work(cfg, w_format="e4m3"):
    """Figures used for roofline.achieved: useful work only, no padding rows, no re-reads."""
    T, H, I, E, K = cfg["T"], cfg["H"], cfg["I"], cfg["E"], cfg["K"]
    wb = (0.5 if w_format == "e2m1" else 1.0) + 1 / 32  # bytes per weight element incl. its share of the scale
    return {
        "gemm1_flops": 4.0 * T * K * H * I,
        "gemm2_flops": 2.0 * T * K * H * I,
        "layer_flops": 6.0 * T * K * H * I,
        # decode: every expert's weights and scales once, tokens in and out, router weight
        "decode_bytes": E * 3.0 * H * I * wb + 2.0 * T * H * 2 + H * E * 2,
        "gemm1_weight_bytes": E * 2.0 * H * I * wb,
        "gemm2_weight_bytes": E * 1.0 * H * I * wb,
    }


def library_mxfp8_tflops(M, N, K):
    """cuBLASLt's dense MXFP8 GEMM of the gate/up projection's shape, for context next to the roofline (or None)."""
    import torch
    try:
        a = (torch.randn(M, K, device="cuda") * 0.5).to(torch.float8_e4m3fn)
        b = (torch.randn(N, K, device="cuda") * 0.5).to(torch.float8_e4m3fn)

        def sf(rows):
            n = ((rows + 127) // 128) * ((K // 32 + 3) // 4) * 512
            return torch.full((n,), 127, dtype=torch.uint8, device="cuda").view(torch.float8_e8m0fnu)
        sa, sb = sf(M), sf(N)
        for _ in range(3):
            torch._scaled_mm(a, b.t(), scale_a=sa, scale_b=sb, out_dtype=torch.bfloat16)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(10):
            torch._scaled_mm(a, b.t(), scale_a=sa, scale_b=sb, out_dtype=torch.bfloat16)
        e.record()
        torch.cuda.synchronize()
        return 2.0 * M * N * K / (s.elapsed_time(e) / 10 * 1e-3) / 1e12
    except Exception:
        return None


def make_inputs(cfg, device, seed):
    import torch
    g = torch.Generator()
    g.manual_seed(1234 + seed)
    T, H, E = cfg["T"], cfg["H"], cfg["E"]
    hidden = torch.randn((T, H), generator=g, dtype=torch.float32).to(torch.bfloat16)
    router_w = (torch.randn((H, E), generator=g, dtype=torch.float32) * 0.02).to(torch.bfloat16)
    bias = None
    if cfg["zipf"] is not None:
        rank = torch.randperm(E, generator=g).float() + 1.0
        bias = (-cfg["zipf"] * torch.log(rank)).to(torch.bfloat16)
    return hidden, router_w, bias


# ------------------------------------------------------------------ CPU legs (oracle)
def cpu_sample(cfg, steps, warmup, threads, budget_s=None):
    """Time the oracle restatement of the reference's per-block golden loop on a bounded sample.

    Sample: ``n_rows`` token-expert rows of one expert at the workload's H and I
    (one weight dequantisation + the block recipe), which is how the reference's
    golden walks blocks.  tokens/s = rows / K / time.
    """
    import numpy as np
    import torch

    from oracle import moe, mx
    torch.set_num_threads(threads)
    H, I, K = cfg["H"], cfg["I"], cfg["K"]
    n_rows = min(cfg["T"] * K // max(cfg["E"], 1), 512) if cfg["kind"] == "prefill" else max(cfg["T"] * K // cfg["E"], 1)
    n_rows = max(n_rows, 1)
    rng = np.random.default_rng(0)
    c1 = rng.integers(0, 0x7E, size=(1, 2, I, H), dtype=np.uint8)
    s1 = rng.integers(110, 120, size=(1, 2, I, H // 32), dtype=np.uint8)
    c2 = rng.integers(0, 0x7E, size=(1, H, I), dtype=np.uint8)
    s2 = rng.integers(110, 120, size=(1, H, I // 32), dtype=np.uint8)
    x = torch.randn(n_rows, H).to(torch.bfloat16).float().numpy()
    times = []
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        ew = moe.ExpertWeights(c1, s1, c2, s2, 0)
        y = moe.expert_mlp_rows(x, ew)
        dt = time.perf_counter() - t0
        if it >= warmup:
            times.append(dt)
        del ew, y
        if budget_s is not None and times and sum(times) + times[-1] > budget_s:
            break  # the next step would overrun the wall-clock budget of this leg
    t = sum(times) / len(times)
    return dict(value=n_rows / K / t, seconds_per_step=t, rows=n_rows, steps=len(times),
                sample=f"{n_rows} token-expert rows through one expert (dequantise weights + quantise/gate-up/SwiGLU/"
                       f"re-quantise/down) at H={H}, I={I}; tokens/s = rows/K/time")


def run_reference(args, cfg, name):
    threads = os.cpu_count() or 1
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # every step is the same bounded sample; run the K steps asked for unless that would take over ~2.5 minutes
    warm = max(0, min(args.warmup, 2))
    r = cpu_sample(cfg, max(1, args.steps), warm, threads, budget_s=150.0)
    steps = r["steps"]
    line = {
        "impl": "reference", "metric": "moe_layer_tokens_per_s", "value": r["value"], "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warm,
        "ms_per_step": r["seconds_per_step"] * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "mxfp8_e4m3", "data": "synthetic", "config": {"workload": name, **{k: cfg[k] for k in "THIEKB"}},
        "cpu_baseline": {"value": r["value"], "unit": "tokens/s", "cores": threads, "kind": "port",
                         "sample": r["sample"]},
        "e2e": {"value": r["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------ GPU leg
def decode_leg(weights, peaks, device, w_format="e4m3"):
    """Mixtral decode workload (T = 64 tokens, Mixtral-8x7B shapes) on the given expert weights: tokens/s and HBM fraction."""
    import torch

    from nki_library_b200.layer import MoELayer
    cfg = WORKLOADS["mixtral_decode"]
    T, H, E, K, B = cfg["T"], cfg["H"], cfg["E"], cfg["K"], cfg["B"]
    hidden, router_w, _ = make_inputs(cfg, device, 99)
    layer = MoELayer(router_w.to(device), weights, K, B, T)
    x = hidden.to(device)
    for _ in range(3):
        layer.forward(x)
    torch.cuda.synchronize()
    layer.capture(x)
    layer.replay()
    steps = 100
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    s.record()
    for _ in range(steps):
        layer.replay()
    e.record()
    torch.cuda.synchronize()
    ms = s.elapsed_time(e) / steps
    if any(layer.device_status()):
        return {"error": f"device status {layer.device_status()}"}
    gbs = algorithmic_work(cfg, w_format)["decode_bytes"] / (ms * 1e-3) / 1e9
    return {"workload": "mixtral_decode", "weight_format": w_format, "T": T, "ms_per_step": ms, "tokens_per_s": T / (ms * 1e-3),
            "algorithmic_gb_per_s": gbs, "frac_of_hbm_peak": gbs / peaks["hbm_gbs"], "hbm_peak_gbs": peaks["hbm_gbs"],
            "steps": steps, "launch_mode": "cuda graph replay"}


def run_ours(args, cfg, name):
    import torch
    import torch.distributed as dist

    import nki_library_b200 as m
    from nki_library_b200.layer import MoELayer, random_expert_weights

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    peaks = load_peaks()
    T, H, I, E, K, B = (cfg[k] for k in "THIEKB")

    hidden_h, router_w, bias = make_inputs(cfg, dev, rank)
    hidden_pin = hidden_h.pin_memory()
    out_pin = torch.empty((T, H), dtype=torch.bfloat16).pin_memory()
    hidden_d = hidden_h.to(dev)
    bias_d = None if bias is None else bias.to(dev)
    if world == 1:
        weights = random_expert_weights(E, H, I, dev, seed=7, w_format=W_FORMATS[args.weight_format])
        layer = MoELayer(router_w.to(dev), weights, K, B, T, bias_d, router_path=args.router_path,
                         gemm_variant=args.gemm_variant)
        n_blocks = layer.N

        def forward(h, timers=None):
            return layer.forward(h, timers)

        def device_status():
            return layer.device_status()

        def launches_per_step():
            return layer.kernels_per_forward
    else:
        # Expert parallelism: every rank keeps its own T tokens (weak scaling) and E / world experts;
        # token rows travel to the owning rank and back through NCCL all-to-all.
        from nki_library_b200.ep import CudaOps, ExpertParallelMoE, PeerExpertParallelMoE
        if E % world != 0:
            raise SystemExit(f"workload has {E} experts, not divisible by {world} ranks")
        weights = random_expert_weights(E // world, H, I, dev, seed=7 + rank, w_format=W_FORMATS[args.weight_format])
        n_blocks = None
        if args.ep_backend == "peer":
            # dispatch / combine by this library's own kernels storing into peer GPUs' memory (NVLink)
            layer = PeerExpertParallelMoE(router_w.to(dev), weights, E, K, B, T, router_bias=bias_d,
                                          capacity_factor=args.capacity_factor, fuse_return={"auto": None, "on": True, "off": False}[args.fuse_return])

            def forward(h, timers=None):
                layer.timers = timers
                return layer.forward(h)

            def device_status():
                return layer.device_status()

            def launches_per_step():
                return layer.kernels_per_forward
        else:
            ops = CudaOps(router_w.to(dev), weights, E, K, B, bias_d)
            ep = ExpertParallelMoE(ops, E)

            def forward(h, timers=None):
                ops.timers = timers
                return ep.forward(h)

            def device_status():
                from nki_library_b200 import pipeline
                return [int(v) for ws in pipeline._workspaces.values() for v in ws.status.cpu().tolist()[1:3]]

            _count = {"n": 0}

            def launches_per_step():
                return _count["n"]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        forward(hidden_d)
    barrier()
    if world > 1 and args.ep_backend != "peer":
        ops.launches = 0
        forward(hidden_d)
        _count["n"] = ops.launches
        barrier()
    status = device_status()
    if any(status):
        raise RuntimeError(f"device status after warm-up: {status}")

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    # -------- resident-input leg (value): the captured launch sequence (single GPU) or eager steps (EP)
    use_graph = (world == 1 or args.ep_backend == "peer") and not args.no_graph
    if use_graph:
        layer.capture(hidden_d)
        layer.replay()
    barrier()
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_start.record()
    for _ in range(args.steps):
        if use_graph:
            layer.replay()
        else:
            forward(hidden_d)
    t_end.record()
    barrier()
    ms_total = t_start.elapsed_time(t_end)
    status = device_status()
    if any(status):
        raise RuntimeError(f"device status after the timed steps: {status}")
    # -------- the same steps again, eagerly, with CUDA events around every kernel (roofline input)
    probe = torch.zeros(4, dtype=torch.int64, device=dev)
    if world == 1:
        layer.clock_probe = probe
    timers = {}
    barrier()
    for _ in range(args.steps):
        forward(hidden_d, timers)
    barrier()
    if world == 1:
        layer.clock_probe = None
    pr = probe.cpu().tolist()
    kernel_sm_mhz = {"gemm1_swiglu": round(1e3 * pr[0] / pr[1], 1) if pr[1] else None,
                     "gemm2_scale": round(1e3 * pr[2] / pr[3], 1) if pr[3] else None}
    if world == 1:
        per_kernel = {k: sum(a.elapsed_time(b) for a, b in v) / len(v) for k, v in timers.items()}
    else:
        n = len(timers["t0"])
        names = ("dispatch" if args.ep_backend == "peer" else "gather_quantize", "gemm1_swiglu", "gemm2_scale")
        per_kernel = {nm: sum(timers[f"t{i}"][j].elapsed_time(timers[f"t{i + 1}"][j]) for j in range(n)) / n
                      for i, nm in enumerate(names)}
    forward(hidden_d)  # drops the event hooks again
    barrier()
    status = device_status()
    if any(status):
        raise RuntimeError(f"device status after the instrumented steps: {status}")
    # -------- end-to-end leg: host buffers through the public layer call
    barrier()
    e_start, e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if use_graph:
        from nki_library_b200.layer import HostPipeline
        pipe = HostPipeline(layer)
        out_pins = [out_pin, torch.empty_like(out_pin).pin_memory()]
        pipe.submit(hidden_pin, out_pins[0])
        pipe.drain()
        pipe.step = 0
        barrier()
        e_start.record()
        for i in range(args.steps):
            pipe.submit(hidden_pin, out_pins[i & 1])
        pipe.drain()
        e_end.record()
    else:
        e_start.record()
        for _ in range(args.steps):
            hidden_d.copy_(hidden_pin, non_blocking=True)
            out = forward(hidden_d)
            out_pin.copy_(out, non_blocking=True)
        e_end.record()
    barrier()
    ms_e2e = e_start.elapsed_time(e_end)
    clocks = sampler.stop() if rank == 0 else None

    if world > 1:
        t = torch.tensor([ms_total, ms_e2e], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total, ms_e2e = t.tolist()
    status = device_status()
    if any(status):
        raise RuntimeError(f"device status after the end-to-end steps: {status}")

    if rank == 0:
        work = algorithmic_work(cfg, args.weight_format)
        ms_step = ms_total / args.steps
        if cfg["kind"] == "prefill":
            dom = "gemm1_swiglu"
            peak = 2.0 * peaks["bf16_tflops"]
            achieved = work["gemm1_flops"] / (per_kernel[dom] * 1e-3) / 1e12
            roofline = {"bound": "tensor", "kernel": "grouped_mxfp8_gemm_kernel<gate_up+SwiGLU>", "achieved": achieved,
                        "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                        "frac_of_sustained_peak": achieved / (2.0 * peaks["bf16_tflops_sustained"]),
                        "traffic": NCU_TRAFFIC_BYTES.get(name) if world == 1 else None,
                        "peak_source": f"2 x {peaks['source']} cuBLAS bf16 burst ({peaks['bf16_tflops']} TF/s); "
                                       "dense fp8/mxfp8 issues at twice the bf16 rate; frac_of_sustained_peak "
                                       f"uses 2 x the sustained bf16 figure ({peaks['bf16_tflops_sustained']} TF/s)",
                        "layer_tflops": work["layer_flops"] / (ms_step * 1e-3) / 1e12,
                        "library_dense_mxfp8_tflops": library_mxfp8_tflops(min(T * K, 8192), 2 * I, H)
                        if world == 1 else None}
        else:
            dom = "gemm1_swiglu"
            peak = peaks["hbm_gbs"]
            achieved = work["gemm1_weight_bytes"] / (per_kernel[dom] * 1e-3) / 1e9
            roofline = {"bound": "hbm", "kernel": "grouped_mxfp8_gemm_kernel<gate_up+SwiGLU>", "achieved": achieved,
                        "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                        "traffic": NCU_TRAFFIC_BYTES.get(name) if world == 1 else None,
                        "peak_source": f"{peaks['source']} copy bandwidth",
                        "layer_gbs": work["decode_bytes"] / (ms_step * 1e-3) / 1e9}
        cpu = (dict(value=None, sample="skipped (--skip-cpu)") if args.skip_cpu
               else cpu_sample(cfg, 4, 1, os.cpu_count() or 1))
        decode = decode_mxfp4 = None
        if world == 1 and name == "mixtral_prefill" and not args.no_decode_leg:
            decode = decode_leg(weights, peaks, dev, args.weight_format)
            if args.weight_format == "e4m3":
                # the same decode step with MXFP4 (e2m1) expert weights: half the bytes to stream
                w4 = random_expert_weights(E, H, I, dev, seed=8, w_format=W_FORMATS["e2m1"])
                decode_mxfp4 = decode_leg(w4, peaks, dev, "e2m1")
                del w4
        line = {
            "metric": "moe_layer_tokens_per_s", "value": world * T / (ms_step * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "mxfp8_e4m3",
            "data": "synthetic",
            "config": {"workload": name, **{k: cfg[k] for k in "THIEKB"}, "n_blocks": n_blocks,
                       "weight_format": args.weight_format,
                       "tokens_per_gpu": T, "experts_per_gpu": E // world,
                       "parallelism": "single" if world == 1 else
                       (f"ep{world} (peer-memory dispatch/combine kernels over NVLink)" if args.ep_backend == "peer"
                        else f"ep{world} (NCCL all-to-all dispatch/combine)"),
                       "l2": "inputs larger than L2 (expert weights %.2f GB streamed every step)" % (weights.nbytes() / 1e9)},
            "roofline": roofline,
            "decode": decode,
            "decode_mxfp4_weights": decode_mxfp4,
            "kernel_ms": per_kernel,
            "kernel_sm_mhz": kernel_sm_mhz,
            "cpu_baseline": {"value": cpu["value"], "unit": "tokens/s", "cores": os.cpu_count() or 1, "kind": "port",
                             "sample": cpu["sample"]},
            "e2e": {"value": world * T / (ms_e2e / args.steps * 1e-3), "unit": "tokens/s",
                    "h2d_bytes_per_step": T * H * 2, "d2h_bytes_per_step": T * H * 2},
            "gpu_launches": launches_per_step() * args.steps * 3,
            "launch_mode": "cuda graph replay (value, e2e) + eager instrumented pass (kernel_ms)" if use_graph
                           else "eager",
            "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="mixtral_prefill", choices=sorted(WORKLOADS))
    ap.add_argument("--skip-cpu", action="store_true", help="omit the CPU baseline leg (profiling runs)")
    ap.add_argument("--weight-format", default="e4m3", choices=sorted(W_FORMATS),
                    help="element type of the expert weights (activations are always MXFP8 e4m3)")
    ap.add_argument("--ep-backend", default="peer", choices=["peer", "nccl"],
                    help="expert-parallel exchange for --gpus > 1: peer-memory kernels (default) or NCCL all-to-all")
    ap.add_argument("--capacity-factor", type=float, default=2.5,
                    help="receive-buffer size of the peer-memory exchange, in multiples of a rank's fair share")
    ap.add_argument("--no-graph", action="store_true", help="launch kernels eagerly instead of replaying a CUDA graph")
    ap.add_argument("--gemm-variant", type=lambda v: int(v, 0), default=0,
                    help="variant word of the grouped contractions (B200MOE_GEMM_* bits; 0 = library default)")
    ap.add_argument("--fuse-return", default="auto", choices=["auto", "on", "off"],
                    help="expert parallelism: let the down contraction's epilogue store result rows into their GPUs "
                         "(on), copy them in a separate kernel (off), or choose by rank count (auto)")
    ap.add_argument("--no-decode-leg", action="store_true", help="omit the secondary decode measurements (profiling runs)")
    ap.add_argument("--router-path", type=int, default=0, help="1 split-K router, 2 tcgen05 router (0 = by shape)")
    args = ap.parse_args()
    cfg = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference(args, cfg, args.workload)
    else:
        run_ours(args, cfg, args.workload)


if __name__ == "__main__":
    main()
