"""MoE-layer throughput benchmark for the B200 MoE expert hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

A step is one pass of the MoE layer (router top-K -> token grouping -> MXFP8
activation quantisation -> grouped gate/up contraction + SwiGLU -> grouped down
contraction + affinity -> combine) over one batch of seeded synthetic tokens.
Rank 0 prints one JSON line:

* ``value``      tokens/s with inputs resident in HBM (the captured launch sequence replayed)
* ``e2e``        the same through host buffers (pinned host -> device and device -> host copies timed)
* ``api_path``   the same step through the drop-in entry points ``router_topk`` -> ``moe_group_tokens`` ->
                 ``moe_cte`` (prefill) and ``router_topk`` -> ``moe_tkg`` (decode), eager, resident inputs
* ``sustained``  the replay again for a few seconds (power-capped clocks), against the sustained peak
* ``roofline``   the dominant kernel against the measured peak; ``kernel_ms`` every kernel's device time
* ``decode`` / ``decode_mxfp4_weights`` / ``finegrained_prefill`` / ``ep_prefill``  the other single-GPU
                 configurations, each with its own ``kernel_ms`` and roofline fraction
* ``cpu_baseline``  the reference's CPU algorithm (the oracle restatement) timed on this host on a bounded
                 sample of the same inputs; the same sample checks the GPU's rows (``parity_sample``)

``--impl reference`` times only that CPU algorithm.  With ``--gpus N`` > 1 the experts are split over the ranks
(expert parallelism, T tokens per rank) and the line adds ``ep_prefill_strong`` (32768 tokens in total).
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
    "ep_prefill_zipf": dict(kind="prefill", T=32768, H=4096, I=1536, E=128, K=8, B=256, zipf=1.2),
    "tiny_prefill": dict(kind="prefill", T=256, H=512, I=1024, E=4, K=2, B=128, zipf=None),
    # cut-down shapes for profiler captures: the Mixtral block geometry with I = 2048 (201 MB of weights, larger
    # than L2, a few hundred MB on the device) and the fine-grained / expert-parallel shapes with fewer experts and
    # tokens at the same rows per expert (256 / 2048), so the same launch forms are taken
    "profile_prefill": dict(kind="prefill", T=4096, H=4096, I=2048, E=8, K=2, B=512, zipf=None),
    "profile_decode": dict(kind="decode", T=64, H=4096, I=2048, E=8, K=2, B=128, zipf=None),
    "profile_finegrained": dict(kind="prefill", T=1024, H=7168, I=2048, E=32, K=8, B=128, zipf=1.2),
    "profile_ep_prefill": dict(kind="prefill", T=8192, H=4096, I=1536, E=32, K=8, B=256, zipf=None),
}

# DRAM bytes (read + write) per launch of the dominant kernel, from the ncu captures summarised under
# profiles/ (file named beside each figure; null where no capture of the current kernel exists).
NCU_TRAFFIC = {
    "mixtral_prefill": {"bytes": 1.623e9, "from": "profiles/grouped_mxfp8_gemm_mixtral_prefill.md (gate/up contraction, "
                        "pair + left-over launch, captured on this workload at full size)"},
    "mixtral_decode": {"bytes": 989.8e6, "from": "profiles/grouped_mxfp8_gemm_mixtral_decode.md (gate/up launch, captured "
                       "on this workload at full size)"},
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


def make_inputs(cfg, seed):
    """Seeded tokens ~N(0,1) bf16 [T,H], router weight ~N(0,0.02) bf16 [H,E], and the Zipf logit bias if the
    workload has one (-s * ln(rank) over a seeded permutation of the experts)."""
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


# ------------------------------------------------------------------ CPU legs (the oracle: reference algorithm, CPU)
def cpu_route(cfg, hidden, router_w, bias):
    """Router top-K and block assignment of the whole batch on the CPU, timed (the oracle's restatements of
    router_topk_torch_ref and of the find_nonzero_indices -> cumsum -> indexed_flatten chain)."""
    from oracle import routing
    T, E, K, B = cfg["T"], cfg["E"], cfg["K"], cfg["B"]
    t0 = time.perf_counter()
    _, idx, aff = routing.router_topk(hidden.float(), router_w.float(), None if bias is None else bias.float(), K,
                                      routing.SOFTMAX, True, True)
    t1 = time.perf_counter()
    idx = idx.numpy().astype("int32")
    N = routing.get_n_blocks(T, K, E, B)
    routing.group_tokens(routing.mask_from_index(idx, E), B, N)
    t2 = time.perf_counter()
    return idx, aff.numpy(), {"router_topk_s": t1 - t0, "group_tokens_s": t2 - t1}


def cpu_synthetic_expert(cfg, e):
    """Seeded weights of one expert for the CPU-only arm (no GPU weights exist to read back): uniformly random finite
    e4m3 codes with block scales of 2^-12 .. 2^-9, which puts the weights at the N(0, 0.02) order of magnitude.  The
    oracle's arithmetic (table lookup, power-of-two scaling, fp32 matmul) takes the same time whatever the values."""
    import numpy as np
    H, I = cfg["H"], cfg["I"]
    rng = np.random.default_rng(7000 + e)

    def codes(shape):
        c = rng.integers(0, 256, shape, dtype=np.uint8)
        c[(c & 0x7F) == 0x7F] = 0x38  # the two NaN patterns -> 1.0
        return c

    return (codes((1, 2, I, H)), rng.integers(115, 119, (1, 2, I, H // 32), dtype=np.uint8),
            codes((1, H, I)), rng.integers(115, 119, (1, H, I // 32), dtype=np.uint8))


def cpu_block_sample(cfg, hidden_np, idx, aff, expert_weights, steps, warmup, threads, n_experts=4,
                     blocks_per_expert=2, budget_s=None):
    """The oracle's per-block recipe on a bounded sample: for the first ``n_experts`` experts that received tokens,
    dequantise the expert's weights and push its first ``blocks_per_expert`` blocks of B token rows through
    quantise -> gate/up -> SwiGLU -> re-quantise -> down -> x affinity (what the reference's golden does per block).

    Returns the seconds per step, the rows covered and the rows' results (for the parity check).
    """
    import numpy as np
    import torch

    from oracle import moe
    torch.set_num_threads(threads)
    B, E = cfg["B"], cfg["E"]
    plan = []
    for e in range(E):
        tok = np.flatnonzero((idx == e).any(axis=1))
        if tok.size:
            plan.append((e, tok[: blocks_per_expert * B]))
        if len(plan) == n_experts:
            break
    weights = {e: expert_weights(e) for e, _ in plan}
    times, results = [], None
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        res = []
        for e, tok in plan:
            ew = moe.ExpertWeights(*weights[e], 0)
            for b0 in range(0, tok.size, B):
                t = tok[b0:b0 + B]
                y = moe.expert_mlp_rows(hidden_np[t], ew) * aff[t, e][:, None]
                res.append((e, t, y))
            del ew
        dt = time.perf_counter() - t0
        if it >= warmup:
            times.append(dt)
        results = res
        if budget_s is not None and times and sum(times) + times[-1] > budget_s:
            break
    rows = sum(t.size for _, t in plan)
    return dict(seconds_per_step=sum(times) / len(times), steps=len(times), rows=rows,
                blocks=sum(-(-t.size // B) for _, t in plan), experts=len(plan), results=results)


def cpu_baseline_line(cfg, sample, route_t, threads, kind_note):
    """tokens/s of the whole layer extrapolated from the sample: T*K token-expert rows at the sample's rate
    (weight dequantisation included in proportion), plus the routing that was timed in full."""
    T, K = cfg["T"], cfg["K"]
    layer_s = sample["seconds_per_step"] * (T * K / sample["rows"]) + sum(route_t.values())
    return {"value": T / layer_s, "unit": "tokens/s", "cores": threads, "kind": "port",
            "extrapolated": True, "seconds_per_sample": sample["seconds_per_step"], "routing_seconds": route_t,
            "sample": f"extrapolated from {sample['blocks']} blocks of up to {cfg['B']} token rows over "
                      f"{sample['experts']} experts ({sample['rows']} of {T * K} token-expert rows: dequantise the "
                      f"expert's weights, quantise/gate-up/SwiGLU/re-quantise/down per block) at H={cfg['H']}, "
                      f"I={cfg['I']}; router top-K and block assignment of all {T} tokens timed in full; {kind_note}"}


def cpu_decode_full(cfg, hidden_np, idx, aff, expert_weights, steps, warmup, threads):
    """The decode layer in full on the CPU: every expert that a token chose, dequantised and applied."""
    import numpy as np
    import torch

    from oracle import moe
    torch.set_num_threads(threads)
    E = cfg["E"]
    active = [e for e in range(E) if (idx == e).any()]
    weights = {e: expert_weights(e) for e in active}
    times, out = [], None
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        out = np.zeros_like(hidden_np)
        for e in active:
            tok = np.flatnonzero((idx == e).any(axis=1))
            ew = moe.ExpertWeights(*weights[e], 0)
            out[tok] += moe.expert_mlp_rows(hidden_np[tok], ew) * aff[tok, e][:, None]
            del ew
        if it >= warmup:
            times.append(time.perf_counter() - t0)
    return dict(seconds_per_step=sum(times) / len(times), steps=len(times), out=out,
                sample=f"the whole decode step: {len(active)} active experts dequantised and applied to their tokens "
                       f"(T={cfg['T']}, H={cfg['H']}, I={cfg['I']})")


def run_reference(args, cfg, name):
    """The reference's CPU algorithm alone (no GPU work): every step is the bounded sample of cpu_block_sample."""
    threads = os.cpu_count() or 1
    if int(os.environ.get("RANK", "0")) != 0:
        return
    hidden, router_w, bias = make_inputs(cfg, 0)
    idx, aff, route_t = cpu_route(cfg, hidden, router_w, bias)
    hidden_np = hidden.float().numpy()
    if cfg["kind"] == "decode":
        s = cpu_decode_full(cfg, hidden_np, idx, aff, lambda e: cpu_synthetic_expert(cfg, e), max(1, args.steps),
                            args.warmup, threads)
        value, sec = cfg["T"] / (s["seconds_per_step"] + sum(route_t.values())), s["seconds_per_step"]
        base = {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port", "extrapolated": False,
                "sample": s["sample"]}
    else:
        s = cpu_block_sample(cfg, hidden_np, idx, aff, lambda e: cpu_synthetic_expert(cfg, e), max(1, args.steps),
                             args.warmup, threads)
        base = cpu_baseline_line(cfg, s, route_t, threads, "tokens and router as in the GPU arm, expert weights "
                                 "random e4m3 codes of the same magnitude (the GPU arm's are quantised on the device)")
        value, sec = base["value"], s["seconds_per_step"]
    line = {
        "impl": "reference", "metric": "moe_layer_tokens_per_s", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": s["steps"], "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "mxfp8_e4m3", "data": "synthetic",
        "config": {"workload": name, **{k: cfg[k] for k in "THIEKB"}},
        "cpu_baseline": base,
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------ GPU legs
def device_expert_rows(weights, e):
    """One expert's device weights back on the host in the oracle's rows form (codes [1,2,I,H] / [1,H,I] + scales)."""
    import numpy as np
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from moe_testlib import gate_up_dev_rows, sf_atoms_to_rows
    n1, n2 = weights.w1_sf.numel() // weights.E, weights.w2_sf.numel() // weights.E
    H, I = weights.H, weights.I
    w1 = weights.w1[e].cpu().numpy()
    w2 = weights.w2[e].cpu().numpy()
    s1 = sf_atoms_to_rows(weights.w1_sf[e * n1:(e + 1) * n1].cpu().numpy(), 2 * I, H)
    s2 = sf_atoms_to_rows(weights.w2_sf[e * n2:(e + 1) * n2].cpu().numpy(), H, I)
    rows = gate_up_dev_rows(I)
    c1 = np.stack([w1[rows[0]], w1[rows[1]]])[None]
    sc1 = np.stack([s1[rows[0]], s1[rows[1]]])[None]
    return c1, sc1, w2[None], s2[None]


def time_replays(layer, steps):
    import torch
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    s.record()
    for _ in range(steps):
        layer.replay()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / steps


def roofline_block(cfg, name, per_kernel, ms_step, peaks, w_format, with_library=False):
    work = algorithmic_work(cfg, w_format)
    traffic = NCU_TRAFFIC.get(name, {"bytes": None, "from": None})
    if cfg["kind"] == "prefill":
        peak = 2.0 * peaks["bf16_tflops"]
        achieved = work["gemm1_flops"] / (per_kernel["gemm1_swiglu"] * 1e-3) / 1e12
        down = work["gemm2_flops"] / (per_kernel["gemm2_scale"] * 1e-3) / 1e12
        layer = work["layer_flops"] / (ms_step * 1e-3) / 1e12
        return {"bound": "tensor", "kernel": "grouped_mxfp8_gemm_kernel<gate_up+SwiGLU>", "achieved": achieved,
                "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "frac_of_sustained_peak": achieved / (2.0 * peaks["bf16_tflops_sustained"]),
                "traffic": traffic["bytes"], "traffic_from": traffic["from"],
                "peak_source": f"2 x {peaks['source']} cuBLAS bf16 burst ({peaks['bf16_tflops']} TF/s): dense fp8/mxfp8 "
                               f"issues at twice the bf16 rate; frac_of_sustained_peak uses 2 x the sustained figure "
                               f"({peaks['bf16_tflops_sustained']} TF/s)",
                "down_tflops": down, "down_frac": down / peak, "layer_tflops": layer, "layer_frac": layer / peak,
                "library_dense_mxfp8_tflops": library_mxfp8_tflops(min(cfg["T"] * cfg["K"], 8192), 2 * cfg["I"], cfg["H"])
                if with_library else None}
    peak = peaks["hbm_gbs"]
    achieved = work["gemm1_weight_bytes"] / (per_kernel["gemm1_swiglu"] * 1e-3) / 1e9
    down = work["gemm2_weight_bytes"] / (per_kernel["gemm2_scale"] * 1e-3) / 1e9
    layer = work["decode_bytes"] / (ms_step * 1e-3) / 1e9
    return {"bound": "hbm", "kernel": "grouped_mxfp8_gemm_kernel<gate_up+SwiGLU>", "achieved": achieved,
            "peak": peak, "unit": "GB/s", "frac": achieved / peak, "traffic": traffic["bytes"],
            "traffic_from": traffic["from"], "peak_source": f"{peaks['source']} copy bandwidth",
            "down_gbs": down, "down_frac": down / peak, "layer_gbs": layer, "layer_frac": layer / peak}


def gpu_leg(name, cfg, dev, peaks, steps, w_format="e4m3", weights=None, router_path=0, gemm_variant=0, seed=0):
    """One workload on one GPU through the fused layer: graph replay (ms/step) and an eager pass with CUDA events
    around every kernel.  Returns the summary and the live objects."""
    import torch

    from nki_library_b200.layer import MoELayer, random_expert_weights
    T, H, I, E, K, B = (cfg[k] for k in "THIEKB")
    hidden_h, router_w, bias = make_inputs(cfg, seed)
    if weights is None:
        weights = random_expert_weights(E, H, I, dev, seed=7, w_format=W_FORMATS[w_format])
    layer = MoELayer(router_w.to(dev), weights, K, B, T, None if bias is None else bias.to(dev),
                     router_path=router_path, gemm_variant=gemm_variant)
    x = hidden_h.to(dev)
    for _ in range(3):
        layer.forward(x)
    torch.cuda.synchronize()
    layer.capture(x)
    layer.replay()
    ms = time_replays(layer, steps)
    timers = {}
    for _ in range(max(3, min(steps, 10))):
        layer.forward(x, timers)
    torch.cuda.synchronize()
    per_kernel = {k: sum(a.elapsed_time(b) for a, b in v) / len(v) for k, v in timers.items()}
    status = layer.device_status()
    out = {"workload": name, **{k: cfg[k] for k in "THIEKB"}, "zipf": cfg["zipf"], "weight_format": w_format,
           "n_blocks": layer.N, "ms_per_step": ms, "tokens_per_s": T / (ms * 1e-3), "kernel_ms": per_kernel,
           "steps": steps, "launches_per_step": layer.kernels_per_forward, "launch_mode": "cuda graph replay",
           "roofline": roofline_block(cfg, name, per_kernel, ms, peaks, w_format)}
    if any(status):
        out["error"] = f"device status {status}"
    return out, layer, x, (hidden_h, router_w, bias)


def api_path_leg(cfg, layer, x, steps, ms_value):
    """The same step through the drop-in entry points with the reference's argument lists (eager, inputs resident):
    router_topk -> moe_group_tokens -> moe_cte for prefill, router_topk -> moe_tkg for decode."""
    import torch

    import nki_library_b200 as m
    T, E, K, B = cfg["T"], cfg["E"], cfg["K"], cfg["B"]
    dev = x.device
    logits = torch.empty((T, E), dtype=torch.float32, device=dev)
    aff = torch.empty((T, E), dtype=torch.float32, device=dev)
    idx = torch.empty((T, K), dtype=torch.int32, device=dev)
    spec = m.MoECTESpec(m.MoECTEImplementation.shard_on_block_mx)
    N = m.get_n_blocks(T, K, E, B)

    def step():
        m.router_topk(x, layer.w, layer.bias, logits, aff, idx, m.RouterActFnType.SOFTMAX, K, 1, 0,
                      router_pre_norm=True, norm_topk_prob=True, use_indirect_dma_scatter=True)
        if cfg["kind"] == "decode":
            return m.moe_tkg(x, layer.weights, None, aff, idx, False,
                             expert_affinities_scaling_mode=m.ExpertAffinityScaleMode.POST_SCALE)
        g = m.moe_group_tokens(idx, E, B, N)
        return m.moe_cte(x, aff.reshape(-1, 1), layer.weights, None, g["token_position_to_id"], g["block_to_expert"], B,
                         spec, conditions=g["conditions"], skip_dma=m.SkipMode(True, False))

    for _ in range(3):
        out = step()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(steps):
        out = step()
    e.record()
    torch.cuda.synchronize()
    ms = s.elapsed_time(e) / steps
    same = bool(torch.equal(out, layer.replay()))
    return {"ms_per_step": ms, "tokens_per_s": T / (ms * 1e-3), "vs_value": ms_value / ms,
            "calls": "router_topk -> moe_tkg" if cfg["kind"] == "decode" else "router_topk -> moe_group_tokens -> moe_cte",
            "launch_mode": "eager, per-call allocations included, prepared weights passed (cache hit)",
            "output_equals_fused_layer": same}


def parity_and_cpu(cfg, layer, inputs, threads, steps=2, warmup=1):
    """CPU baseline on the GPU run's own inputs (routing from the GPU, sampled experts' weights read back from the
    device) and, on the same rows, the GPU's per-position results against the CPU's."""
    import numpy as np
    import torch
    hidden_h, router_w, bias = inputs
    hidden_np = hidden_h.float().numpy()
    _, _, route_t = cpu_route(cfg, hidden_h, router_w, bias)
    idx = layer.idx.cpu().numpy()
    aff = layer.aff.cpu().numpy()
    inv = layer.inv.cpu().numpy()
    s = cpu_block_sample(cfg, hidden_np, idx, aff, lambda e: device_expert_rows(layer.weights, e), steps, warmup, threads)
    y_pos = layer.ws.y_pos
    worst, scale, n = 0.0, 0.0, 0
    for e, tok, y in s["results"]:
        k = (idx[tok] == e).argmax(axis=1)
        pos = torch.from_numpy(inv[tok, k].astype(np.int64)).to(y_pos.device)
        got = y_pos[pos].float().cpu().numpy()
        ref = torch.from_numpy(y).to(torch.bfloat16).float().numpy()
        worst = max(worst, float(np.abs(got - ref).max()))
        scale = max(scale, float(np.abs(ref).max()))
        n += tok.size
    parity = {"rows": n, "experts": s["experts"], "max_abs_err": worst, "max_abs_ref": scale,
              "max_rel_err": worst / max(scale, 1e-30), "tolerance": 2e-2, "ok": worst / max(scale, 1e-30) <= 2e-2,
              "what": "bf16(y * affinity) rows of the down contraction at the sampled positions vs the CPU oracle "
                      "on the same tokens, routing and device weights"}
    base = cpu_baseline_line(cfg, s, route_t, threads, "tokens, routing and the sampled experts' weights are the "
                             "GPU run's own (weights read back from the device)")
    return base, parity


def decode_leg(weights, peaks, dev, w_format, threads, with_cpu):
    """BASELINE's decode configuration (T = 64, Mixtral-8x7B shapes) on the given expert weights."""
    import numpy as np
    cfg = WORKLOADS["mixtral_decode"]
    out, layer, x, inputs = gpu_leg("mixtral_decode", cfg, dev, peaks, 100, w_format, weights, seed=99)
    out["algorithmic_gb_per_s"] = out["roofline"]["layer_gbs"]
    out["frac_of_hbm_peak"] = out["roofline"]["layer_frac"]
    out["api_path"] = api_path_leg(cfg, layer, x, 50, out["ms_per_step"])
    if with_cpu and w_format == "e4m3":
        idx, aff = layer.idx.cpu().numpy(), layer.aff.cpu().numpy()
        s = cpu_decode_full(cfg, inputs[0].float().numpy(), idx, aff, lambda e: device_expert_rows(weights, e), 1, 1,
                            threads)
        got = layer.replay().float().cpu().numpy()
        ref = s["out"]
        err = float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-30))
        out["cpu_baseline"] = {"value": cfg["T"] / s["seconds_per_step"], "unit": "tokens/s", "cores": threads,
                               "kind": "port", "extrapolated": False, "sample": s["sample"]}
        out["parity_sample"] = {"rows": cfg["T"], "max_rel_err": err, "tolerance": 2e-2, "ok": err <= 2e-2,
                                "what": "the whole [T, H] output vs the CPU oracle on the same tokens, routing and "
                                        "device weights"}
    return out


def run_single(args, cfg, name, dev, peaks):
    import torch

    from nki_library_b200.layer import HostPipeline, random_expert_weights
    threads = os.cpu_count() or 1
    T, H, I, E, K, B = (cfg[k] for k in "THIEKB")
    sampler = ClockSampler(dev.index or 0)
    sampler.start()
    steps = args.steps
    main_leg, layer, x, inputs = gpu_leg(name, cfg, dev, peaks, steps, args.weight_format, None, args.router_path,
                                         args.gemm_variant)
    if "error" in main_leg:
        raise RuntimeError(main_leg["error"])
    # the timed region proper: W warm-up replays, then exactly K
    for _ in range(max(args.warmup, 3)):
        layer.replay()
    ms_step = time_replays(layer, steps)
    # in-kernel clock probe over an eager pass
    probe = torch.zeros(4, dtype=torch.int64, device=dev)
    layer.clock_probe = probe
    layer.forward(x)
    torch.cuda.synchronize()
    layer.clock_probe = None
    pr = probe.cpu().tolist()
    kernel_sm_mhz = {"gemm1_swiglu": round(1e3 * pr[0] / pr[1], 1) if pr[1] else None,
                     "gemm2_scale": round(1e3 * pr[2] / pr[3], 1) if pr[3] else None}
    roofline = roofline_block(cfg, name, main_leg["kernel_ms"], ms_step, peaks, args.weight_format, with_library=True)
    # -------- CPU baseline + parity on the same rows (outside every timed region)
    cpu = parity = None
    if not args.skip_cpu and cfg["kind"] == "prefill" and args.weight_format == "e4m3":
        layer.replay()
        torch.cuda.synchronize()
        cpu, parity = parity_and_cpu(cfg, layer, inputs, threads)
    # -------- drop-in entry points
    api = api_path_leg(cfg, layer, x, steps, ms_step)
    # -------- sustained: the same replay for a few seconds
    sustained = None
    if args.sustained_s > 0:
        n = max(steps, int(args.sustained_s * 1e3 / ms_step))
        ms_s = time_replays(layer, n)
        sustained = {"seconds": ms_s * n * 1e-3, "steps": n, "ms_per_step": ms_s, "tokens_per_s": T / (ms_s * 1e-3)}
        if cfg["kind"] == "prefill":
            tf = algorithmic_work(cfg, args.weight_format)["layer_flops"] / (ms_s * 1e-3) / 1e12
            sustained.update(layer_tflops=tf, layer_frac_of_sustained_peak=tf / (2.0 * peaks["bf16_tflops_sustained"]),
                             layer_frac_of_burst_peak=tf / (2.0 * peaks["bf16_tflops"]))
    # -------- end to end through host buffers
    hidden_pin = inputs[0].pin_memory()
    out_pins = [torch.empty((T, H), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    pipe = HostPipeline(layer)
    pipe.submit(hidden_pin, out_pins[0])
    pipe.drain()
    pipe.step = 0
    e_start, e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e_start.record()
    for i in range(steps):
        pipe.submit(hidden_pin, out_pins[i & 1])
    pipe.drain()
    e_end.record()
    torch.cuda.synchronize()
    ms_e2e = e_start.elapsed_time(e_end) / steps
    status = layer.device_status()
    if any(status):
        raise RuntimeError(f"device status after the timed steps: {status}")
    clocks = sampler.stop()
    weights_bytes = layer.weights.nbytes()
    # -------- the other single-GPU configurations
    secondary = {}
    if name == "mixtral_prefill" and not args.no_secondary:
        secondary["decode"] = decode_leg(layer.weights, peaks, dev, args.weight_format, threads, not args.skip_cpu)
        if args.weight_format == "e4m3":
            w4 = random_expert_weights(E, H, I, dev, seed=8, w_format=W_FORMATS["e2m1"])
            secondary["decode_mxfp4_weights"] = decode_leg(w4, peaks, dev, "e2m1", threads, False)
            del w4
        del pipe, layer
        torch.cuda.empty_cache()
        for other in ("finegrained_prefill", "ep_prefill"):
            o, lay, _, _ = gpu_leg(other, WORKLOADS[other], dev, peaks, 10, args.weight_format)
            secondary[other] = o
            del lay
            torch.cuda.empty_cache()
    line = {
        "metric": "moe_layer_tokens_per_s", "value": T / (ms_step * 1e-3), "unit": "tokens/s",
        "n_gpus": 1, "steps": steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "mxfp8_e4m3",
        "data": "synthetic",
        "config": {"workload": name, **{k: cfg[k] for k in "THIEKB"}, "n_blocks": main_leg["n_blocks"],
                   "weight_format": args.weight_format, "tokens_per_gpu": T, "experts_per_gpu": E,
                   "parallelism": "single",
                   "l2": "inputs larger than L2 (expert weights %.2f GB streamed every step)" % (weights_bytes / 1e9)},
        "roofline": roofline,
        "kernel_ms": main_leg["kernel_ms"],
        "kernel_sm_mhz": kernel_sm_mhz,
        "api_path": api,
        "sustained": sustained,
        "parity_sample": parity,
        **secondary,
        "cpu_baseline": cpu if cpu is not None else {"value": None, "unit": "tokens/s", "cores": threads,
                                                     "kind": "port", "sample": "skipped"},
        "e2e": {"value": T / (ms_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": T * H * 2,
                "d2h_bytes_per_step": T * H * 2},
        "gpu_launches": main_leg["launches_per_step"] * steps,
        "launch_mode": "cuda graph replay (value, e2e, sustained) + eager instrumented pass (kernel_ms) + eager "
                       "drop-in calls (api_path)",
        "clocks": clocks,
    }
    print(json.dumps(line), flush=True)


def run_multi(args, cfg, name, dev, peaks, world, rank):
    """Expert parallelism: every rank keeps its own T tokens (weak scaling) and E / world experts; token rows
    travel to the owning rank and back through this library's peer-memory kernels (or NCCL all-to-all)."""
    import torch
    import torch.distributed as dist

    from nki_library_b200.ep import CudaOps, ExpertParallelMoE, PeerExpertParallelMoE
    from nki_library_b200.layer import HostPipeline, MoELayer, random_expert_weights

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    def build(cfg_, tokens, seed):
        H_, I_, E_, K_, B_ = cfg_["H"], cfg_["I"], cfg_["E"], cfg_["K"], cfg_["B"]
        hidden_h, router_w, bias = make_inputs(dict(cfg_, T=tokens), seed)
        w = random_expert_weights(E_ // world, H_, I_, dev, seed=7 + rank, w_format=W_FORMATS[args.weight_format])
        bias_d = None if bias is None else bias.to(dev)
        if args.ep_backend == "peer":
            lay = PeerExpertParallelMoE(router_w.to(dev), w, E_, K_, B_, tokens, router_bias=bias_d,
                                        capacity_factor=args.capacity_factor,
                                        fuse_return={"auto": None, "on": True, "off": False}[args.fuse_return])
        else:
            lay = ExpertParallelMoE(CudaOps(router_w.to(dev), w, E_, K_, B_, bias_d), E_)
        return lay, hidden_h, router_w, bias

    def timed(lay, x, steps, use_graph):
        for _ in range(max(args.warmup, 3)):
            lay.forward(x)
        barrier()
        if use_graph:
            lay.capture(x)
            lay.replay()
        barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(steps):
            lay.replay() if use_graph else lay.forward(x)
        e.record()
        barrier()
        t = torch.tensor([s.elapsed_time(e)], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item() / steps

    T, H, I, E, K, B = (cfg[k] for k in "THIEKB")
    if E % world != 0:
        raise SystemExit(f"workload has {E} experts, not divisible by {world} ranks")
    use_graph = args.ep_backend == "peer" and not args.no_graph
    layer, hidden_h, router_w, bias = build(cfg, T, rank)
    x = hidden_h.to(dev)
    sampler = ClockSampler(dev.index or 0)
    if rank == 0:
        sampler.start()
    ms_step = timed(layer, x, args.steps, use_graph)
    status = layer.device_status() if hasattr(layer, "device_status") else []
    if any(status):
        raise RuntimeError(f"device status after the timed steps: {status}")
    # eager pass with events around the phases
    def phase_ms(lay, inp, n_steps):
        """Eager steps with events around the exchange and the two contractions (this rank's own clock)."""
        timers = {}
        lay.timers = timers
        for _ in range(n_steps):
            lay.forward(inp)
        barrier()
        lay.timers = None
        n = len(timers["t0"])
        return {nm: sum(timers[f"t{i}"][j].elapsed_time(timers[f"t{i + 1}"][j]) for j in range(n)) / n
                for i, nm in enumerate(("dispatch", "gemm1_swiglu", "gemm2_scale"))}

    per_kernel = phase_ms(layer, x, args.steps) if args.ep_backend == "peer" else None
    # parity: rank 0's output against the single-GPU fused layer on the same tokens and all ranks' weights
    parity = None
    out_ep = layer.forward(x).clone()
    barrier()
    if rank == 0 and not args.skip_cpu:
        from nki_library_b200.weights import ExpertWeights
        parts = [random_expert_weights(E // world, H, I, dev, seed=7 + r, w_format=W_FORMATS[args.weight_format])
                 for r in range(world)]
        full = ExpertWeights(E, H, I, torch.cat([p.w1 for p in parts]), torch.cat([p.w1_sf for p in parts]),
                             torch.cat([p.w2 for p in parts]), torch.cat([p.w2_sf for p in parts]), None, None, False,
                             parts[0].w_format)
        del parts
        single = MoELayer(router_w.to(dev), full, K, B, T, None if bias is None else bias.to(dev))
        ref = single.forward(x).float()
        err = float((out_ep.float() - ref).abs().max() / ref.abs().max().clamp_min(1e-30))
        parity = {"rows": T, "max_rel_err": err, "tolerance": 1e-2, "ok": err <= 1e-2,
                  "what": "rank 0's expert-parallel output vs the single-GPU fused layer on the same tokens and all "
                          "ranks' weights (same kernels; a token's rows are summed in a different order)"}
        del single, full, ref
        torch.cuda.empty_cache()
    barrier()
    # end to end through host buffers
    hidden_pin = hidden_h.pin_memory()
    out_pins = [torch.empty((T, H), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    e_start, e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    # the copy engine alone (all ranks at once), for the ceiling of the host link per rank
    c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    c0.record()
    for _ in range(5):
        x.copy_(hidden_pin, non_blocking=True)
    c1.record()
    torch.cuda.synchronize()
    h2d_alone = 5 * T * H * 2 / (c0.elapsed_time(c1) * 1e-3) / 1e9
    pipe = None
    if use_graph:
        pipe = HostPipeline(layer)
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
        barrier()
        e_start.record()
        for i in range(args.steps):
            x.copy_(hidden_pin, non_blocking=True)
            out = layer.forward(x)
            out_pins[i & 1].copy_(out, non_blocking=True)
        e_end.record()
    barrier()
    t = torch.tensor([e_start.elapsed_time(e_end)], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_e2e = t.item() / args.steps
    clocks = sampler.stop() if rank == 0 else None
    launches = getattr(layer, "kernels_per_forward", 12)
    # strong scaling of the large expert-parallel configuration: 32768 tokens in total, split over the ranks
    strong = {}
    if name == "mixtral_prefill" and not args.no_secondary and args.ep_backend == "peer":
        del layer, pipe
        torch.cuda.empty_cache()
        for wl in ("ep_prefill", "ep_prefill_zipf"):
            c5 = WORKLOADS[wl]
            if c5["E"] % world or c5["T"] % world:
                continue
            try:
                lay5, h5, _, _ = build(c5, c5["T"] // world, 100 + rank)
                x5 = h5.to(dev)
                ms5 = timed(lay5, x5, 10, use_graph)
                k5 = phase_ms(lay5, x5, 5)
                st5 = lay5.device_status()
                strong[wl] = {"total_tokens": c5["T"], "tokens_per_gpu": c5["T"] // world,
                              "experts_per_gpu": c5["E"] // world, "ms_per_step": ms5,
                              "tokens_per_s": c5["T"] / (ms5 * 1e-3), "kernel_ms": k5, "device_status": st5,
                              "capacity_factor": args.capacity_factor,
                              "layer_tflops_per_gpu": algorithmic_work(c5)["layer_flops"] / world / (ms5 * 1e-3) / 1e12}
                del lay5
            except Exception as exc:  # reported in the line, never hidden
                strong[wl] = {"error": str(exc)[:300]}
            torch.cuda.empty_cache()
            barrier()
    if rank == 0:
        work = algorithmic_work(cfg, args.weight_format)
        roofline = None
        if per_kernel is not None:
            peak = 2.0 * peaks["bf16_tflops"]
            ach = work["gemm1_flops"] / (per_kernel["gemm1_swiglu"] * 1e-3) / 1e12
            roofline = {"bound": "tensor", "kernel": "grouped_mxfp8_gemm_kernel<gate_up+SwiGLU>", "achieved": ach,
                        "peak": peak, "unit": "TFLOP/s", "frac": ach / peak, "traffic": None,
                        "peak_source": f"2 x {peaks['source']} cuBLAS bf16 burst ({peaks['bf16_tflops']} TF/s)",
                        "layer_tflops_per_gpu": work["layer_flops"] / (ms_step * 1e-3) / 1e12}
        line = {
            "metric": "moe_layer_tokens_per_s", "value": world * T / (ms_step * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "mxfp8_e4m3",
            "data": "synthetic",
            "config": {"workload": name, **{k: cfg[k] for k in "THIEKB"}, "weight_format": args.weight_format,
                       "tokens_per_gpu": T, "experts_per_gpu": E // world,
                       "parallelism": (f"ep{world} (peer-memory dispatch/combine kernels over NVLink)"
                                       if args.ep_backend == "peer" else f"ep{world} (NCCL all-to-all dispatch/combine)"),
                       "l2": "inputs larger than L2 (expert weights streamed every step)"},
            "roofline": roofline,
            "kernel_ms": per_kernel,
            "parity_sample": parity,
            "ep_prefill_strong": strong or None,
            "cpu_baseline": {"value": None, "unit": "tokens/s", "cores": os.cpu_count() or 1, "kind": "port",
                             "sample": "timed at N=1 only"},
            "e2e": {"value": world * T / (ms_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": T * H * 2,
                    "d2h_bytes_per_step": T * H * 2,
                    "per_rank_gb_per_s": {"h2d": T * H * 2 / (ms_e2e * 1e-3) / 1e9,
                                          "d2h": T * H * 2 / (ms_e2e * 1e-3) / 1e9,
                                          "h2d_copy_alone_all_ranks_at_once": h2d_alone},
                    "cpu_affinity": getattr(args, "cpu_affinity", None)},
            "gpu_launches": launches * args.steps,
            "launch_mode": "cuda graph replay" if use_graph else "eager",
            "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    dist.destroy_process_group()


def bind_to_gpu_cpus(local: int):
    """Run this process on the CPUs NVML names as local to its GPU, so that pinned host buffers (first touched
    from here) sit in the memory next to the GPU's PCIe root.  Returns a short description for the JSON line."""
    try:
        import pynvml
        pynvml.nvmlInit()
        visible = os.environ.get("CUDA_VISIBLE_DEVICES")
        phys = int(visible.split(",")[local]) if visible and visible.split(",")[local].isdigit() else local
        handle = pynvml.nvmlDeviceGetHandleByIndex(phys)
        n_cpu = os.cpu_count() or 1
        words = pynvml.nvmlDeviceGetCpuAffinity(handle, (n_cpu + 63) // 64)
        ideal = {64 * w + b for w, word in enumerate(words) for b in range(64) if (int(word) >> b) & 1}
        allowed = os.sched_getaffinity(0)
        use = ideal & allowed
        if not use or use == allowed:
            return "unchanged (%d cpus)" % len(allowed)
        os.sched_setaffinity(0, use)
        return "gpu-local (%d of %d cpus)" % (len(use), len(allowed))
    except Exception as exc:  # no NVML, no permission: keep the default placement
        return "unchanged (%s)" % type(exc).__name__


def run_ours(args, cfg, name):
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    peaks = load_peaks()
    if world == 1:
        run_single(args, cfg, name, dev, peaks)
    else:
        args.cpu_affinity = bind_to_gpu_cpus(local)   # before any pinned buffer exists; N = 1 keeps all cores
        dist.init_process_group("nccl", device_id=dev)   # (its CPU leg uses them)
        run_multi(args, cfg, name, dev, peaks, world, rank)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="mixtral_prefill", choices=sorted(WORKLOADS))
    ap.add_argument("--skip-cpu", action="store_true", help="omit the CPU baseline and parity legs (profiling runs)")
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
    ap.add_argument("--no-secondary", action="store_true",
                    help="omit the other configurations' measurements (profiling runs)")
    ap.add_argument("--sustained-s", type=float, default=2.0, help="length of the sustained replay leg in seconds (0 = off)")
    ap.add_argument("--router-path", type=int, default=0, help="1 split-K router, 2 tcgen05 router (0 = by shape)")
    args = ap.parse_args()
    cfg = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference(args, cfg, args.workload)
    else:
        run_ours(args, cfg, args.workload)


if __name__ == "__main__":
    main()
