"""The reference arm of bench.py runs on the host alone: check the JSON line it prints against the bench contract."""

import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(extra_env=None):
    env = dict(os.environ)
    env.update(extra_env or {})
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--workload",
                          "tiny_prefill", "--gpus", "1", "--steps", "2", "--warmup", "1"],
                         capture_output=True, text=True, timeout=300, env=env, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    return [json.loads(l) for l in out.stdout.splitlines() if l.startswith("{")]


def test_reference_arm_prints_one_contract_line():
    lines = _run()
    assert len(lines) == 1
    d = lines[0]
    assert d["impl"] == "reference" and d["metric"] == "moe_layer_tokens_per_s" and d["unit"] == "tokens/s"
    assert d["higher_is_better"] is True and d["steps"] == 2 and d["n_gpus"] == 1 and d["value"] > 0
    assert d["config"]["workload"] == "tiny_prefill" and d["vs_baseline"] is None
    cpu = d["cpu_baseline"]
    assert cpu["kind"] == "port" and cpu["cores"] >= 1 and cpu["value"] == d["value"] and cpu["sample"]
    assert d["e2e"] == {"value": d["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_reference_arm_other_ranks_stay_silent():
    """Under a multi-rank launch only rank 0 runs the host arm; the others exit 0 without output."""
    assert _run({"RANK": "1", "WORLD_SIZE": "2", "LOCAL_RANK": "1"}) == []


def test_gpu_local_cpu_binding_uses_the_nvml_mask(monkeypatch):
    """``bind_to_gpu_cpus`` narrows the process to the CPUs NVML reports for the GPU (a fake NVML here), keeps the
    placement when the mask covers everything or nothing, and never raises."""
    import types
    sys.path.insert(0, ROOT)
    import bench
    allowed = set(range(8))
    calls = []
    fake = types.SimpleNamespace(nvmlInit=lambda: None, nvmlDeviceGetHandleByIndex=lambda i: ("gpu", i),
                                 nvmlDeviceGetCpuAffinity=lambda h, n: [0b00001111] + [0] * (n - 1))
    monkeypatch.setitem(sys.modules, "pynvml", fake)
    monkeypatch.setattr(os, "sched_getaffinity", lambda pid: set(allowed), raising=False)
    monkeypatch.setattr(os, "sched_setaffinity", lambda pid, cpus: calls.append(set(cpus)), raising=False)
    monkeypatch.delenv("CUDA_VISIBLE_DEVICES", raising=False)
    assert bench.bind_to_gpu_cpus(0).startswith("gpu-local (4 of 8")
    assert calls == [{0, 1, 2, 3}]
    fake.nvmlDeviceGetCpuAffinity = lambda h, n: [0xFF] + [0] * (n - 1)      # mask = everything allowed
    assert bench.bind_to_gpu_cpus(0).startswith("unchanged") and len(calls) == 1
    fake.nvmlDeviceGetCpuAffinity = lambda h, n: [0xFF00] + [0] * (n - 1)    # mask disjoint from the allowed set
    assert bench.bind_to_gpu_cpus(0).startswith("unchanged") and len(calls) == 1

    def broken(h, n):
        raise RuntimeError("no NVML")
    fake.nvmlDeviceGetCpuAffinity = broken
    assert bench.bind_to_gpu_cpus(0) == "unchanged (RuntimeError)"
