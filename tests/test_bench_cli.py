"""CPU: bench.py's command line without a GPU — the reference arm prints exactly one JSON line with the contract's
keys, and the GPU arm fails loudly instead of falling back to anything."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_bench(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                          timeout=900, cwd=ROOT)


def test_reference_arm_prints_one_json_line():
    r = run_bench("--impl", "reference", "--steps", "1", "--warmup", "1", "--M", "16", "--workload", "llama7b_mlp")
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.strip()]
    assert len(lines) == 1, r.stdout[:500]
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["n_gpus"] == 1 and d["higher_is_better"] is True
    for key in ("metric", "value", "unit", "steps", "warmup", "ms_per_step", "scaling", "vs_baseline", "dtype", "data",
                "config", "cpu_baseline", "e2e"):
        assert key in d, key
    assert d["config"]["workload"] == "llama7b_mlp" and d["config"]["M"] == 16
    assert d["cpu_baseline"]["kind"] in ("reference", "port") and d["cpu_baseline"]["cores"] >= 1
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0
    assert d["value"] > 0 and d["scaling"] == "strong"


def test_default_workload_is_the_same_at_every_gpu_count():
    import importlib.util
    spec = importlib.util.spec_from_file_location("bench_module_cli", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    assert bench.DEFAULT_WORKLOAD == "llama70b_mlp"
    w = bench.WORKLOADS[bench.DEFAULT_WORKLOAD]
    assert (w["H"], w["I"], w["M"]) == (8192, 28672, 4096)
    for world in (1, 2, 4, 8):
        assert w["I"] % world == 0 and (w["I"] // world) % 32 == 0 and w["M"] % world == 0
    a = bench.host_normal_bf16((37, 64), 0.02, 5)
    assert a.shape == (37, 64) and (a == bench.host_normal_bf16((37, 64), 0.02, 5)).all()


def test_gpu_arm_fails_loudly_without_a_gpu():
    import torch
    if torch.cuda.is_available():
        return   # on a GPU box the arm runs; the GPU suite and the driver cover it
    r = run_bench("--steps", "1", "--warmup", "1", "--no-cpu")
    assert r.returncode != 0
    assert r.stdout.strip() == ""          # no result line from a run that computed nothing
