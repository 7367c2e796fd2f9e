#!/usr/bin/env python
"""Benchmark of the fully-connected hot path (fused Llama MLP) on B200, one JSON line on stdout.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--M rows] [--workload name]

Workloads (synthetic, seeded; shapes from the reference's own benchmark configuration list):
  llama7b_mlp   x[M,4096] ~N(0,1), W_gate/W_up [11008,4096], W_down [4096,11008] ~N(0,0.02), bf16, fp32 accumulate,
                bf16 output.  Default at 1 GPU with M = 2048 (prefill-shaped, tensor-core bound).
  llama70b_mlp  hidden 8192, intermediate 28672, M = 4096, tensor-parallel over N GPUs (gate/up column split, down
                row split, one all-reduce on the output: inside the down-projection kernel when torch symmetric
                memory offers an NVLink multicast mapping, else NCCL; --tp-mode).  Default when N > 1; strong scaling.
A step is one MLP forward over one batch.  value = 6*M*H*I flops / time, whole job.  Weights (>= 270 MB) exceed the
126 MB L2, so every step streams them from HBM again.

The line also carries: e2e (the same step through the host-buffer C-ABI call, pinned host x in, host out back),
roofline of the dominant kernel (gate/up GEMM, timed live with CUDA events), a decode-shaped leg (M = 1, weight
stream GB/s), the CPU baseline (the reference's own AMX kernels on the host cores when the CPU has AMX, else the
plain C++ oracle port), clocks sampled during the timed region, and the number of kernels this library launched.

--impl reference times only the CPU arm (reference AMX code or port) on the same configuration.
"""
import argparse
import ctypes
import datetime
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "FC TFLOP/s (prefill) & weight-stream GB/s (decode) vs B200 roofline"
WORKLOADS = {
    "llama7b_mlp": dict(H=4096, I=11008, M=2048),
    "llama70b_mlp": dict(H=8192, I=28672, M=4096),
}
# DRAM traffic of one gate/up GEMM launch (dram__bytes_read.sum + dram__bytes_write.sum), from the ncu capture
# summarised in the profiles/ file named beside it; None where no capture exists for the workload.
NCU_TRAFFIC_BYTES = {"llama7b_mlp": 233.73e6, "llama70b_mlp": None}  # profiles/gemm_tc2_kernel_llama7b_mlp_M2048.md


_REAL_STDOUT = None


def claim_stdout():
    """The contract is ONE JSON line on stdout, but native libraries write to file descriptor 1 too (NCCL prints its
    version there).  Keep a private duplicate of the real stdout for the JSON line and point descriptor 1 at stderr
    for everything else."""
    global _REAL_STDOUT
    if _REAL_STDOUT is None:
        sys.stdout.flush()
        _REAL_STDOUT = os.dup(1)
        os.dup2(2, 1)


def emit(line):
    data = (json.dumps(line) + "\n").encode()
    if _REAL_STDOUT is None:
        sys.stdout.write(data.decode()); sys.stdout.flush()
    else:
        os.write(_REAL_STDOUT, data)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], bf16_burst=p["bf16_tflops"], bf16_sustained=p["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16_burst=1590.0, bf16_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi.  The process is started before the warm-up (it needs
    tens of milliseconds to produce its first line) and every line carries nvidia-smi's own timestamp; the summary
    uses the samples that fall inside the timed region, marked with begin() / end()."""
    Q = ("timestamp,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []
        self.t0 = self.t1 = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "20"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def begin(self):
        self.t0 = datetime.datetime.now()

    def end(self):
        self.t1 = datetime.datetime.now()

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.03)   # let the sample that covers the end of the region arrive
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        return summarise_clock_lines(self.lines, self.t0, self.t1)


def summarise_clock_lines(lines, t0, t1):
    """lines: 'YYYY/MM/DD HH:MM:SS.mmm, sm MHz, max MHz, 4 x Active|Not Active'.  Samples stamped inside [t0, t1] (one
    sampling period of slack) are used; if none is, the last lines read (sampling stops right after the region); if the
    timestamps cannot be read, all samples."""
    rows = []
    for ln in lines:
        f = [x.strip() for x in ln.split(",")]
        if len(f) < 7:
            continue
        try:
            mhz, mx = float(f[1]), float(f[2])
        except ValueError:
            continue
        try:
            ts = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f")
        except ValueError:
            ts = None
        rows.append((ts, mhz, mx, [n for n, v in zip(ClockSampler.NAMES, f[3:7]) if v.lower().startswith("active")]))
    window = "all samples"
    if rows and t0 is not None and t1 is not None and all(r[0] is not None for r in rows):
        slack = datetime.timedelta(milliseconds=20)
        inside = [r for r in rows if t0 - slack <= r[0] <= t1 + slack]
        if inside:
            rows, window = inside, "timed region"
        else:
            # no stamp inside the region (clock or time-zone mismatch between nvidia-smi and this process): sampling
            # stops right after the region, so the last lines read are the ones that cover it
            n = max(2, int((t1 - t0).total_seconds() / 0.02) + 1)
            rows, window = rows[-n:], "last samples before the end of the timed region"
    mhz = sorted(r[1] for r in rows)
    reasons = sorted({n for r in rows for n in r[3]})
    return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": rows[-1][2] if rows else None,
            "samples": len(mhz), "window": window, "reasons": reasons}


def flops_of(w, M):
    return 6.0 * M * w["H"] * w["I"]


def weight_bytes(w):
    return 3.0 * w["H"] * w["I"] * 2


# ------------------------------------------------------------------------------------------------ CPU arm
def cpu_arm(w, M, budget_s=20.0, min_reps=1):
    """Times the CPU implementation of the same MLP on the host cores.  Returns (seconds per full step, info)."""
    import numpy as np
    from oracle import ref as oref
    from oracle._common import bf16_bits
    H, I = w["H"], w["I"]
    rng = np.random.default_rng(1001)

    def gen(shape, std):
        out = np.empty(shape, np.uint16)
        rows = max(1, (1 << 22) // shape[1])
        for r0 in range(0, shape[0], rows):
            blk = rng.standard_normal((min(rows, shape[0] - r0), shape[1]), dtype=np.float32) * np.float32(std)
            out[r0:r0 + blk.shape[0]] = bf16_bits(blk)
        return out

    if oref.available():
        nthr = os.cpu_count() or 1
        gate, up, down = gen((I, H), 0.02), gen((I, H), 0.02), gen((H, I), 0.02)
        mlp = oref.MLP(gate, up, down, nthr=nthr)
        x = gen((M, H), 1.0)
        t0 = time.perf_counter(); mlp.run(x); first = time.perf_counter() - t0   # packs the weights (constB)
        reps, t_acc = 0, 0.0
        while reps < min_reps or (t_acc < budget_s and reps < 50):
            t0 = time.perf_counter(); mlp.run(x); t_acc += time.perf_counter() - t0; reps += 1
        sec = t_acc / reps
        info = dict(kind="reference", cores=nthr,
                    sample="full workload M=%d, %d repeats after one packing run (%.1f s); reference AMX Matmul + "
                           "restated SiLU / split-K down on %d threads" % (M, reps, first, nthr))
        return sec, info
    # no AMX (or shim not built): the plain C++ port on a reduced number of rows, scaled to the full batch
    from oracle import port
    Ms = min(M, 16)
    gate, up, down = gen((I, H), 0.02), gen((I, H), 0.02), gen((H, I), 0.02)
    x = gen((Ms, H), 1.0)
    t0 = time.perf_counter(); port.mlp(x, gate, up, down); sec_s = time.perf_counter() - t0
    sec = sec_s * (M / Ms)
    info = dict(kind="port", cores=port.threads(),
                sample="oracle C++ port (no AMX on this host) on %d of %d rows, time scaled by %.0fx" % (Ms, M, M / Ms))
    return sec, info


def run_reference(args, w, M, name):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sec, info = cpu_arm(w, M, budget_s=12.0 * max(1, args.steps) / 10.0, min_reps=max(1, min(args.steps, 3)))
    val = flops_of(w, M) / sec / 1e12
    info["value"] = val; info["unit"] = "TFLOP/s"
    line = {"impl": "reference", "metric": METRIC, "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
            "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": name, "M": M, "hidden": w["H"], "intermediate": w["I"],
                       "cold": "weights larger than last-level cache"},
            "cpu_baseline": info,
            "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    emit(line)


# ------------------------------------------------------------------------------------------------ GPU arm
def run_ours(args, w, M, name):
    import torch
    import torch.distributed as dist
    from mm_amx_b200 import capi, tp

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    capi.lib()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()     # long before the timed region: the synthetic weights are created and packed meanwhile
    H, I = w["H"], w["I"]
    Is = I // world
    stream = torch.cuda.current_stream().cuda_stream
    peaks = measured_peaks()

    g = torch.Generator(device=dev); g.manual_seed(1001 + rank)
    def randn(shape, std):
        return (torch.randn(shape, generator=g, device=dev, dtype=torch.float32) * std).to(torch.bfloat16)
    # this rank's shard, generated in place (synthetic weights need no global consistency)
    gate, up, down = randn((Is, H), 0.02), randn((Is, H), 0.02), randn((H, Is), 0.02)
    gx = torch.Generator(device=dev); gx.manual_seed(7)
    x = (torch.randn((M, H), generator=gx, device=dev, dtype=torch.float32)).to(torch.bfloat16)
    mlp = capi.Mlp(gate.data_ptr(), up.data_ptr(), down.data_ptr(), H, Is, 0, 1, stream)
    del gate, up, down
    mlp.reserve(M)
    out = torch.empty((M, H), dtype=torch.bfloat16, device=dev)

    if world == 1:
        def step():
            mlp.run(x.data_ptr(), H * 2, M, out.data_ptr(), H * 2, stream)
    else:
        class Local:
            def run_partial(self, xx, oo):
                dt = capi.F32 if oo.dtype == torch.float32 else capi.BF16
                mlp.run_partial(xx.data_ptr(), H * 2, xx.shape[0], oo.data_ptr(), dt, oo.stride(0) * oo.element_size(),
                                torch.cuda.current_stream().cuda_stream)

            def gate_up(self, xx):
                mlp.gate_up(xx.data_ptr(), H * 2, xx.shape[0], torch.cuda.current_stream().cuda_stream)

            def down_rows(self, row0, rows, oo):
                dt = capi.F32 if oo.dtype == torch.float32 else capi.BF16
                mlp.down_rows(row0, rows, oo.data_ptr(), dt, oo.stride(0) * oo.element_size(),
                              torch.cuda.current_stream().cuda_stream)
        mode = args.tp_mode
        if mode == "auto":
            # the in-kernel pull all-reduce needs symmetric memory with an NVLink multicast mapping on every rank
            try:
                pull = tp.PullFusedTensorParallelMLP(mlp, H, M, comm_sms=args.comm_sms)
                ok = 1
            except Exception as ex:  # noqa: BLE001 - any failure means "not available here"
                sys.stderr.write("rank %d: pull all-reduce unavailable (%s); using NCCL\n" % (rank, ex))
                pull, ok = None, 0
            t_ok = torch.tensor([ok], device=dev)
            dist.all_reduce(t_ok, op=dist.ReduceOp.MIN)
            mode = "pull" if int(t_ok.item()) == 1 else "nccl"
        elif mode == "pull":
            pull = tp.PullFusedTensorParallelMLP(mlp, H, M, comm_sms=args.comm_sms)
        args.tp_mode = mode
        if mode == "fused":
            fused = tp.FusedTensorParallelMLP(mlp, H, M)
            def step():
                return fused.forward(x)
        elif mode == "pull":
            def step():
                return pull.forward(x)
        else:
            tpm = tp.TensorParallelMLP(Local(), H, partial_dtype=torch.bfloat16, chunk_rows=args.chunk_rows)
            def step():
                return tpm.forward(x, out)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    l0 = capi.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    sampler.begin()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    sampler.end()
    launches = capi.launch_count() - l0
    ms = e0.elapsed_time(e1) / args.steps
    capi.sync_check(stream)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        lt = torch.tensor([launches], device=dev, dtype=torch.int64)
        dist.all_reduce(lt)
        launches = int(lt.item())
    clocks = sampler.stop() if rank == 0 else None
    value = flops_of(w, M) / (ms * 1e-3) / 1e12

    # ---- dominant kernel alone: gate/up GEMM of this rank, K launches back to back (sustained regime) ----
    roofline = None
    for _ in range(3 if "kernel" in args.legs else 0):
        mlp.gate_up(x.data_ptr(), H * 2, M, stream)
    if "kernel" in args.legs:
      torch.cuda.synchronize()
      k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
      k0.record()
      for _ in range(args.steps):
        mlp.gate_up(x.data_ptr(), H * 2, M, stream)
      k1.record(); torch.cuda.synchronize()
      k_ms = k0.elapsed_time(k1) / args.steps
      k_flops = 4.0 * M * H * Is
      achieved = k_flops / (k_ms * 1e-3) / 1e12
      roofline = {"kernel": "gemm_tc2_kernel (gate/up projection + SiLU*up epilogue)", "bound": "tensor",
                "achieved": achieved, "peak": peaks["bf16_burst"], "unit": "TFLOP/s",
                "frac": achieved / peaks["bf16_burst"],
                "peak_source": peaks["source"] + " (cuBLAS bf16 burst figure: the kernel is timed alone, in a loop "
                                                 "far shorter than the power-cap time constant)",
                "frac_of_sustained_peak": achieved / peaks["bf16_sustained"], "us_per_launch": k_ms * 1e3,
                "flops_per_launch": k_flops, "traffic": NCU_TRAFFIC_BYTES.get(name)}

    line = {"metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": name, "M": M, "hidden": H, "intermediate": I,
                       "parallelism": ("tp%d (%s all-reduce)" % (world, args.tp_mode)) if world > 1 else "single GPU",
                       "cold": "weights (%.0f MB per GPU) larger than the 126 MB L2" % (weight_bytes(w) / world / 1e6)},
            "gpu_launches": launches, "roofline": roofline}

    if rank == 0:
        line["clocks"] = clocks

    # ---- end to end through the host-buffer entry point (1 GPU) / host x in + host out back (N GPUs) ----
    if "e2e" in args.legs:
        xh = torch.empty((M, H), dtype=torch.bfloat16).pin_memory(); xh.copy_(x.cpu())
        oh = torch.empty((M, H), dtype=torch.bfloat16).pin_memory()
        if world == 1:
            def e2e_step():
                mlp.run_host(xh.data_ptr(), H * 2, M, oh.data_ptr(), H * 2, stream)
        else:
            def e2e_step():
                x.copy_(xh, non_blocking=True)
                oh.copy_(step(), non_blocking=True)
                torch.cuda.current_stream().synchronize()
        for _ in range(3):
            e2e_step()
        barrier()
        e0.record()
        for _ in range(args.steps):
            e2e_step()
        e1.record()
        barrier()
        e_ms = e0.elapsed_time(e1) / args.steps
        if world > 1:
            t = torch.tensor([e_ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e_ms = float(t.item())
        line["e2e"] = {"value": flops_of(w, M) / (e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e_ms,
                       "h2d_bytes_per_step": M * H * 2 * world, "d2h_bytes_per_step": M * H * 2 * world,
                       "api": "b200fc_mlp_run_host (pinned host buffers)" if world == 1 else
                              "host x -> device, tensor-parallel forward, device out -> host, per rank"}

    # ---- decode-shaped leg: M = 1, the weight stream in GB/s against the measured HBM copy bandwidth ----
    if world == 1 and "decode" in args.legs:
        x1 = x[:1].contiguous()
        o1 = torch.empty((1, H), dtype=torch.bfloat16, device=dev)
        def dstep():
            mlp.run(x1.data_ptr(), H * 2, 1, o1.data_ptr(), H * 2, stream)
        for _ in range(5):
            dstep()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        reps = 20
        try:
            with torch.cuda.graph(graph):
                s2 = torch.cuda.current_stream().cuda_stream
                for _ in range(reps):
                    mlp.run(x1.data_ptr(), H * 2, 1, o1.data_ptr(), H * 2, s2)
            graph.replay(); torch.cuda.synchronize()
            e0.record(); graph.replay(); e1.record(); torch.cuda.synchronize()
            d_ms = e0.elapsed_time(e1) / reps
            how = "CUDA graph of %d forwards" % reps
        except Exception as ex:  # graph capture unavailable: plain launches
            torch.cuda.synchronize()
            e0.record()
            for _ in range(reps):
                dstep()
            e1.record(); torch.cuda.synchronize()
            d_ms = e0.elapsed_time(e1) / reps
            how = "plain launches (%s)" % type(ex).__name__
        gbs = weight_bytes(w) / (d_ms * 1e-3) / 1e9
        line["decode"] = {"M": 1, "value": gbs, "unit": "GB/s", "us_per_step": d_ms * 1e3, "timing": how,
                          "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                       "frac": gbs / peaks["hbm_gbs"], "peak_source": peaks["source"]}}

    # ---- the other single-GPU configurations of the reference's list, as extra keys (not the headline) ----
    if world == 1 and "configs" in args.legs:
        line["other_configs"] = other_configs(torch, capi, dev, peaks)

    # ---- CPU baseline beside it (rank 0, 1 GPU only) ----
    if rank == 0 and world == 1 and "cpu" in args.legs:
        try:
            sec, info = cpu_arm(w, M, budget_s=15.0)
            info["value"] = flops_of(w, M) / sec / 1e12; info["unit"] = "TFLOP/s"
            line["cpu_baseline"] = info
        except Exception as ex:
            line["cpu_baseline"] = {"value": None, "unit": "TFLOP/s", "cores": 0, "kind": "port",
                                    "sample": "failed: %s" % ex}
    if rank == 0:
        emit(line)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def other_configs(torch, capi, dev, peaks):
    """Single bf16 Linear (M=256, +bias, fp32 out), int8-weight decode GEMV (K=4096, N in {4096, 11008}, M in
    {1, 4, 16}), int8 GEMM 2048x4096x4096 with quantised post-ops.  Each case rotates over enough independently packed
    weight sets to exceed L2 several times and is timed as one CUDA graph (kernels of a few microseconds)."""
    out = {}
    side = torch.cuda.Stream()
    g = torch.Generator(device=dev); g.manual_seed(1002)

    def timed_graph(launch_all, n_launch, reps=5):
        with torch.cuda.stream(side):
            s = side.cuda_stream
            launch_all(s); side.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                launch_all(torch.cuda.current_stream().cuda_stream)
            graph.replay(); torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                graph.replay()
            e1.record(); torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e-3 / reps / n_launch

    # config 1: A[256,4096] x B[4096,4096] + bias -> fp32
    M, K, N = 256, 4096, 4096
    A = (torch.rand((M, K), generator=g, device=dev) * 2 - 1).to(torch.bfloat16)
    bias = torch.randn(N, generator=g, device=dev)
    C = torch.empty((M, N), dtype=torch.float32, device=dev)
    ws = []
    for _ in range(16):
        B = (torch.rand((K, N), generator=g, device=dev) * 2 - 1).to(torch.bfloat16)
        ws.append(capi.Weight(B.data_ptr(), capi.BF16, K, N, N * 2, False)); del B
    ep = capi.make_epilogue(C.data_ptr(), N * 4, capi.F32, capi.STEP_BIAS, bias.data_ptr())
    t = timed_graph(lambda s: [w.matmul(A.data_ptr(), capi.BF16, M, K, K * 2, ep, stream=s) for w in ws], len(ws))
    nbytes = M * K * 2 + K * N * 2 + M * N * 4 + N * 4
    out["bf16_linear_256x4096x4096_bias_f32"] = {"us": t * 1e6, "tflops": 2.0 * M * K * N / t / 1e12,
                                                   "gbs": nbytes / t / 1e9, "hbm_frac": nbytes / t / 1e9 / peaks["hbm_gbs"],
                                                   "weight_sets": len(ws)}
    del ws
    # config 3: int8-weight decode GEMV
    K = 4096
    for N in (4096, 11008):
        nset = int(600e6 / (K * N)) + 1
        ws, keep = [], []
        for _ in range(nset):
            B = torch.randint(-127, 128, (N, K), dtype=torch.int8, device=dev, generator=g)
            sc = torch.rand(N, generator=g, device=dev) * 0.019 + 0.001
            ws.append(capi.Weight(B.data_ptr(), capi.S8, K, N, K, True, capi.PACK_INT8_CHANNEL, sc.data_ptr())); del B
        for M in (1, 4, 16):
            x = torch.randn((M, K), generator=g, device=dev).to(torch.bfloat16)
            C = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
            ep = capi.make_epilogue(C.data_ptr(), N * 2, capi.BF16, capi.STEP_DEQUANT)
            t = timed_graph(lambda s: [w.matmul(x.data_ptr(), capi.BF16, M, K, K * 2, ep, stream=s) for w in ws], nset)
            nbytes = K * N + N * 4 + M * (K + N) * 2
            out["int8w_gemv_M%d_4096x%d" % (M, N)] = {"us": t * 1e6, "gbs": nbytes / t / 1e9,
                                                      "hbm_frac": nbytes / t / 1e9 / peaks["hbm_gbs"], "weight_sets": nset}
        del ws
    # config 4: int8 x int8 GEMM with quantised post-ops
    M, K, N = 2048, 4096, 4096
    A = torch.randint(-128, 128, (M, K), dtype=torch.int8, device=dev, generator=g)
    ws = []
    for _ in range(8):
        B = torch.randint(-128, 128, (K, N), dtype=torch.int8, device=dev, generator=g)
        ws.append(capi.Weight(B.data_ptr(), capi.S8, K, N, N, False)); del B
    sB = torch.rand(N, generator=g, device=dev) * 0.049 + 0.001
    bias = torch.randn(N, generator=g, device=dev)
    C32 = torch.empty((M, N), dtype=torch.int32, device=dev)
    Cf = torch.empty((M, N), dtype=torch.float32, device=dev)
    C8 = torch.empty((M, N), dtype=torch.int8, device=dev)
    cases = {
        "raw_int32": capi.make_epilogue(C32.data_ptr(), N * 4, capi.S32),
        "dequant_bias_f32": capi.make_epilogue(Cf.data_ptr(), N * 4, capi.F32, capi.STEP_DEQUANT | capi.STEP_BIAS,
                                               bias.data_ptr(), 0.02, sB.data_ptr()),
        "dequant_bias_requant_s8": capi.make_epilogue(C8.data_ptr(), N, capi.S8,
                                                      capi.STEP_DEQUANT | capi.STEP_BIAS | capi.STEP_QUANT,
                                                      bias.data_ptr(), 0.02, sB.data_ptr(), 0.05),
    }
    for name, ep in cases.items():
        t = timed_graph(lambda s: [w.matmul(A.data_ptr(), capi.S8, M, K, K, ep, stream=s) for w in ws], len(ws))
        out["int8_gemm_2048x4096x4096_" + name] = {"us": t * 1e6, "tops": 2.0 * M * K * N / t / 1e12}
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, choices=[None] + list(WORKLOADS))
    ap.add_argument("--M", type=int, default=None)
    ap.add_argument("--chunk-rows", type=int, default=2048)
    ap.add_argument("--tp-mode", default="auto", choices=["auto", "nccl", "fused", "pull"],
                    help="N > 1: 'pull' = all-reduce inside the down-projection kernel (multimem.ld_reduce / multimem.st "
                         "by reducing CTAs), 'nccl' = NCCL all-reduce in row chunks overlapping the GEMMs, 'fused' = "
                         "in-switch reduction from the down-projection epilogue (multimem.red); 'auto' = pull when "
                         "symmetric memory with multicast is available, else nccl")
    ap.add_argument("--comm-sms", type=int, default=8, help="SMs reserved for the reduction in 'pull' mode")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--legs", default="kernel,e2e,decode,configs,cpu",
                    help="optional legs after the main timed loop (comma list of kernel,e2e,decode,configs,cpu; '' = none)")
    args = ap.parse_args()
    claim_stdout()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        args.gpus = world
    args.legs = set(x for x in args.legs.split(",") if x)
    if args.no_cpu:
        args.legs.discard("cpu")
    name = args.workload or ("llama7b_mlp" if args.gpus == 1 else "llama70b_mlp")
    w = WORKLOADS[name]
    M = args.M or w["M"]
    if args.impl == "reference":
        run_reference(args, w, M, name)
    else:
        run_ours(args, w, M, name)


if __name__ == "__main__":
    main()
