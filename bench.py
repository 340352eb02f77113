#!/usr/bin/env python
"""Benchmark of the causal self-attention hot path (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one forward + backward pass of the attention layer over one batch of synthetic
input.  The workload is the GPT-2 124M block shape the metric is quoted on: B=8, T=1024, H=12,
D=64, fp32 in/out, qkv and dout i.i.d. N(0,1) from a fixed seed.  With N > 1 (launched through
torch.distributed.run, one rank per GPU) every rank processes its own batch of 8 for the headline
value (weak scaling: the (batch, head) units are independent, there is no collective on the data
path); the same line also carries a strong-scaling block in which ONE fixed workload is cut into
contiguous batch slices, one per rank.

Printed JSON line (rank 0):
  value      whole-job algorithmic TFLOP/s (6*B*H*T^2*D / 2 per pass, causal count) with inputs
             resident in HBM, CUDA-event time, max over ranks; the K-step timed loop is repeated
             `repeats` times and value / ms_per_step are the median repeat (min and max beside it)
  e2e        the same metric through the C ABI with pinned HOST buffers: the H2D copy of qkv and
             dout and the D2H copy of out and dqkv are inside the timed region, every step; upload,
             kernels and download run on three event-chained streams so consecutive steps overlap.
             e2e.copy_only is the same loop with the kernel calls left out: what the copies alone cost
  stage_us   launch duration of each of the four kernels, from a second pass over the same K steps
             with an event between the kernels (those events idle the GPU for a few microseconds
             each, so the headline pass runs without them)
  graph      the same K steps replayed from CUDA graphs (one per buffer set): no host in the loop
  roofline   the dominant kernel (backward core) timed live with CUDA events, against the measured
             burst cuBLAS bf16 rate (the kernel is timed in a millisecond burst)
  cpu_baseline  the reference's own CPU attention (OpenBLAS) on this box's host cores, rank 0, N=1
  gpu_baseline  the reference's own CUDA attention (cuBLAS TF32 + SIMT kernels compiled for sm_100a,
             unchanged) through its layer API on this GPU, and this repository's kernels through the
             same layer API (allocation included), rank 0, N=1
  train      GPT-2 124M training step through the unchanged train_gpt (12 layers, B=8, T=1024) with the
             reference's kernels and with this repository's: ms per step and tokens/s, rank 0, N=1
  strong     N > 1 (and N = 1 for the single-GPU time): GPT-2 XL shape B=64 H=25 forward+backward and
             GPT-2 medium shape B=32 H=16 forward only, generated per batch entry from the seed, cut
             into contiguous batch slices; per-rank kernel time (max over ranks), aggregate TFLOP/s
             and efficiency against the whole workload on one GPU measured in the same run

--impl reference times the reference's own CPU implementation of the path (compiled out of tree
into oracle/_ref, else the plain-C port in oracle/) on the host cores, one full B=8 pass per step,
and prints the same line with "impl": "reference".
"""
from __future__ import annotations

import argparse
import json
import os
import re
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# The default is the configuration the metric is quoted on; the others are the remaining shapes of the
# reference's configuration list, selectable with --workload for per-configuration tables.
WORKLOADS = {
    "gpt2-124M-T1024": {"B": 8, "T": 1024, "H": 12, "D": 64, "backward": True},     # the benchmark line
    "gpt2-124M-T128": {"B": 8, "T": 128, "H": 12, "D": 64, "backward": True},
    "gpt2-medium-fwd": {"B": 32, "T": 1024, "H": 16, "D": 64, "backward": False},   # forward only
    "gpt2-xl-B64": {"B": 64, "T": 1024, "H": 25, "D": 64, "backward": True},
}
DEFAULT_WORKLOAD = "gpt2-124M-T1024"
STRONG_WORKLOADS = ("gpt2-xl-B64", "gpt2-medium-fwd")  # cut over the ranks in the strong-scaling block
WORKLOAD = dict(WORKLOADS[DEFAULT_WORKLOAD])
SEED = 1234
METRIC = "attn fwd+bwd TFLOP/s"
UNIT = "TFLOP/s"
NOMINAL_BF16_TFLOPS = 2250.0
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
ROTATE = 4  # buffer sets cycled through so that a set is evicted from L2 before it is reused
REPEATS = 10  # the K-step timed loop is run this many times; median and range are reported
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the backward core kernel on the bench
# workload as captured with ncu (profiles/): shown for reference, never as this run's measurement
BWD_CORE_DRAM_BYTES_PROFILED = {"bytes": 193467136, "source": "profiles/ncu_full_attention_B8_T1024_H12.txt"}
REF_GPTC = os.path.join(ROOT, "oracle", "_ref", "gptc_reference")
OUR_GPTC = os.path.join(ROOT, "gpt.c_b200", "overlay", "_build", "gptc_overlay")


def flops_fwd(B, T, H, D):
    return 2.0 * B * H * T * T * D


def flops_bwd(B, T, H, D):
    return 4.0 * B * H * T * T * D


def algorithmic_bytes(B, T, H, D):
    C = H * D
    return {"fwd": 16.0 * B * T * C + 4.0 * B * H * T, "bwd": 32.0 * B * T * C + 4.0 * B * H * T}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {k: float(p[k]) for k in FALLBACK_PEAKS if k in p} | {"source": "measured"}
    return dict(FALLBACK_PEAKS) | {"source": "fallback"}


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.002):
        super().__init__(daemon=True)
        self.index, self.period = index, period_s
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop_evt = threading.Event()
        self.ok = False
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:  # NVML missing: report nulls rather than fail the bench
            self.ok = False

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
            "hw_power_brake": getattr(nv, "nvmlClocksEventReasonHwPowerBrakeSlowdown", 0x80),
        }
        while not self._stop_evt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(self.period)

    def stop(self):
        self._stop_evt.set()
        self.join(timeout=1.0)
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def physical_gpu_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except (ValueError, IndexError):
            return local_rank
    return local_rank


def seeded_host_inputs(rank: int, batch: int | None = None):
    import numpy as np

    B, T, H, D = (WORKLOAD[k] for k in "BTHD")
    if batch is not None:
        B = min(B, batch)
    rng = np.random.default_rng(SEED + rank)
    x = rng.standard_normal((B, T, 3 * H * D), dtype=np.float32)
    g = rng.standard_normal((B, T, H * D), dtype=np.float32)
    return x, g


# ------------------------------------------------------------------------------------------------
# reference arm and CPU baseline (host cores only)
# ------------------------------------------------------------------------------------------------
def cpu_attention_runner():
    """Returns (kind, run(x, g, H) -> seconds, info)."""
    from oracle import build as oracle_build
    from oracle import oracle

    cores = os.cpu_count() or 1
    if oracle.have_reference():
        def run(x, g, H):
            t0 = time.perf_counter()
            oracle.reference_run(x, g, H, threads=cores)
            return time.perf_counter() - t0

        info = oracle.reference_info()
        return "reference", run, {"cores": cores, "blas": info["blas"]}
    oracle_build.build_oracle()

    def run(x, g, H):
        t0 = time.perf_counter()
        oracle.forward(x, H)
        oracle.backward(x, g, H)
        return time.perf_counter() - t0

    return "port", run, {"cores": oracle.num_threads(), "blas": None}


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return  # rank 0 alone measures the host cores
    B, T, H, D = (WORKLOAD[k] for k in "BTHD")
    with_bwd = WORKLOAD["backward"]
    x, g = seeded_host_inputs(0)  # the whole batch, every step: the same workload as our arm
    kind, run, info = cpu_attention_runner()
    for _ in range(args.warmup):
        run(x, g, H)
    times = [run(x, g, H) for _ in range(args.steps)]
    total = sum(times)
    fl = (flops_fwd(B, T, H, D) + (flops_bwd(B, T, H, D) if with_bwd else 0.0)) * args.steps
    value = fl / total / 1e12
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": total / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"causal attention fwd+bwd, fused qkv [B,T,3C] fp32 io, B={B} T={T} H={H} D={D} per GPU",
                   "name": args.workload, "global_batch": B, "seq_len": T, "n_heads": H, "head_dim": D, "seed": SEED},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": info["cores"], "kind": kind,
                         "sample": f"the full workload (all {B} batch entries) per step, fwd+bwd, {args.steps} steps",
                         "blas": info["blas"]},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def measure_cpu_baseline():
    B, T, H, D = (WORKLOAD[k] for k in "BTHD")
    sample_b = min(B, 8)  # bounded: the largest configurations would take minutes on the host
    x, g = seeded_host_inputs(0, sample_b)
    kind, run, info = cpu_attention_runner()
    secs = run(x, g, H)  # forward + backward of the sample (the CPU kernels are timed as a pair)
    fl = flops_fwd(sample_b, T, H, D) + flops_bwd(sample_b, T, H, D)
    what = "the full workload" if sample_b == B else f"{sample_b} of {B} batch entries"
    return {"value": fl / secs / 1e12, "unit": UNIT, "cores": info["cores"], "kind": kind,
            "sample": f"one fwd+bwd pass of {what} (B={sample_b}), {secs:.2f} s", "blas": info["blas"]}


# ------------------------------------------------------------------------------------------------
# GPU baselines through gpt.c's own executables (rank 0, N=1)
# ------------------------------------------------------------------------------------------------
def measure_gpu_baseline(pairs: int = 10):
    """The attention layer of gpt.c driven through its public API (include/attention.h) by the layer driver:
    the unmodified reference build (its cuBLAS TF32 + SIMT attention, kernels/src/cuda/Attention.cu:170-324)
    and this repository's build, same inputs, wall time per forward+backward pair with the allocations the
    layer makes; `pooled` repeats the measurement with the default memory pool kept (see layer_driver.c)."""
    import numpy as np

    B, T, H, D = (WORKLOAD[k] for k in "BTHD")
    C = H * D
    out = {"unit": "ms per forward+backward pair through the layer API", "pairs": pairs,
           "config": f"B={B} T={T} H={H} D={D}"}
    exes = {"reference_cuda": os.path.join(REF_GPTC, "layer_driver"), "this_repo": os.path.join(OUR_GPTC, "layer_driver")}
    missing = [k for k, e in exes.items() if not os.path.exists(e)]
    if missing:
        return {"unavailable": f"layer_driver builds missing: {missing}"}
    with tempfile.TemporaryDirectory() as tmp:
        x, g = seeded_host_inputs(0)
        x.tofile(os.path.join(tmp, "x.bin"))
        g.tofile(os.path.join(tmp, "g.bin"))
        for name, exe in exes.items():
            for mode in ("as_shipped", "pooled"):
                cmd = [exe, "cuda", str(B), str(T), str(C), str(H), os.path.join(tmp, "x.bin"), os.path.join(tmp, "g.bin"),
                       os.path.join(tmp, "o.bin"), os.path.join(tmp, "dx.bin"), str(pairs)]
                if mode == "pooled":
                    cmd.append("keep-pool")
                try:
                    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
                    m = re.search(r"mean_ms=([\d.]+)", res.stdout)
                    out.setdefault(name, {})[mode] = float(m.group(1)) if (res.returncode == 0 and m) else None
                    if res.returncode != 0 or not m:
                        out[name][mode + "_error"] = (res.stdout + res.stderr)[-300:]
                except Exception as e:  # a missing CUDA runtime for keep-pool, a timeout: report, do not fail the bench
                    out.setdefault(name, {})[mode] = None
                    out[name][mode + "_error"] = repr(e)[:300]
    fl = flops_fwd(B, T, H, D) + flops_bwd(B, T, H, D)
    for name in exes:
        ms = out.get(name, {}).get("pooled")
        if ms:
            out[name]["tflops_pooled"] = fl / (ms * 1e-3) / 1e12
    out["kernel_time_profiled"] = {"reference_cuda_us_per_pair": 2907.0,
                                   "source": "profiles/reference_cuda_attention_layer_B8_T1024_H12.txt (ncu launch list)"}
    return out


def measure_train(steps: int = 8):
    """Config 4: GPT-2 124M training step through the unchanged train_gpt, ms/step and tokens/s parsed from
    its stdout (train_gpt.c:517), for the unmodified reference and for this repository's build."""
    import importlib.util

    path = os.path.join(ROOT, "gpt.c_b200", "overlay", "run_train_config.py")
    spec = importlib.util.spec_from_file_location("gptc_b200_run_train_config", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    try:
        return mod.run(steps=steps)
    except Exception as e:
        return {"unavailable": repr(e)[:300]}


# ------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------
def bind_to_gpu_cpus(local_rank: int):
    """Runs this process on the CPU cores next to its GPU (what nvidia-smi topo prints as CPU affinity), so
    that the pinned host buffers of the end-to-end leg are allocated on that socket's memory: with eight ranks
    on a two-socket host, buffers on the far socket halve the copy rate.  A process setting, not a GPU one.
    Returns the number of cores bound to, or None when NVML or the call is not available."""
    try:
        import pynvml

        pynvml.nvmlInit()
        import torch

        try:  # the CUDA device's own PCI address: NVML counts all GPUs of the host, CUDA only the visible ones
            pr = torch.cuda.get_device_properties(local_rank)
            bus = "%08x:%02x:%02x.0" % (pr.pci_domain_id, pr.pci_bus_id, pr.pci_device_id)
            handle = pynvml.nvmlDeviceGetHandleByPciBusId(bus.encode())
        except Exception:
            handle = pynvml.nvmlDeviceGetHandleByIndex(local_rank)
        words = pynvml.nvmlDeviceGetCpuAffinity(handle, (os.cpu_count() + 63) // 64)
        cpus = {64 * i + b for i, w in enumerate(words) for b in range(64) if (int(w) >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
            return len(cpus)
    except Exception:
        pass
    return None


def seeded_device_entries(dev, start: int, stop: int, T: int, H: int, D: int, with_bwd: bool):
    """Batch entries [start, stop) of a fixed workload: entry b is drawn from a generator seeded with
    (SEED, b), so every rank produces exactly the entries of its slice whatever the number of ranks."""
    import torch

    C = H * D
    x = torch.empty((stop - start, T, 3 * C), device=dev)
    g = torch.empty((stop - start, T, C), device=dev) if with_bwd else None
    gen = torch.Generator(device=dev)
    for i, b in enumerate(range(start, stop)):
        gen.manual_seed(SEED * 100003 + b)
        x[i].normal_(generator=gen)
        if with_bwd:
            g[i].normal_(generator=gen)
    return x, g


def run_ours(args):
    import torch
    import torch.distributed as dist

    import __graft_entry__ as entry

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run for N > 1")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    cpu_affinity = bind_to_gpu_cpus(local_rank)

    pkg = entry.load_package()
    pkg.init()
    shard = entry.load_submodule("shard")
    B, T, H, D = (WORKLOAD[k] for k in "BTHD")
    with_bwd = WORKLOAD["backward"]
    C = H * D
    dev = torch.device("cuda", local_rank)
    xh, gh = seeded_host_inputs(rank)
    x_pin = torch.from_numpy(xh).pin_memory()
    g_pin = torch.from_numpy(gh).pin_memory()
    out_pin = torch.empty((B, T, C), dtype=torch.float32).pin_memory()
    dx_pin = torch.empty((B, T, 3 * C), dtype=torch.float32).pin_memory()

    def make_set():
        return {
            "x": x_pin.to(dev), "g": g_pin.to(dev),
            "out": torch.empty((B, T, C), device=dev), "lse": torch.empty((B, H, T), device=dev),
            "saved": torch.empty(pkg.saved_bytes(B, T, H, D), device=dev, dtype=torch.uint8),
            "scratch": torch.empty(pkg.backward_scratch_bytes(B, T, H, D), device=dev, dtype=torch.uint8),
            "dx": torch.empty((B, T, 3 * C), device=dev),
        }

    sets = [make_set()]
    set_bytes = sum(t.numel() * t.element_size() for t in sets[0].values())
    # enough sets that the others together exceed twice the L2 before one is reused
    rotate = max(ROTATE, int(2 * 126e6 // set_bytes) + 2)
    while len(sets) < rotate:
        sets.append(make_set())
    stream = torch.cuda.current_stream()

    def step(i, events=None):
        s = sets[i % rotate]
        if events is None:  # the calls a user makes: one forward, one backward
            pkg.forward_into(s["x"], s["out"], None, s["lse"], s["saved"], H)
            if with_bwd:
                pkg.backward_into(s["saved"], s["out"], s["lse"], s["g"], s["dx"], s["scratch"], H)
            return
        # staged variant: the same four kernels launched one by one with an event between them
        events[0].record(stream)
        pkg.forward_into(s["x"], s["out"], None, s["lse"], s["saved"], H, pkg.FLAG_PREPARE_ONLY)
        events[1].record(stream)
        pkg.forward_into(s["x"], s["out"], None, s["lse"], s["saved"], H, pkg.FLAG_CORE_ONLY)
        events[2].record(stream)
        if with_bwd:
            pkg.backward_into(s["saved"], s["out"], s["lse"], s["g"], s["dx"], s["scratch"], H, pkg.FLAG_PREPARE_ONLY)
        events[3].record(stream)
        if with_bwd:
            pkg.backward_into(s["saved"], s["out"], s["lse"], s["g"], s["dx"], s["scratch"], H, pkg.FLAG_CORE_ONLY)
        events[4].record(stream)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed(fn, n):
        """n calls of fn(i) between a barrier + synchronise on both sides; device time, max over ranks."""
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        a.record(stream)
        for i in range(n):
            fn(i)
        b.record(stream)
        barrier()
        return max_over_ranks(a.elapsed_time(b))

    # clock ramp (untimed, not counted as warm-up): the GPU idles at a low clock
    t_end = time.perf_counter() + (0.0 if args.no_ramp else 0.3)
    i = 0
    while time.perf_counter() < t_end:
        step(i)
        i += 1
    torch.cuda.synchronize()

    # ---------------- device-resident timed region ----------------
    for i in range(args.warmup):
        step(i)
    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    loop_ms = [timed(step, args.steps) for _ in range(args.repeats)]
    ms_total = statistics.median(loop_ms)
    # Second timed pass over the same K steps with an event between the kernels: it gives the launch
    # duration of each kernel (the roofline uses the backward core's).  The events cost a few
    # microseconds of idle GPU each, which is why the headline pass above runs without them.
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(5)] for _ in range(args.steps)]
    staged_ms_total = timed(lambda i: step(i, ev[i]), args.steps)
    clocks = sampler.stop()
    status = pkg.device_status()
    if status != 0:
        raise SystemExit(f"kernel status word {status}: a bounded wait ran out")
    stage_ms = [statistics.mean(ev[i][k].elapsed_time(ev[i][k + 1]) for i in range(args.steps)) for k in range(4)]
    stage_med = [statistics.median(ev[i][k].elapsed_time(ev[i][k + 1]) for i in range(args.steps)) for k in range(4)]

    # ---------------- optional: the same steps replayed from CUDA graphs ----------------
    # For short sequences the four launches of a step take less GPU time than the host needs to issue
    # them; one captured graph per buffer set removes the host from the loop.
    graph_info = None
    if args.graph:
        graphs = []
        side = torch.cuda.Stream()
        side.wait_stream(stream)
        with torch.cuda.stream(side):
            for k in range(rotate):
                gr = torch.cuda.CUDAGraph()
                s_k = sets[k]
                with torch.cuda.graph(gr, stream=side):
                    pkg.forward_into(s_k["x"], s_k["out"], None, s_k["lse"], s_k["saved"], H, stream=side)
                    if with_bwd:
                        pkg.backward_into(s_k["saved"], s_k["out"], s_k["lse"], s_k["g"], s_k["dx"], s_k["scratch"], H,
                                          stream=side)
                graphs.append(gr)
        stream.wait_stream(side)
        for i in range(args.warmup):
            graphs[i % rotate].replay()
        graph_ms = timed(lambda i: graphs[i % rotate].replay(), args.steps)
        if pkg.device_status() != 0:
            raise SystemExit("kernel status word set during graph replay")
        graph_info = {"ms_per_step": graph_ms / args.steps}

    # ---------------- end-to-end through the C ABI with host buffers ----------------
    # Every step copies its qkv and dout from pinned host memory, runs forward + backward through the
    # C ABI and copies out and dqkv back to pinned host memory.  The three legs run on three streams
    # chained by events, so the upload of step i+1 and the download of step i-1 overlap the kernels of
    # step i (PCIe is full duplex); a buffer set is reused only after its previous download finished.
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    in_done = [torch.cuda.Event() for _ in range(rotate)]
    comp_done = [torch.cuda.Event() for _ in range(rotate)]
    out_done = [torch.cuda.Event() for _ in range(rotate)]

    def e2e_step(i, kernels=True):
        k = i % rotate
        s = sets[k]
        with torch.cuda.stream(s_in):
            s_in.wait_event(comp_done[k])  # the kernels that last read this set's inputs
            s["x"].copy_(x_pin, non_blocking=True)
            if with_bwd:
                s["g"].copy_(g_pin, non_blocking=True)
            in_done[k].record(s_in)
        stream.wait_event(in_done[k])
        stream.wait_event(out_done[k])  # the download that last read this set's outputs
        if kernels:
            pkg.forward_into(s["x"], s["out"], None, s["lse"], s["saved"], H, stream=stream)
            if with_bwd:
                pkg.backward_into(s["saved"], s["out"], s["lse"], s["g"], s["dx"], s["scratch"], H, stream=stream)
        comp_done[k].record(stream)
        with torch.cuda.stream(s_out):
            s_out.wait_event(comp_done[k])
            out_pin.copy_(s["out"], non_blocking=True)
            if with_bwd:
                dx_pin.copy_(s["dx"], non_blocking=True)
            out_done[k].record(s_out)

    def e2e_join():
        stream.wait_stream(s_in)
        stream.wait_stream(s_out)

    def e2e_timed(kernels: bool) -> float:
        for i in range(args.warmup):
            e2e_step(i, kernels)
        e2e_join()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record(stream)
        s_in.wait_event(e0)
        for i in range(args.steps):
            e2e_step(i, kernels)
        e2e_join()
        e1.record(stream)
        barrier()
        return max_over_ranks(e0.elapsed_time(e1))

    e2e_ms = e2e_timed(True)
    e2e_copy_ms = e2e_timed(False)  # the same three streams and copies, kernel calls left out
    if pkg.device_status() != 0:
        raise SystemExit("kernel status word set during the end-to-end pass")

    flops_step = flops_fwd(B, T, H, D) + (flops_bwd(B, T, H, D) if with_bwd else 0.0)
    to_tflops = lambda total_ms: flops_step * world * args.steps / (total_ms * 1e-3) / 1e12  # noqa: E731
    value = to_tflops(ms_total)
    e2e_value = to_tflops(e2e_ms)
    h2d = x_pin.numel() * 4 + (g_pin.numel() * 4 if with_bwd else 0)
    d2h = out_pin.numel() * 4 + (dx_pin.numel() * 4 if with_bwd else 0)

    peaks = load_peaks()
    ab = algorithmic_bytes(B, T, H, D)
    is_default = all(WORKLOAD[k] == WORKLOADS[DEFAULT_WORKLOAD][k] for k in WORKLOAD)
    if with_bwd:
        # dominant kernel: the backward core.  The tensor pipe really executes 15 passes per 4
        # algorithmic products: S is recomputed (5 products) and every product is three bf16 passes.
        core_s, core_fl, core_bytes, passes = stage_med[3] * 1e-3, flops_bwd(B, T, H, D), ab["bwd"], 15.0 / 4.0
        kernel_name = "attn_bwd_kernel (backward core)"
    else:
        core_s, core_fl, core_bytes, passes = stage_med[1] * 1e-3, flops_fwd(B, T, H, D), ab["fwd"], 3.0
        kernel_name = "attn_fwd_kernel (forward core)"
    achieved = core_fl / core_s / 1e12
    peak_tf = peaks["bf16_tflops"]  # the kernel is timed alone in a millisecond burst: the burst figure applies
    roofline = {
        "kernel": kernel_name, "bound": "tensor", "achieved": achieved, "peak": peak_tf,
        "unit": "TFLOP/s", "frac": achieved / peak_tf,
        "traffic": None,  # not captured in this run (ncu is never run inside the bench)
        "traffic_profiled": BWD_CORE_DRAM_BYTES_PROFILED if (with_bwd and is_default) else None,
        "peak_source": peaks["source"] + " (cuBLAS bf16, burst)",
        "frac_of_sustained_peak": achieved / peaks["bf16_tflops_sustained"], "sustained_peak": peaks["bf16_tflops_sustained"],
        "launch_us": core_s * 1e6,
        "executed": {"tflops": achieved * passes, "frac": achieved * passes / peak_tf,
                     "passes_per_algorithmic_product": passes},
        "hbm": {"achieved_gbs": core_bytes / core_s / 1e9, "peak_gbs": peaks["hbm_gbs"],
                "frac": core_bytes / core_s / 1e9 / peaks["hbm_gbs"], "algorithmic_bytes": core_bytes},
    }

    # ---------------- strong scaling: one fixed workload cut into contiguous batch slices ----------------
    strong = None
    if args.strong and is_default:
        strong = {}
        del sets[:]
        torch.cuda.empty_cache()
        for name in STRONG_WORKLOADS:
            wl = WORKLOADS[name]
            sB, sT, sH, sD, sbwd = wl["B"], wl["T"], wl["H"], wl["D"], wl["backward"]
            fl_all = flops_fwd(sB, sT, sH, sD) + (flops_bwd(sB, sT, sH, sD) if sbwd else 0.0)

            def run_slice(lo, hi, reps=args.steps):
                """Kernel time (ms per pass) of batch entries [lo, hi) on this rank's GPU."""
                n = hi - lo
                if n == 0:
                    return 0.0
                x, g = seeded_device_entries(dev, lo, hi, sT, sH, sD, sbwd)
                out = torch.empty((n, sT, sH * sD), device=dev)
                lse = torch.empty((n, sH, sT), device=dev)
                saved = torch.empty(pkg.saved_bytes(n, sT, sH, sD), device=dev, dtype=torch.uint8)
                dx = torch.empty((n, sT, 3 * sH * sD), device=dev) if sbwd else None
                scratch = torch.empty(pkg.backward_scratch_bytes(n, sT, sH, sD), device=dev, dtype=torch.uint8) if sbwd else None

                def one(_i):
                    pkg.forward_into(x, out, None, lse, saved, sH)
                    if sbwd:
                        pkg.backward_into(saved, out, lse, g, dx, scratch, sH)

                for w in range(3):
                    one(w)
                torch.cuda.synchronize()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream)
                for r in range(reps):
                    one(r)
                b.record(stream)
                torch.cuda.synchronize()
                del x, g, out, lse, saved, dx, scratch
                torch.cuda.empty_cache()
                return a.elapsed_time(b) / reps

            lo, hi = shard.batch_slices(sB, world)[rank]
            barrier()
            ms_rank = run_slice(lo, hi)
            ms_split = max_over_ranks(ms_rank)
            # the whole workload on ONE GPU, in the same run (rank 0; the others wait at the barrier)
            ms_single = run_slice(0, sB) if rank == 0 else 0.0
            ms_single = max_over_ranks(ms_single)
            barrier()
            strong[name] = {
                "B": sB, "T": sT, "H": sH, "D": sD, "passes": "fwd+bwd" if sbwd else "fwd",
                "slices": shard.batch_slices(sB, world), "ms_per_pass_max_over_ranks": ms_split,
                "tflops": fl_all / (ms_split * 1e-3) / 1e12,
                "single_gpu_ms_per_pass": ms_single, "single_gpu_tflops": fl_all / (ms_single * 1e-3) / 1e12,
                "efficiency": ms_single / (world * ms_split),
            }
        if pkg.device_status() != 0:
            raise SystemExit("kernel status word set during the strong-scaling block")

    cpu_baseline = gpu_baseline = train = None
    if rank == 0 and world == 1:
        if not args.no_cpu_baseline:
            cpu_baseline = measure_cpu_baseline()
        if is_default and args.gpu_baseline:
            gpu_baseline = measure_gpu_baseline()
        if is_default and args.train:
            train = measure_train()

    if rank == 0:
        line = {
            "metric": METRIC if with_bwd else "attn fwd TFLOP/s", "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_total / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {
                "workload": f"causal attention {'fwd+bwd' if with_bwd else 'fwd only'}, fused qkv [B,T,3C] fp32 io, "
                            f"B={B} T={T} H={H} D={D} per GPU",
                "name": args.workload,
                "global_batch": B * world, "seq_len": T, "n_heads": H, "head_dim": D, "seed": SEED,
                "precision": "bf16 hi/lo split operands (3 MMAs per product), fp32 accumulate and softmax",
                "l2": f"{rotate} rotating buffer sets of {set_bytes / 1e6:.0f} MB each (> 126 MB L2 between reuses)",
                "parallelism": f"batch shards on {world} GPU(s), no collective",
            },
            "repeats": {"n": args.repeats, "ms_per_step_median": ms_total / args.steps,
                        "ms_per_step_min": min(loop_ms) / args.steps, "ms_per_step_max": max(loop_ms) / args.steps,
                        "value_min": to_tflops(max(loop_ms)), "value_max": to_tflops(min(loop_ms))},
            "pct_of_nominal_bf16_peak": 100.0 * value / (NOMINAL_BF16_TFLOPS * world),
            "pct_of_measured_bf16_peak": 100.0 * value / (peaks["bf16_tflops"] * world),
            "pct_of_measured_sustained_bf16_peak": 100.0 * value / (peaks["bf16_tflops_sustained"] * world),
            "staged_pass_ms_per_step": staged_ms_total / args.steps,
            "stage_us": {"fwd_split": stage_ms[0] * 1e3, "fwd_core": stage_ms[1] * 1e3,
                         "bwd_prepare": stage_ms[2] * 1e3, "bwd_core": stage_ms[3] * 1e3},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms / args.steps,
                    "copy_only": {"ms_per_step": e2e_copy_ms / args.steps,
                                  "host_gbs_per_direction": h2d * world / (e2e_copy_ms / args.steps * 1e-3) / 1e9,
                                  "note": "the same three streams and copies with the kernel calls left out, all ranks at once"}},
            "gpu_launches": (4 if with_bwd else 2) * args.steps,  # per K-step timed loop (each of the `repeats` loops)
            "host_cores_bound": cpu_affinity,
            "clocks": clocks,
            "graph": (graph_info | {"value": flops_step * world / (graph_info["ms_per_step"] * 1e-3) / 1e12,
                                    "unit": UNIT}) if graph_info else None,
            "roofline": roofline,
            "strong": strong,
            "cpu_baseline": cpu_baseline,
            "gpu_baseline": gpu_baseline,
            "train": train,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------------
# --linear: the Linear kernels either side of the layer against cuBLAS TF32 (not part of the JSON line above)
# ------------------------------------------------------------------------------------------------
LINEAR_SHAPES = [  # name, M, N (out_features), K (in_features)
    ("qkv", 8192, 2304, 768),
    ("attn c_proj", 8192, 768, 768),
    ("mlp c_fc", 8192, 3072, 768),
    ("mlp c_proj", 8192, 768, 3072),
]


def run_linear(args) -> None:
    """--linear: times the Linear kernels either side of the layer (include/linear_sm100.h) on one B200 against
    the library GEMM the reference uses for the same layers (cuBLAS in TF32 tensor-op math, here through
    torch.addmm / torch.matmul with TF32 allowed), for the Linear shapes of GPT-2 124M at B=8, T=1024.  One
    JSON line per shape: microseconds and algorithmic TFLOP/s (2*M*N*K per product) of forward (with and
    without the fused bf16 planes), backward (dx + dW + db) and its two products alone, next to the cuBLAS
    time of the same product.  --cold writes a 512 MB buffer between launches so that every launch starts with
    a cold L2 (default: warm, back to back); --shape M,N,K times one other shape (e.g. 8192,50257,768, the
    vocabulary projection); --only fwd|dx|dw launches nothing but that product (for a profiler capture)."""
    import torch

    import __graft_entry__ as entry

    pkg = entry.load_package()
    pkg.init()
    torch.backends.cuda.matmul.allow_tf32 = True
    flush = torch.empty(512 << 20, device="cuda", dtype=torch.uint8) if args.cold else None

    def timed(fn) -> float:
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        total = 0.0
        if flush is None:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(args.steps):
                fn()
            b.record()
            torch.cuda.synchronize()
            total = a.elapsed_time(b)
        else:
            for _ in range(args.steps):
                flush.zero_()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                fn()
                b.record()
                torch.cuda.synchronize()
                total += a.elapsed_time(b)
        return total / args.steps * 1e3  # microseconds

    shapes = LINEAR_SHAPES
    if args.shape:
        m, n, k = (int(v) for v in args.shape.split(","))
        shapes = [("custom", m, n, k)]
    for name, M, N, K in shapes:
        x = torch.randn(M, K, device="cuda")
        w = torch.randn(N, K, device="cuda") * 0.05
        b = torch.randn(N, device="cuda")
        dy = torch.randn(M, N, device="cuda")
        dw = torch.zeros(N, K, device="cuda")
        db = torch.zeros(N, device="cuda")
        fl = 2.0 * M * N * K
        if args.only:
            one = {"fwd": lambda: pkg.linear_forward(x, w, b),
                   "dx": lambda: pkg.linear_backward(dy, x, w, None, None),
                   "dw": lambda: pkg.linear_backward(dy, x, w, dw, None, want_dx=False)}[args.only]
            t_us = timed(one)
            print(json.dumps({"layer": name, "M": M, "N": N, "K": K, "us": {args.only: round(t_us, 1)},
                              "tflops": {args.only: round(fl / t_us / 1e6, 1)}, "status": pkg.device_status()}), flush=True)
            continue
        planes = torch.empty(4 * M * N + 512, device="cuda", dtype=torch.uint8) if N % 8 == 0 else None

        def cublas_bwd():
            _ = dy @ w
            dw.addmm_(dy.t(), x)
            db.add_(dy.sum(0))

        us = {
            "fwd": timed(lambda: pkg.linear_forward(x, w, b)),
            "fwd_with_planes": timed(lambda: pkg.linear_forward(x, w, b, planes=planes)) if planes is not None else None,
            "fwd_cublas_tf32": timed(lambda: torch.addmm(b, x, w.t())),
            "bwd": timed(lambda: pkg.linear_backward(dy, x, w, dw, db)),
            "bwd_cublas_tf32": timed(cublas_bwd),
            "dx": timed(lambda: pkg.linear_backward(dy, x, w, None, None)),
            "dx_cublas_tf32": timed(lambda: dy @ w),
            "dw": timed(lambda: pkg.linear_backward(dy, x, w, dw, None, want_dx=False)),
            "dw_cublas_tf32": timed(lambda: dw.addmm_(dy.t(), x)),
        }
        status = pkg.device_status()
        if status != 0:
            raise SystemExit(f"kernel status word {status}")
        line = {"layer": name, "M": M, "N": N, "K": K, "l2": "cold" if args.cold else "warm",
                "us": {k: round(v, 1) for k, v in us.items() if v is not None},
                "tflops": {k: round((fl if k.startswith(("fwd", "dx", "dw")) else 2 * fl) / v / 1e6, 1)
                           for k, v in us.items() if v is not None}}
        print(json.dumps(line), flush=True)



def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--repeats", type=int, default=REPEATS, help="how many times the K-step timed loop is run")
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the host-core baseline leg")
    ap.add_argument("--no-gpu-baseline", dest="gpu_baseline", action="store_false",
                    help="skip the reference-CUDA / layer-API leg (rank 0, N=1)")
    ap.add_argument("--no-train", dest="train", action="store_false",
                    help="skip the GPT-2 124M train_gpt leg (rank 0, N=1)")
    ap.add_argument("--no-strong", dest="strong", action="store_false", help="skip the strong-scaling block")
    ap.add_argument("--no-ramp", action="store_true", help="skip the untimed clock ramp (for profiler captures)")
    ap.add_argument("--no-graph", dest="graph", action="store_false",
                    help="skip the extra pass that replays the steps from CUDA graphs (one per buffer set)")
    ap.add_argument("--kernels-only", action="store_true",
                    help="profiler runs: headline and staged passes only (implies every --no-* leg)")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default=DEFAULT_WORKLOAD,
                    help="shape to run; the default is the one the metric is quoted on")
    ap.add_argument("--linear", action="store_true",
                    help="time the Linear kernels either side of the layer against cuBLAS TF32 instead (see run_linear)")
    ap.add_argument("--cold", action="store_true", help="--linear: cold L2 between launches")
    ap.add_argument("--shape", default=None, metavar="M,N,K", help="--linear: one shape instead of GPT-2 124M's four")
    ap.add_argument("--only", default=None, choices=["fwd", "dx", "dw"], help="--linear: launch only that product")
    args = ap.parse_args()
    if args.linear:
        if args.steps == 200:
            args.steps = 30
        return run_linear(args)
    WORKLOAD.clear()
    WORKLOAD.update(WORKLOADS[args.workload])
    if args.warmup < 3:
        args.warmup = 3
    if args.repeats < 1:
        args.repeats = 1
    if args.kernels_only:
        args.no_cpu_baseline, args.gpu_baseline, args.train, args.strong, args.graph = True, False, False, False, False
        args.repeats = 1
    if args.impl == "reference":
        if args.steps > 20:
            args.steps = 20  # each step is ~a second of host work; keep the arm within minutes
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
