"""Attention forward+backward benchmark (TFLOP/s, and fraction of the measured bf16 tensor peak).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload llm_gqa|wide_head|dit_masked|...]
    python bench.py --impl reference ...      # CPU oracle port of the reference path, host cores

A step is one forward+backward pass of the attention operator over one batch of seeded synthetic
input.  The default workload is the LLM grouped-query configuration the throughput target is
quoted on: B=4, Hq=32, Hkv=8, S=4096, D=128, bf16, causal, q scaled by 8, keys with a per-head
constant offset (run with key centering), small output gradients.  At N > 1 every rank runs the
same configuration on its own data (independent batch x head units, no collective): weak scaling.

One JSON line is printed by rank 0.  ``value`` is device-timed with the inputs resident in HBM;
``e2e`` starts from pinned host buffers and includes the host->device copy of q, k, v, dO and
the device->host copy of O, dQ, dK, dV.  The timed region is stretched to ``--min-seconds`` (2 s by
default) by timing more steps than ``--steps`` asks for: a 50 ms burst runs at clocks a sustained job
never sees.  ``others`` holds short runs of the remaining benchmark configurations (and, at N > 1,
the ring context-parallel run, the one path with a collective), ``comparator`` PyTorch's own fused
attention on one published shape; both are context, the headline is ``value`` / ``e2e``.
"""

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "kohakufa-cute_b200"))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (B, Hq, Hkv, S, D, dtype, causal)
    "llm_gqa": dict(B=4, Hq=32, Hkv=8, S=4096, D=128, dtype="bf16", causal=True, center_keys=True, seed=3),
    # the same operator at a size small enough for multi-pass profiler captures (still larger than L2)
    "llm_gqa_small": dict(B=2, Hq=16, Hkv=4, S=4096, D=128, dtype="bf16", causal=True, center_keys=True, seed=3),
    "wide_head": dict(B=1, Hq=16, Hkv=16, S=1024, D=512, dtype="bf16", causal=True, center_keys=False, seed=21,
                      graph=True, published_tflops=214.7),
    # further shapes the reference publishes for B200 (its own kernels: 70 and 138 TFLOP/s fwd+bwd)
    "wide_head_4k": dict(B=1, Hq=16, Hkv=16, S=4096, D=512, dtype="bf16", causal=True, center_keys=False, seed=22,
                         published_tflops=70.0),
    "d128_4k": dict(B=1, Hq=16, Hkv=16, S=4096, D=128, dtype="bf16", causal=True, center_keys=False, seed=23,
                    graph=True, published_tflops=138.0),
    "d64_4k": dict(B=1, Hq=16, Hkv=16, S=4096, D=64, dtype="bf16", causal=True, center_keys=False, seed=24,
                   graph=True, published_tflops=118.0),
    "dit_masked": dict(B=2, Hq=24, Hkv=24, S=32768, D=128, dtype="bf16", causal=False, center_keys=False, seed=4,
                       masked_fraction=0.1),
    # The video/DiT shape as ONE long sequence sharded over the ranks (ring context parallelism).
    # The sequence is divided by the number of ranks, so the job is fixed as N grows (strong scaling).
    "dit_ring": dict(B=1, Hq=24, Hkv=24, S=262144, D=128, dtype="bf16", causal=False, center_keys=False, seed=6,
                     masked_fraction=0.1, ring=True),
    "dit_ring_small": dict(B=1, Hq=24, Hkv=24, S=65536, D=128, dtype="bf16", causal=False, center_keys=False, seed=6,
                           masked_fraction=0.1, ring=True),
    # A causal language-model sequence of 131072 tokens over the ranks: zig-zag shards (rank r owns chunks r and
    # 2N-1-r of 2N), so every rank has the same visible work in every ring step.  Random data: a shard is a shard.
    "llm_ring_causal": dict(B=1, Hq=32, Hkv=8, S=131072, D=128, dtype="bf16", causal=True, center_keys=False, seed=8,
                            ring=True),
    # the reference's published 2-D neighbourhood shape on B200: 151.28 us forward+backward (CUDA-graph median)
    "neighborhood_2d": dict(B=1, Hq=8, Hkv=8, S=64 * 64, D=64, dtype="bf16", causal=False, center_keys=False,
                            seed=7, grid=(64, 64), window=(7, 7), graph=True,
                            published_tflops=3.5 * 4 * 8 * 64 * 4096 * 49 / 151.28e-6 / 1e12),
    "neighborhood_3d": dict(B=1, Hq=16, Hkv=16, S=16 * 32 * 32, D=64, dtype="fp16", causal=False, center_keys=False,
                            seed=5, grid=(16, 32, 32), window=(3, 7, 7), graph=True),
}
# short runs added to the headline line: (workload, steps, minimum seconds of timed region)
OTHERS_SINGLE = (("wide_head", 20, 0.2), ("wide_head_4k", 20, 0.2), ("d128_4k", 20, 0.2), ("d64_4k", 20, 0.2),
                 ("dit_masked", 3, 0.3), ("neighborhood_3d", 20, 0.2), ("neighborhood_2d", 20, 0.2))
OTHERS_MULTI = (("dit_ring", 2, 0.0), ("llm_ring_causal", 2, 0.0))

# GEMMs of the seven algorithmic ones (S, PV forward; S, dP, dV, dK, dQ backward counted as 5) attributed to a
# kernel, and GEMMs it executes.  The two backward owners each recompute S and dP: 9 executed per 7.
GEMM_SHARE = {"pipeline_forward": (2.0, 2), "general_forward": (2.0, 2), "neighborhood_forward": (2.0, 2),
              "na_pipeline_forward": (2.0, 2), "wide_forward": (2.0, 3), "wide_scores_p": (1.0, 1),
              "wide_scores_ds": (1.0, 1), "wide_grad": (3.0, 3)}
# DRAM bytes (read + write) per launch of the pipeline kernels on `llm_gqa`, scaled x4 from the ncu capture of
# `llm_gqa_small` (a quarter of the batch x heads; traffic grows with the units): profiles/pipeline_kernels_llm_gqa_small_ncu.md
NCU_TRAFFIC = {"llm_gqa": {"pipeline_forward": 4 * (50.42e6 + 5.32e6), "pipeline_backward_q": 4 * (85.51e6 + 11.51e6),
                           "pipeline_backward_kv": 4 * (88.05e6 + 4.82e6)}}


def algorithmic_flops(w):
    """fwd = 4 * B * Hq * D * visible (query, key) pairs; fwd+bwd = 3.5 * fwd."""
    S = w["S"]
    if "window" in w:
        pairs = S * math.prod(w["window"])
    elif w["causal"]:
        pairs = S * S / 2
    else:
        pairs = S * (S - int(S * w.get("masked_fraction", 0.0) + 0.5))
    return 3.5 * 4 * w["B"] * w["Hq"] * w["D"] * pairs


def algorithmic_bytes(w):
    """One read of Q, K, V, dO, O and one write of O, dQ, dK, dV (16-bit) plus the two FP32 row statistics."""
    q = w["B"] * w["Hq"] * w["S"] * w["D"] * 2
    kv = w["B"] * w["Hkv"] * w["S"] * w["D"] * 2
    return 5 * q + 4 * kv + 2 * w["B"] * w["Hq"] * w["S"] * 4 * 2


def make_host_inputs(w, rank, world=1):
    """Seeded synthetic q, k, v, dO (and mask) in pinned host memory.  Ring workloads get this rank's
    contiguous shard of the sequence (and of the key-padding mask)."""
    dtype = torch.bfloat16 if w["dtype"] == "bf16" else torch.float16
    gen = torch.Generator().manual_seed(w["seed"] * 1000 + rank)
    B, Hq, Hkv, S, D = w["B"], w["Hq"], w["Hkv"], w["S"], w["D"]
    total, first = S, 0
    if w.get("ring"):
        S = total // world
        first = rank * S

    def randn(*shape):
        out = torch.empty(shape, dtype=torch.float32)
        for b in range(shape[0]):  # chunked to bound the FP32 staging memory
            out[b] = torch.randn(shape[1:], generator=gen)
        return out

    name = w["name"]
    q = randn(B, Hq, S, D)
    k = randn(B, Hkv, S, D)
    v = randn(B, Hkv, S, D)
    g = randn(B, Hq, S, D)
    if name.startswith("llm_gqa"):
        q *= 8.0
        k += 2.0 * torch.randn(B, Hkv, 1, D, generator=gen)  # N(0, 4): std 2 per component
        g *= math.sqrt(1e-3)  # N(0, 1e-3): std sqrt(1e-3)
    pin = (lambda t: t.pin_memory()) if torch.cuda.is_available() else (lambda t: t)
    tensors = [pin(t.to(dtype)) for t in (q, k, v, g)]
    mask = None
    if "masked_fraction" in w:
        keep = total - int(total * w["masked_fraction"] + 0.5)
        mask = pin((torch.arange(first, first + S) < keep)[None, None, None, :].expand(B, 1, 1, S).contiguous())
    return tensors, mask


def build_step(w):
    import kohakufa_cute

    if w.get("ring"):
        from kohakufa_cute import parallel

        causal = bool(w["causal"])

        def forward(q, k, v, mask):
            return parallel.ring_attention(q, k, v, key_mask=mask, causal=causal)
    elif "window" in w:
        grid, window = w["grid"], w["window"]

        def forward(q, k, v, mask):
            return kohakufa_cute.neighborhood_attention(q, k, v, spatial_shape=grid, window_size=window, scale=0.125)
    else:
        def forward(q, k, v, mask):
            return kohakufa_cute.attention(q, k, v, mask=mask, causal=w["causal"], center_keys=w["center_keys"])

    def step(q, k, v, g, mask):
        out = forward(q, k, v, mask)
        dq, dk, dv = torch.autograd.grad(out, (q, k, v), g)
        return out, dq, dk, dv

    return step


def describe_config(w, world, launch, l2_note):
    """The ``config`` object; both arms print the same keys for the same workload."""
    return {"workload": w["name"], "launch": launch, "B": w["B"], "Hq": w["Hq"], "Hkv": w["Hkv"], "S": w["S"],
            "D": w["D"], "causal": w["causal"], "center_keys": w["center_keys"],
            "sharding": ((f"ring context parallel, S/{world} per rank" + (", zig-zag chunks" if w["causal"] else ""))
                         if w.get("ring") else f"replica-per-gpu x{world}"),
            "l2": l2_note,
            "input_stds": {"q": 8.0, "k_offset": 2.0, "dout": math.sqrt(1e-3)} if w["name"].startswith("llm_gqa") else None}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap,power.draw")

    def __init__(self, index):
        self.index, self.samples, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.time(), line.strip()))

    def stop(self, begin, end):
        if self.proc is None:
            return None
        time.sleep(0.15)
        self.proc.terminate()
        rows = [line for stamp, line in self.samples if begin - 0.05 <= stamp <= end + 0.15] or \
               [line for _, line in self.samples]
        clocks, power, peak, reasons = [], [], None, set()
        for line in rows:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 6 or not parts[0].isdigit():
                continue
            clocks.append(int(parts[0]))
            peak = int(parts[1]) if parts[1].isdigit() else peak
            for label, flag in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                   parts[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(label)
            if len(parts) > 6:
                try:
                    power.append(float(parts[6]))
                except ValueError:
                    pass
        if not clocks:
            return None
        return {"sm_mhz": int(statistics.median(clocks)), "sm_min_mhz": min(clocks), "sm_max_mhz": peak,
                "reasons": sorted(reasons), "samples": len(clocks),
                "power_w_median": statistics.median(power) if power else None}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            data = json.load(f)
        return data["bf16_tflops"], data.get("bf16_tflops_sustained"), data["hbm_gbs"], "measured"
    return 1590.0, 1400.0, 6650.0, "fallback"


def host_threads(world):
    """Threads for CPU work on this box: torchrun exports OMP_NUM_THREADS=1, which would time the CPU
    baseline on a single core, so the count is set from the cores this process may run on."""
    try:
        cores = len(os.sched_getaffinity(0))
    except AttributeError:
        cores = os.cpu_count() or 1
    return max(1, cores)


def cpu_oracle_sample(w, budget_seconds=10.0):
    """Times the CPU oracle (the reference's PyTorch path restated) on (batch, query-head) units of the
    workload, one after another with fresh seeded data of the workload's distribution (keys centred when the
    workload centres them), until about ``budget_seconds`` of CPU work is done."""
    from oracle import attention_oracle as ao

    dtype = torch.bfloat16 if w["dtype"] == "bf16" else torch.float16
    S = min(w["S"], 4096)
    D = w["D"]
    gen = torch.Generator().manual_seed(w["seed"])
    causal = w["causal"]
    llm = w["name"].startswith("llm_gqa")

    def unit(length):
        q = torch.randn(1, 1, length, D, generator=gen) * (8.0 if llm else 1.0)
        k = torch.randn(1, 1, length, D, generator=gen) + (2.0 * torch.randn(1, 1, 1, D, generator=gen) if llm else 0.0)
        v = torch.randn(1, 1, length, D, generator=gen)
        g = torch.randn(1, 1, length, D, generator=gen) * (math.sqrt(1e-3) if llm else 1.0)
        return tuple(t.to(dtype) for t in (q, k, v, g))

    def run(q, k, v, g):
        if w["center_keys"]:
            k = ao.center_keys(k)
        ao.contract_reference((q, k, v), g, None, causal, None)

    run(*unit(256))
    units, seconds = 0, 0.0
    while units < 2 or (seconds < budget_seconds and units < 4096):
        tensors = unit(S)
        begin = time.perf_counter()
        run(*tensors)
        seconds += time.perf_counter() - begin
        units += 1
    flops = units * 3.5 * 4 * D * (S * S / 2 if causal else S * S)
    return (flops / seconds / 1e12, seconds,
            f"{units} (batch, query head) units: S={S}, D={D}, causal={causal}, center_keys={w['center_keys']}, {w['dtype']}")


def reference_arm(args, w, rank, world):
    if rank != 0:
        return
    torch.set_num_threads(host_threads(world))
    steps, warmup = max(1, args.steps), max(0, args.warmup)
    for _ in range(warmup):
        cpu_oracle_sample(w, 1.0)
    # each step is a bounded sample (about three seconds of host work) of the same workload
    values = [cpu_oracle_sample(w, 3.0) for _ in range(min(steps, 20))]
    value = statistics.mean(x[0] for x in values)
    seconds = statistics.mean(x[1] for x in values)
    h2d = 2 * (2 * w["B"] * w["Hq"] + 2 * w["B"] * w["Hkv"]) * w["S"] * w["D"]
    line = {
        "impl": "reference", "metric": "attn fwd+bwd TFLOP/s", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": len(values), "warmup": warmup, "ms_per_step": seconds * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
        "config": describe_config(w, max(1, args.gpus), "eager",
                                  "inputs larger than L2 (q+k+v+dO+O > 126 MB)" if h2d > 126e6 else "inputs fit in L2"),
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": values[0][2]},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "CPU restatement (oracle/) of the reference's FP32/FP64 PyTorch attention path on the host cores; "
                "the reference's CuTe-DSL GPU kernels cannot be imported on this image",
    }
    print(json.dumps(line), flush=True)


def pin_to_gpu_cpus(local_rank):
    """Runs this process on the CPUs NVML lists as closest to its GPU, so that its pinned buffers are allocated
    (first touched) on that memory node.  Returns what was done, for the record."""
    try:
        import pynvml

        pynvml.nvmlInit()
        handle = pynvml.nvmlDeviceGetHandleByIndex(local_rank)
        words = pynvml.nvmlDeviceGetCpuAffinity(handle, (os.cpu_count() + 63) // 64)
        cpus = {64 * i + bit for i, word in enumerate(words) for bit in range(64) if (word >> bit) & 1}
        allowed = os.sched_getaffinity(0)
        target = (cpus & allowed) or allowed
        os.sched_setaffinity(0, target)
        return {"cpus_near_gpu": len(cpus), "cpus_allowed": len(allowed), "cpus_used": len(target)}
    except Exception as error:  # no NVML, no permission: keep the default placement
        return {"error": type(error).__name__}


class Harness:
    """Timing of one workload on this rank's GPU (device-timed, max over ranks)."""

    def __init__(self, rank, local_rank, world, device):
        self.rank, self.local_rank, self.world, self.device = rank, local_rank, world, device

    def barrier(self):
        if self.world > 1:
            import torch.distributed as dist

            dist.barrier()
        torch.cuda.synchronize()

    def reduce_max(self, values):
        t = torch.tensor(values, device=self.device, dtype=torch.float64)
        if self.world > 1:
            import torch.distributed as dist

            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(x) for x in t.cpu()]

    def run(self, w, steps, warmup, min_seconds, launch="auto", sample_clocks=False, keep=False):
        """Times ``steps`` steps (more if needed to fill ``min_seconds``).  Returns a dict; with ``keep`` the
        device tensors stay alive in it for the end-to-end pass."""
        from kohakufa_cute import native

        (hq, hk, hv, hg), hmask = make_host_inputs(w, self.rank, self.world)
        step = build_step(w)
        dq_, dk_, dv_, dg_ = (t.to(self.device).requires_grad_(i < 3) for i, t in enumerate((hq, hk, hv, hg)))
        dmask = None if hmask is None else hmask.to(self.device)
        use_graph = launch == "graph" or (launch == "auto" and w.get("graph", False))
        for _ in range(warmup):
            step(dq_, dk_, dv_, dg_, dmask)
        self.barrier()
        launches_per_step, rotation, probe_ms = None, 1, None
        if use_graph:
            # One CUDA graph of forward + backward through the public API per input set, replayed once per step.
            # Small workloads fit in L2, so the steps rotate over enough independent input sets to exceed it.
            set_bytes = 2 * sum(t.numel() * t.element_size() for t in (hq, hk, hv, hg))
            rotation = max(1, int(math.ceil(2 * 126e6 / set_bytes)))
            sets = [(dq_, dk_, dv_, dg_)]
            for _ in range(1, rotation):
                sets.append(tuple(torch.randn_like(t).requires_grad_(t.requires_grad) for t in sets[0]))
            graphs = []
            before = native.launch_count()
            for tensors in sets:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    kept = step(*tensors, dmask)
                graphs.append((graph, kept))
            launches_per_step = (native.launch_count() - before) // rotation
            cursor = [0]

            def run_step():
                graphs[cursor[0] % rotation][0].replay()
                cursor[0] += 1

            for _ in range(warmup):
                run_step()
            self.barrier()
        else:
            def run_step():
                step(dq_, dk_, dv_, dg_, dmask)

        # Stretch the timed region: estimate the step time from a short probe, then time enough steps.
        if min_seconds > 0:
            b0, e0 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            b0.record()
            for _ in range(steps):
                run_step()
            e0.record()
            torch.cuda.synchronize()
            probe_ms = self.reduce_max([b0.elapsed_time(e0) / steps])[0]
            steps = max(steps, int(math.ceil(min_seconds * 1e3 / max(probe_ms, 1e-3))))
        native.profile_read(reset=True)
        sampler = ClockSampler(self.local_rank) if sample_clocks else None
        if sampler:
            sampler.start()
            time.sleep(0.3)
        launches_before = native.launch_count()
        begin_evt, end_evt = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.barrier()
        wall_begin = time.time()
        begin_evt.record()
        for _ in range(steps):
            run_step()
        end_evt.record()
        self.barrier()
        wall_end = time.time()
        elapsed_ms = self.reduce_max([begin_evt.elapsed_time(end_evt)])[0]
        launches = launches_per_step * steps if use_graph else native.launch_count() - launches_before
        clocks = sampler.stop(wall_begin, wall_end) if sampler else None
        # Per-kernel times come from a profiled pass right after the timed region: with per-kernel events on, the
        # library launches its kernels one after another on one stream (in the timed region the two backward
        # owners overlap on two streams, and a captured graph cannot hold the events at all).  For short steps
        # the launches are queued behind a device-side delay, so that host launch gaps stay out of the events.
        prof_steps = 3 if use_graph else min(steps, 20)
        native.profile_enable(True)
        for _ in range(prof_steps):
            if use_graph:
                torch.cuda._sleep(4_000_000)
            step(dq_, dk_, dv_, dg_, dmask)
        self.barrier()
        native.profile_enable(False)
        kernels = native.profile_read(reset=True)
        flops = algorithmic_flops(w)
        jobs = 1 if w.get("ring") else self.world  # a ring step is ONE job shared by all ranks
        h2d = sum(t.numel() * t.element_size() for t in (hq, hk, hv, hg)) + (0 if hmask is None else hmask.numel())
        result = {
            "workload": w["name"], "steps": steps, "ms_per_step": elapsed_ms / steps, "probe_ms": probe_ms,
            "value": flops * steps * jobs / (elapsed_ms * 1e-3) / 1e12, "timed_seconds": elapsed_ms * 1e-3,
            "launch": "cuda_graph" if use_graph else "eager", "rotation": rotation, "launches": launches,
            "kernels": kernels, "prof_steps": prof_steps, "clocks": clocks, "h2d": h2d,
            "l2": "inputs larger than L2 (q+k+v+dO+O > 126 MB)" if h2d > 126e6 else (
                f"steps rotate over {rotation} input sets, together larger than L2" if rotation > 1 else "inputs fit in L2"),
        }
        if keep:
            result["host"] = ((hq, hk, hv, hg), hmask)
            result["step"] = step
        return result


def end_to_end(harness, w, host, step, steps):
    """The same step from pinned host memory: ONE host->device copy of a staging buffer that holds q, k, v, dO
    (and the mask), the step, a device-side gather of O, dQ, dK, dV into one buffer and ONE device->host copy.
    Like a training loop with a prefetching loader, the upload of step i+1 and the download of step i-1 run on
    side streams while step i computes (PCIe is full duplex), over two sets of device buffers."""
    (hq, hk, hv, hg), hmask = host
    device = harness.device
    parts = [hq, hk, hv, hg] + ([] if hmask is None else [hmask])
    sizes = [t.numel() * t.element_size() for t in parts]
    offsets = [sum(((s + 255) // 256) * 256 for s in sizes[:i]) for i in range(len(parts))]
    total_in = offsets[-1] + sizes[-1]
    stage_in = torch.empty(total_in, dtype=torch.uint8).pin_memory()
    for t, off, size in zip(parts, offsets, sizes):
        stage_in[off:off + size].copy_(t.contiguous().view(torch.uint8).flatten())
    out_like = (hq, hq, hk, hv)
    out_sizes = [t.numel() * t.element_size() for t in out_like]
    out_offsets = [sum(out_sizes[:i]) for i in range(4)]
    total_out = sum(out_sizes)
    stage_out = torch.empty(total_out, dtype=torch.uint8).pin_memory()
    dev_in = [torch.empty(total_in, dtype=torch.uint8, device=device) for _ in range(2)]
    dev_out = [torch.empty(total_out, dtype=torch.uint8, device=device) for _ in range(2)]

    def views(buffer):
        tensors = []
        for t, off, size in zip(parts, offsets, sizes):
            tensors.append(buffer[off:off + size].view(t.dtype).view(t.shape))
        return tensors

    compute = torch.cuda.current_stream()
    up_stream, down_stream = torch.cuda.Stream(), torch.cuda.Stream()
    uploaded = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]
    gathered = [torch.cuda.Event() for _ in range(2)]
    downloaded = [torch.cuda.Event() for _ in range(2)]

    def run(count):
        for i in range(count):
            slot = i % 2
            with torch.cuda.stream(up_stream):
                if i >= 2:
                    up_stream.wait_event(consumed[slot])  # the step that last read this buffer set
                dev_in[slot].copy_(stage_in, non_blocking=True)
                uploaded[slot].record(up_stream)
            compute.wait_event(uploaded[slot])
            tensors = views(dev_in[slot])
            q, k, v = (t.detach().requires_grad_(True) for t in tensors[:3])
            results = step(q, k, v, tensors[3], tensors[4] if hmask is not None else None)
            consumed[slot].record(compute)
            if i >= 2:
                compute.wait_event(downloaded[slot])  # the download that last read this output buffer
            for t, off, size in zip(results, out_offsets, out_sizes):
                dev_out[slot][off:off + size].view(t.dtype).view(t.shape).copy_(t.detach())
            gathered[slot].record(compute)
            with torch.cuda.stream(down_stream):
                down_stream.wait_event(gathered[slot])
                stage_out.copy_(dev_out[slot], non_blocking=True)
                downloaded[slot].record(down_stream)
        compute.wait_stream(down_stream)

    run(2)
    harness.barrier()
    b2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    b2.record()
    run(steps)
    e2.record()
    harness.barrier()
    ms = harness.reduce_max([b2.elapsed_time(e2)])[0]
    return ms, total_in, total_out


def sdpa_comparator(device, steps=20):
    """PyTorch's fused attention (cuDNN backend) forward+backward on the published `d128_4k` shape, timed the same
    way on this GPU.  Context only: a vendor library kernel, never on the product path."""
    try:
        from torch.nn.attention import SDPBackend, sdpa_kernel

        w = dict(WORKLOADS["d128_4k"], name="d128_4k")
        gen = torch.Generator(device=device).manual_seed(23)
        shape = (w["B"], w["Hq"], w["S"], w["D"])
        q, k, v = (torch.randn(shape, device=device, dtype=torch.bfloat16, generator=gen).requires_grad_(True) for _ in range(3))
        g = torch.randn(shape, device=device, dtype=torch.bfloat16, generator=gen)

        def step():
            with sdpa_kernel(SDPBackend.CUDNN_ATTENTION):
                out = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)
            torch.autograd.grad(out, (q, k, v), g)

        for _ in range(3):
            step()
        torch.cuda.synchronize()
        b, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        b.record()
        for _ in range(steps):
            step()
        e.record()
        torch.cuda.synchronize()
        ms = b.elapsed_time(e) / steps
        return {"what": "torch SDPA, cuDNN backend, d128_4k fwd+bwd, eager", "ms_per_step": ms,
                "value": algorithmic_flops(w) / (ms * 1e-3) / 1e12, "unit": "TFLOP/s"}
    except Exception as error:
        return {"what": "torch SDPA, cuDNN backend, d128_4k fwd+bwd", "unavailable": f"{type(error).__name__}: {error}"[:200]}


def decode_probe(device, steps=200):
    """One query row per head against 32768 keys (B=1, Hq=32, Hkv=8, D=128, bf16), forward only and without
    gradients: the decoding kernel.  Memory-bound: reported as time and as K/V bytes per second, eager and as a CUDA graph."""
    import kohakufa_cute

    try:
        gen = torch.Generator(device=device).manual_seed(9)
        sets = []
        for _ in range(4):  # rotate over K/V sets that together exceed L2
            q = torch.randn(1, 32, 1, 128, device=device, dtype=torch.bfloat16, generator=gen)
            k, v = (torch.randn(1, 8, 32768, 128, device=device, dtype=torch.bfloat16, generator=gen) for _ in range(2))
            sets.append((q, k, v))
        with torch.no_grad():
            for q, k, v in sets:
                kohakufa_cute.attention(q, k, v)
            torch.cuda.synchronize()
            b, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            b.record()
            for i in range(steps):
                kohakufa_cute.attention(*sets[i % 4])
            e.record()
            torch.cuda.synchronize()
            ms = b.elapsed_time(e) / steps
            # the same four calls as one CUDA graph: the device time without the host's launch cost
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                kept = [kohakufa_cute.attention(*inputs) for inputs in sets]
            for _ in range(3):
                graph.replay()
            b.record()
            for _ in range(steps // 4):
                graph.replay()
            e.record()
            torch.cuda.synchronize()
            graph_ms = b.elapsed_time(e) / (steps // 4 * 4)
            del kept
        kv_bytes = 2 * 8 * 32768 * 128 * 2
        return {"workload": "decode (B1 Hq32 Hkv8 Sq1 Sk32768 D128, forward only, no gradients)",
                "ms_per_call": ms, "kv_gbs": kv_bytes / (ms * 1e-3) / 1e9, "launch": "eager",
                "graph_ms_per_call": graph_ms, "graph_kv_gbs": kv_bytes / (graph_ms * 1e-3) / 1e9}
    except Exception as error:
        return {"workload": "decode", "error": f"{type(error).__name__}: {error}"[:200]}


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=10)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="ours")
    parser.add_argument("--workload", default="llm_gqa", choices=sorted(WORKLOADS))
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-others", action="store_true", help="skip the short runs of the other configurations")
    parser.add_argument("--min-seconds", type=float, default=2.0,
                        help="least length of the timed region; more steps than --steps are timed to fill it")
    parser.add_argument("--launch", default="auto", choices=("auto", "eager", "graph"),
                        help="eager Python launches, or one CUDA graph of the step replayed per step; auto picks "
                             "the graph for workloads whose step is shorter than the host's launch time")
    args = parser.parse_args()
    w = dict(WORKLOADS[args.workload], name=args.workload)
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        reference_arm(args, w, rank, world)
        return

    import torch.distributed as dist
    from kohakufa_cute import native

    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    placement = pin_to_gpu_cpus(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    if world == 1 and w.get("ring"):
        # the ring layer talks to torch.distributed even when it has a single member
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29531")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=device)
    warmup = max(3, args.warmup)
    steps = max(1, args.steps)
    harness = Harness(rank, local_rank, world, device)

    head = harness.run(w, steps, warmup, args.min_seconds, launch=args.launch, sample_clocks=True, keep=True)
    status = native.device_status(reset=True)
    e2e_steps = max(2, min(steps, 6))
    e2e_ms, h2d, d2h = end_to_end(harness, w, head.pop("host"), head.pop("step"), e2e_steps)
    torch.cuda.empty_cache()

    others = []
    if not args.no_others and args.workload == "llm_gqa":
        for name, n, seconds in (OTHERS_MULTI if world > 1 else OTHERS_SINGLE):
            ow = dict(WORKLOADS[name], name=name)
            try:
                r = harness.run(ow, n, 3 if not ow.get("ring") else 1, seconds)
                per = max(1, world if not ow.get("ring") else 1)
                others.append({"workload": name, "value": r["value"], "unit": "TFLOP/s", "ms_per_step": r["ms_per_step"],
                               "steps": r["steps"], "launch": r["launch"],
                               "sharding": describe_config(ow, world, r["launch"], r["l2"])["sharding"],
                               "vs_published": (r["value"] / per / ow["published_tflops"]) if "published_tflops" in ow else None,
                               "kernels_ms": {k: v[0] / v[1] for k, v in r["kernels"].items()}})
            except Exception as error:  # an auxiliary run must not take the headline down
                others.append({"workload": name, "error": f"{type(error).__name__}: {error}"[:200]})
            torch.cuda.empty_cache()
        status = status or native.device_status(reset=True)
    comparator = sdpa_comparator(device) if (rank == 0 and not args.no_others and world == 1) else None
    if rank == 0 and not args.no_others and world == 1 and args.workload == "llm_gqa":
        others.append(decode_probe(device))

    flops = algorithmic_flops(w)
    jobs = 1 if w.get("ring") else world
    value, elapsed_steps = head["value"], head["steps"]
    e2e_value = flops * e2e_steps * jobs / (e2e_ms * 1e-3) / 1e12

    if rank == 0:
        burst, sustained, hbm, source = measured_peaks()
        long_region = head["timed_seconds"] >= 1.0
        kernels = head["kernels"]
        roofline = None
        if kernels:
            # dominant kernel = largest share of device time among this library's kernels
            name, (total_ms, count) = max(kernels.items(), key=lambda item: item[1][0])
            share, executed = GEMM_SHARE.get(name, (1.5, 3) if name.endswith("_q") else (3.5, 4))
            per_step = max(1, int(round(count / head["prof_steps"])))  # a ring step launches each kernel once per block
            per_launch = flops / (world if w.get("ring") else 1) * share / 7.0 / per_step
            achieved = per_launch / (total_ms / count * 1e-3) / 1e12
            # a region of seconds runs at sustained clocks (power cap), a burst does not: pick the matching peak
            peak = sustained if (long_region and sustained) else burst
            roofline = {"bound": "tensor", "kernel": name, "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                        "frac": achieved / peak,
                        "frac_burst": achieved / burst, "frac_sustained": achieved / sustained if sustained else None,
                        "traffic": NCU_TRAFFIC.get(w["name"], {}).get(name),
                        "traffic_note": "dram read+write bytes per launch, ncu capture of llm_gqa_small scaled x4 by the units",
                        "algorithmic_bytes_per_step": algorithmic_bytes(w),
                        "algorithmic_gemms": share, "executed_gemms": executed,
                        "step_algorithmic_gemms": 7, "step_executed_gemms": 9,
                        "peak_source": f"{source} ({'sustained' if peak == sustained else 'burst'} bf16 GEMM; "
                                       f"timed region {head['timed_seconds']:.2f} s)",
                        "timing": f"CUDA events of a profiled pass of {head['prof_steps']} steps after the timed region, kernels serialised",
                        "kernel_ms": total_ms / count,
                        "all_kernels_ms": {k: v[0] / v[1] for k, v in kernels.items()}}
        cpu = None
        if not args.no_cpu_baseline:
            torch.set_num_threads(host_threads(world))
            cpu_value, cpu_seconds, sample = cpu_oracle_sample(w)
            cpu = {"value": cpu_value, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                   "sample": sample, "seconds": cpu_seconds}
        line = {
            "metric": "attn fwd+bwd TFLOP/s", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": elapsed_steps,
            "requested_steps": steps, "warmup": warmup, "ms_per_step": head["ms_per_step"], "higher_is_better": True,
            "scaling": "strong" if w.get("ring") else "weak",
            "vs_baseline": (value / world / w["published_tflops"]) if "published_tflops" in w else None,
            "dtype": w["dtype"], "data": "synthetic",
            "config": describe_config(w, world, head["launch"], head["l2"]),
            "timed_seconds": head["timed_seconds"],
            # the requested steps alone, right after the warm-up (tens of milliseconds at boost clocks): context for
            # the sustained figure above, not a result
            "short_burst": None if not head["probe_ms"] else {
                "steps": steps, "ms_per_step": head["probe_ms"],
                "value": flops * jobs / (head["probe_ms"] * 1e-3) / 1e12, "unit": "TFLOP/s"},
            "frac_of_peak": {"burst": value / world / burst, "sustained": value / world / sustained if sustained else None,
                             "source": source, "sm_mhz_median": head["clocks"]["sm_mhz"] if head["clocks"] else None},
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms / e2e_steps, "steps": e2e_steps,
                    "h2d_gbs_if_alone": h2d / (e2e_ms / e2e_steps * 1e-3) / 1e9,
                    "copies_per_step": {"h2d": 1, "d2h": 1}, "host_placement": placement,
                    "overlap": "one staging buffer per direction; uploads and downloads of neighbouring steps run on "
                               "side streams during compute"},
            "gpu_launches": head["launches"], "clocks": head["clocks"], "roofline": roofline, "cpu_baseline": cpu,
            "others": others, "comparator": comparator, "device_status": status,
        }
        print(json.dumps(line), flush=True)
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
