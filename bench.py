"""Attention forward+backward benchmark (TFLOP/s, and fraction of the measured bf16 tensor peak).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload llm_gqa|wide_head|dit_masked|neighborhood_3d]
    python bench.py --impl reference ...      # CPU oracle port of the reference path, host cores

A step is one forward+backward pass of the attention operator over one batch of seeded synthetic
input.  The default workload is the LLM grouped-query configuration the throughput target is
quoted on: B=4, Hq=32, Hkv=8, S=4096, D=128, bf16, causal, q scaled by 8, keys with a per-head
constant offset (run with key centering), small output gradients.  At N > 1 every rank runs the
same configuration on its own data (independent batch x head units, no collective): weak scaling.

One JSON line is printed by rank 0.  ``value`` is device-timed with the inputs resident in HBM;
``e2e`` starts from pinned host buffers and includes the host->device copies of q, k, v, dO and
the device->host copies of O, dQ, dK, dV.
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
    # the reference's published 2-D neighbourhood shape on B200: 151.28 us forward+backward (CUDA-graph median)
    "neighborhood_2d": dict(B=1, Hq=8, Hkv=8, S=64 * 64, D=64, dtype="bf16", causal=False, center_keys=False,
                            seed=7, grid=(64, 64), window=(7, 7), graph=True,
                            published_tflops=3.5 * 4 * 8 * 64 * 4096 * 49 / 151.28e-6 / 1e12),
    "neighborhood_3d": dict(B=1, Hq=16, Hkv=16, S=16 * 32 * 32, D=64, dtype="fp16", causal=False, center_keys=False,
                            seed=5, grid=(16, 32, 32), window=(3, 7, 7)),
}


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

        def forward(q, k, v, mask):
            return parallel.ring_attention(q, k, v, key_mask=mask)
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


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

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
        clocks, peak, reasons = [], None, set()
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
        if not clocks:
            return None
        return {"sm_mhz": int(statistics.median(clocks)), "sm_max_mhz": peak, "reasons": sorted(reasons),
                "samples": len(clocks)}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            data = json.load(f)
        return data["bf16_tflops"], data.get("bf16_tflops_sustained"), data["hbm_gbs"], "measured"
    return 1590.0, 1400.0, 6650.0, "fallback"


def cpu_oracle_sample(w, budget_seconds=10.0):
    """Times the CPU oracle (the reference's PyTorch path restated) on (batch, query-head) units of the
    workload, one after another with fresh seeded data, until about ``budget_seconds`` of CPU work is done."""
    from oracle import attention_oracle as ao

    dtype = torch.bfloat16 if w["dtype"] == "bf16" else torch.float16
    S = min(w["S"], 4096)
    D = w["D"]
    gen = torch.Generator().manual_seed(w["seed"])
    causal = w["causal"]
    warm = [torch.randn(1, 1, 256, D, generator=gen).to(dtype) for _ in range(4)]
    ao.contract_reference(tuple(warm[:3]), warm[3], None, causal, None)
    units, seconds = 0, 0.0
    while units < 2 or (seconds < budget_seconds and units < 4096):
        q, k, v, g = (torch.randn(1, 1, S, D, generator=gen).to(dtype) for _ in range(4))
        begin = time.perf_counter()
        ao.contract_reference((q, k, v), g, None, causal, None)
        seconds += time.perf_counter() - begin
        units += 1
    flops = units * 3.5 * 4 * D * (S * S / 2 if causal else S * S)
    return (flops / seconds / 1e12, seconds,
            f"{units} (batch, query head) units: S={S}, D={D}, causal={causal}, {w['dtype']}")


def reference_arm(args, w, rank):
    if rank != 0:
        return
    steps, warmup = max(1, args.steps), max(0, args.warmup)
    for _ in range(min(warmup, 1)):
        cpu_oracle_sample(w, 1.0)
    # each step is a bounded sample (about three seconds of host work) of the same workload
    values = [cpu_oracle_sample(w, 3.0) for _ in range(min(steps, 20))]
    value = statistics.mean(x[0] for x in values)
    seconds = statistics.mean(x[1] for x in values)
    line = {
        "impl": "reference", "metric": "attn fwd+bwd TFLOP/s", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": len(values), "warmup": min(warmup, 1), "ms_per_step": seconds * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
        "config": {"workload": w["name"], "B": w["B"], "Hq": w["Hq"], "Hkv": w["Hkv"], "S": w["S"], "D": w["D"],
                   "causal": w["causal"]},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": values[0][2]},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "CPU restatement (oracle/) of the reference's FP32/FP64 PyTorch attention path on the host cores; "
                "the reference's CuTe-DSL GPU kernels cannot be imported on this image",
    }
    print(json.dumps(line), flush=True)


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=10)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="ours")
    parser.add_argument("--workload", default="llm_gqa", choices=sorted(WORKLOADS))
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--launch", default="auto", choices=("auto", "eager", "graph"),
                        help="eager Python launches, or one CUDA graph of the step replayed per step; auto picks "
                             "the graph for workloads whose step is shorter than the host's launch time")
    args = parser.parse_args()
    w = dict(WORKLOADS[args.workload], name=args.workload)
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        reference_arm(args, w, rank)
        return

    import torch.distributed as dist
    from kohakufa_cute import native

    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    elif w.get("ring"):
        # the ring layer talks to torch.distributed even when it has a single member
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29531")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=device)
    warmup = max(3, args.warmup)
    steps = max(1, args.steps)

    (hq, hk, hv, hg), hmask = make_host_inputs(w, rank, world)
    step = build_step(w)
    dq_, dk_, dv_, dg_ = (t.to(device).requires_grad_(i < 3) for i, t in enumerate((hq, hk, hv, hg)))
    dmask = None if hmask is None else hmask.to(device)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    use_graph = args.launch == "graph" or (args.launch == "auto" and w.get("graph", False))
    for _ in range(warmup):
        step(dq_, dk_, dv_, dg_, dmask)
    barrier()
    launches_per_step = None
    rotation = 1
    if use_graph:
        # One CUDA graph of forward + backward through the public API per input set, replayed once per step.
        # Small workloads fit in L2, so the steps rotate over enough independent input sets to exceed it.
        set_bytes = 2 * sum(t.numel() * t.element_size() for t in (hq, hk, hv, hg))
        rotation = max(1, int(math.ceil(2 * 126e6 / set_bytes)))
        sets = [(dq_, dk_, dv_, dg_)]
        for i in range(1, rotation):
            sets.append(tuple(torch.randn_like(t).requires_grad_(t.requires_grad) for t in sets[0]))
        graphs = []
        before = native.launch_count()
        for tensors in sets:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                keep = step(*tensors, dmask)
            graphs.append((graph, keep))
        launches_per_step = (native.launch_count() - before) // rotation
        cursor = [0]

        def run():
            graphs[cursor[0] % rotation][0].replay()
            cursor[0] += 1

        for _ in range(warmup):
            run()
        barrier()
    else:
        def run():
            step(dq_, dk_, dv_, dg_, dmask)

    native.profile_read(reset=True)
    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.3)
    launches_before = native.launch_count()
    begin_evt, end_evt = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    wall_begin = time.time()
    begin_evt.record()
    for _ in range(steps):
        run()
    end_evt.record()
    barrier()
    wall_end = time.time()
    elapsed_ms = begin_evt.elapsed_time(end_evt)
    launches = launches_per_step * steps if use_graph else native.launch_count() - launches_before
    clocks = sampler.stop(wall_begin, wall_end)
    # Per-kernel times come from a profiled pass right after the timed region: with per-kernel events on, the
    # library launches its kernels one after another on one stream (in the timed region the two backward
    # owners overlap on two streams, and a captured graph cannot hold the events at all).  For short steps the
    # launches are queued behind a device-side delay, so that host launch gaps stay out of the events.
    prof_steps = 3 if use_graph else steps
    native.profile_enable(True)
    for _ in range(prof_steps):
        if use_graph:
            torch.cuda._sleep(4_000_000)
        step(dq_, dk_, dv_, dg_, dmask)
    barrier()
    native.profile_enable(False)
    kernels = native.profile_read(reset=True)
    status = native.device_status(reset=True)

    # End to end from pinned host buffers, copies inside the timed region.  Every step uploads its own
    # inputs and downloads its own results; like a training loop with a prefetching loader, the upload of
    # step i+1 and the download of step i-1 run on side streams while step i computes (PCIe is full duplex),
    # over two sets of device buffers.
    host_out = [torch.empty_like(t).pin_memory() for t in (hq, hq, hk, hv)]
    compute = torch.cuda.current_stream()
    up_stream, down_stream = torch.cuda.Stream(), torch.cuda.Stream()
    dev_in = [[torch.empty_like(t, device=device) for t in (hq, hk, hv, hg)] for _ in range(2)]
    dev_mask = [None if hmask is None else torch.empty_like(hmask, device=device) for _ in range(2)]
    uploaded = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]
    downloaded = torch.cuda.Event()

    def e2e_run(count):
        keep = []
        for i in range(count):
            slot = i % 2
            with torch.cuda.stream(up_stream):
                if i >= 2:
                    up_stream.wait_event(consumed[slot])  # the step that last read this buffer set
                for dst, src in zip(dev_in[slot], (hq, hk, hv, hg)):
                    dst.copy_(src, non_blocking=True)
                if hmask is not None:
                    dev_mask[slot].copy_(hmask, non_blocking=True)
                uploaded[slot].record(up_stream)
            compute.wait_event(uploaded[slot])
            q, k, v = (t.detach().requires_grad_(True) for t in dev_in[slot][:3])
            results = step(q, k, v, dev_in[slot][3], dev_mask[slot])
            consumed[slot].record(compute)
            with torch.cuda.stream(down_stream):
                down_stream.wait_event(consumed[slot])
                if i >= 1:
                    down_stream.wait_event(downloaded)  # host_out is reused step after step
                for dst, src in zip(host_out, results):
                    dst.copy_(src.detach(), non_blocking=True)
                downloaded.record(down_stream)
            keep.append(results)  # alive until the downloads have run
        compute.wait_stream(down_stream)
        return keep

    e2e_run(2)
    barrier()
    b2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2e_steps = max(2, min(steps, 6))
    b2.record()
    held = e2e_run(e2e_steps)
    e2.record()
    barrier()
    del held
    e2e_ms = b2.elapsed_time(e2)

    times = torch.tensor([elapsed_ms, e2e_ms], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    elapsed_ms, e2e_ms = (float(x) for x in times.cpu())

    flops = algorithmic_flops(w)
    jobs = 1 if w.get("ring") else world  # a ring step is ONE job shared by all ranks
    value = flops * steps * jobs / (elapsed_ms * 1e-3) / 1e12
    e2e_value = flops * e2e_steps * jobs / (e2e_ms * 1e-3) / 1e12
    h2d = sum(t.numel() * t.element_size() for t in (hq, hk, hv, hg)) + (0 if hmask is None else hmask.numel())
    d2h = sum(t.numel() * t.element_size() for t in host_out)

    if rank == 0:
        burst, sustained, hbm, source = measured_peaks()
        # dominant kernel = largest share of device time among this library's kernels
        roofline = None
        if kernels:
            name, (total_ms, count) = max(kernels.items(), key=lambda item: item[1][0])
            # algorithmic GEMMs (of 7) attributed per kernel: forward 2; the dQ kernel 1 (dQ) + half of the shared
            # S/dP pair; the dK/dV kernel 2 (dK, dV) + the other half; every wide-head backward kernel forms one
            share = {"pipeline_forward": 2.0, "general_forward": 2.0, "neighborhood_forward": 2.0, "na_pipeline_forward": 2.0, "wide_forward": 2.0,
                     "wide_scores_p": 1.0, "wide_scores_ds": 1.0, "wide_grad": 3.0}.get(name)
            if share is None:
                share = 1.5 if name.endswith("_q") else 3.5
            per_step = max(1, int(round(count / prof_steps)))  # a ring step launches each kernel once per block
            per_launch = flops / (world if w.get("ring") else 1) * share / 7.0 / per_step
            achieved = per_launch / (total_ms / count * 1e-3) / 1e12
            peak = sustained or burst
            roofline = {"bound": "tensor", "kernel": name, "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                        "frac": achieved / peak, "traffic": None, "peak_source": f"{source} (sustained bf16 GEMM)",
                        "timing": f"CUDA events of a profiled pass of {prof_steps} steps after the timed region, kernels serialised",
                        "kernel_ms": total_ms / count,
                        "all_kernels_ms": {k: v[0] / v[1] for k, v in kernels.items()}}
        cpu = None
        if not args.no_cpu_baseline:
            cpu_value, cpu_seconds, sample = cpu_oracle_sample(w)
            cpu = {"value": cpu_value, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                   "sample": sample, "seconds": cpu_seconds}
        line = {
            "metric": "attn fwd+bwd TFLOP/s", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": steps,
            "warmup": warmup, "ms_per_step": elapsed_ms / steps, "higher_is_better": True,
            "scaling": "strong" if w.get("ring") else "weak",
            "vs_baseline": (value / world / w["published_tflops"]) if "published_tflops" in w else None,
            "dtype": w["dtype"], "data": "synthetic",
            "config": {"workload": w["name"], "launch": "cuda_graph" if use_graph else "eager", "B": w["B"], "Hq": w["Hq"], "Hkv": w["Hkv"], "S": w["S"], "D": w["D"],
                       "causal": w["causal"], "center_keys": w["center_keys"], "sharding": (f"ring context parallel, S/{world} per rank" if w.get("ring")
                                    else f"replica-per-gpu x{world}"),
                       "l2": "inputs larger than L2 (q+k+v+dO+O > 126 MB)" if h2d > 126e6 else (
                           f"steps rotate over {rotation} input sets, together larger than L2" if rotation > 1
                           else "inputs fit in L2"),
                       "input_stds": {"q": 8.0, "k_offset": 2.0, "dout": math.sqrt(1e-3)} if w["name"].startswith("llm_gqa") else None},
            "frac_of_peak": {"burst": value / world / burst, "sustained": value / world / sustained if sustained else None,
                             "source": source},
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms / e2e_steps, "steps": e2e_steps,
                    "overlap": "uploads and downloads of neighbouring steps run on side streams during compute"},
            "gpu_launches": launches, "clocks": clocks, "roofline": roofline, "cpu_baseline": cpu,
            "device_status": status,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
