"""CPU checks of the benchmark's workload table: algorithmic FLOP counts and ring sharding."""

import importlib.util
import math
import os

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("kfa_bench", os.path.join(ROOT, "bench.py"))
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def test_algorithmic_flops_follow_the_visible_pairs():
    bench = _bench()
    w = bench.WORKLOADS
    # causal square: 3.5 * 4 * B * Hq * D * S^2 / 2
    assert math.isclose(bench.algorithmic_flops(w["llm_gqa"]), 3.5 * 4 * 4 * 32 * 128 * 4096 ** 2 / 2)
    assert math.isclose(bench.algorithmic_flops(w["wide_head"]), 3.5 * 4 * 16 * 512 * 1024 ** 2 / 2)
    # key padding: only the visible 90 % of the keys count
    visible = 32768 - int(32768 * 0.1 + 0.5)
    assert math.isclose(bench.algorithmic_flops(w["dit_masked"]), 3.5 * 4 * 2 * 24 * 128 * 32768 * visible)
    # neighbourhood: every query sees prod(window) keys
    assert math.isclose(bench.algorithmic_flops(w["neighborhood_3d"]), 3.5 * 4 * 16 * 64 * 16384 * 147)
    # the published 2-D figure: 151.28 us for this many FLOPs
    n2 = w["neighborhood_2d"]
    assert math.isclose(n2["published_tflops"], bench.algorithmic_flops(n2) / 151.28e-6 / 1e12)


def test_ring_workload_shards_the_sequence_and_its_mask():
    bench = _bench()
    w = dict(bench.WORKLOADS["dit_ring_small"], name="dit_ring_small", S=2048, Hq=2, Hkv=2, D=64)
    world = 4
    keep = 2048 - int(2048 * 0.1 + 0.5)
    seen = 0
    for rank in range(world):
        (q, k, v, g), mask = bench.make_host_inputs(w, rank, world)
        assert q.shape == (1, 2, 512, 64) and k.shape == v.shape == (1, 2, 512, 64) and g.shape == q.shape
        assert mask.shape == (1, 1, 1, 512) and mask.dtype == torch.bool
        want = torch.arange(rank * 512, (rank + 1) * 512) < keep
        assert torch.equal(mask[0, 0, 0], want)
        seen += int(mask.sum())
    assert seen == keep
    # different ranks draw different data
    (q0, *_), _ = bench.make_host_inputs(w, 0, world)
    (q1, *_), _ = bench.make_host_inputs(w, 1, world)
    assert not torch.equal(q0, q1)
