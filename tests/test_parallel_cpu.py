"""Host logic of the multi-GPU layers, run as gloo ranks on the CPU (world size 2, 3 and 4).

The CUDA kernels are replaced by CPU stand-ins built on the oracle, so these tests cover the
sharding arithmetic, the ring schedule (who holds which block when, also under the causal zig-zag layout),
the running (maximum, sum) state and the travelling FP32 gradient totals - not the kernels themselves.
"""

import math
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import attention_oracle as ao


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


# ---- CPU stand-ins with the block-wise kernels' calling convention ---------------------------
def _visible(q, k, mask, causal):
    visible = torch.ones(q.shape[0], q.shape[1], q.shape[2], k.shape[2], dtype=torch.bool)
    if mask is not None:
        visible &= mask
    if causal:
        visible &= torch.ones(q.shape[2], k.shape[2], dtype=torch.bool).tril()
    return visible


class CpuBlocks:
    """FP64 arithmetic behind the interface of ``parallel.PipelineBlocks`` (state and gradients are FP32
    tensors updated in place, also through views)."""

    @staticmethod
    def new_state(q):
        acc = torch.zeros(q.shape, dtype=torch.float32)
        run_maximum = torch.full(q.shape[:-1], float("-inf"), dtype=torch.float32)
        return acc, run_maximum, torch.zeros_like(run_maximum)

    @staticmethod
    def forward_block(q, k, v, mask, state, scale, causal):
        acc, run_maximum, run_sum = state
        group = q.shape[1] // k.shape[1]
        keys, values = k.repeat_interleave(group, 1).double(), v.repeat_interleave(group, 1).double()
        s = (q.double() @ keys.transpose(-1, -2)) * (1 if scale >= 0 else -1)
        s = s.masked_fill(~_visible(q, k, mask, causal), float("-inf"))
        c2 = abs(scale) * math.log2(math.e)
        new = torch.maximum(run_maximum.double(), s.amax(-1))
        safe = torch.where(torch.isinf(new), torch.zeros_like(new), new)
        p = torch.exp2((s - safe[..., None]) * c2)
        w_old = torch.where(torch.isinf(run_maximum), torch.zeros_like(new), torch.exp2((run_maximum.double() - safe) * c2))
        acc.copy_(acc.double() * w_old[..., None] + p @ values)
        run_sum.copy_(run_sum.double() * w_old + p.sum(-1))
        run_maximum.copy_(new)

    @staticmethod
    def finish(state, dtype):
        acc, run_maximum, run_sum = state
        seen = run_sum > 0
        out = torch.where(seen[..., None], acc / run_sum[..., None], torch.zeros_like(acc)).to(dtype)
        return out, run_maximum, torch.where(seen, torch.log2(run_sum), torch.zeros_like(run_sum))

    @staticmethod
    def backward_block(q, k, v, mask, out, maximum, logsum, dout, scale, causal, dq, dk, dv):
        """Contributions of one (query rows, key block) pair given the statistics of the WHOLE sequence."""
        assert maximum.is_contiguous() and logsum.is_contiguous()  # the CUDA entry point requires dense statistics
        group = q.shape[1] // k.shape[1]
        keys, values = k.repeat_interleave(group, 1).double(), v.repeat_interleave(group, 1).double()
        s = (q.double() @ keys.transpose(-1, -2)) * (1 if scale >= 0 else -1)
        c2 = abs(scale) * math.log2(math.e)
        p = torch.exp2((s - maximum.double()[..., None]) * c2 - logsum.double()[..., None])
        p = p.masked_fill(~_visible(q, k, mask, causal), 0.0)
        delta = (out.double() * dout.double()).sum(-1, keepdim=True)
        ds = p * (dout.double() @ values.transpose(-1, -2) - delta)
        dq.add_(((ds @ keys) * scale).float())
        dk.copy_(((ds.transpose(-1, -2) @ q.double()) * scale).reshape(k.shape[0], k.shape[1], group, *k.shape[2:]).sum(2))
        dv.copy_((p.transpose(-1, -2) @ dout.double()).reshape(v.shape[0], v.shape[1], group, *v.shape[2:]).sum(2))


def _ring_worker(rank, world, port, masked, causal, result):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from kohakufa_cute import parallel

        gen = torch.Generator().manual_seed(7)
        B, Hq, Hkv, S, D = 1, 4, 2, 24 * world, 16
        q, k, v, g = (torch.randn(B, h, S, D, generator=gen).bfloat16() for h in (Hq, Hkv, Hkv, Hq))
        mask = None
        if masked:
            mask = (torch.rand(B, 1, 1, S, generator=gen) > 0.3)
            mask[..., :3] = True
        scale = -0.2
        if causal:
            def shard(t, dim=2):
                return parallel.zigzag_shard(t, world, rank, dim).contiguous()
        else:
            def shard(t, dim=2):
                n = t.shape[dim] // world
                return t.narrow(dim, rank * n, n).contiguous()
        ql, kl, vl, gl = (shard(t) for t in (q, k, v, g))
        ml = None if mask is None else shard(mask, 3)
        out, maximum, logsum = parallel.ring_forward(ql, kl, vl, ml, scale, causal=causal, kernels=CpuBlocks)
        dq, dk, dv = parallel.ring_backward(ql, kl, vl, ml, out, maximum, logsum, gl, scale, causal=causal,
                                            kernels=CpuBlocks)
        full_mask = None if mask is None else mask.expand(B, Hq, S, S)
        exact = ao.math_reference((q, k, v), g, full_mask, causal, scale)
        want_max, want_log = ao.forward_statistics((q, k, v), full_mask, causal, scale)
        errs = dict(
            out=ao.relative_error(out, shard(exact[0])), dq=ao.relative_error(dq, shard(exact[1])),
            dk=ao.relative_error(dk, shard(exact[2])), dv=ao.relative_error(dv, shard(exact[3])),
            maximum=float((maximum.double() - shard(want_max)).abs().max()),
            logsum=float((logsum.double() - shard(want_log)).abs().max()),
        )
        result[rank] = errs
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,masked,causal", ((2, False, False), (2, True, False), (3, True, False),
                                                 (2, False, True), (3, False, True), (3, True, True),
                                                 (4, True, True)))
def test_ring_schedule_and_merge_on_cpu_ranks(world, masked, causal):
    manager = mp.Manager()
    result = manager.dict()
    mp.spawn(_ring_worker, args=(world, _free_port(), masked, causal, result), nprocs=world, join=True)
    assert len(result) == world
    for rank in range(world):
        errs = result[rank]
        for name in ("out", "dq", "dk", "dv"):
            # 16-bit rounding of the final results only: the stand-ins keep FP32/FP64 between blocks
            assert errs[name] < 0.006, (rank, name, errs[name])
        assert errs["maximum"] < 1e-4 and errs["logsum"] < 1e-3, (rank, errs)


def test_zigzag_shards_balance_the_causal_work():
    """Every rank sees the same number of (query, key) pairs in every step of the causal schedule."""
    from kohakufa_cute import parallel

    for world in (2, 3, 8):
        chunk = 5
        position = torch.arange(2 * world * chunk)
        per_rank = []
        for rank in range(world):
            own = parallel.zigzag_shard(position[None, None, :, None], world, rank)[0, 0, :, 0]
            steps = []
            for step in range(world):
                source = (rank - step) % world
                block = parallel.zigzag_shard(position[None, None, :, None], world, source)[0, 0, :, 0]
                rows, keys, flag = parallel._step_views(step, source, rank, True, chunk)
                qs, ks = own[rows], block[keys]
                seen = (ks[None, :] <= qs[:, None])
                if flag:
                    assert torch.equal(seen, torch.ones(len(qs), len(ks), dtype=torch.bool).tril())
                else:
                    assert bool(seen.all())
                # nothing outside the views is visible
                everything = int((block[None, :] <= own[:, None]).sum())
                assert everything == int(seen.sum())
                steps.append(everything)
            per_rank.append(steps)
        assert all(steps[1:] == per_rank[0][1:] for steps in per_rank)
        shards = [parallel.zigzag_shard(position[None, None, :, None], world, r) for r in range(world)]
        assert torch.equal(parallel.zigzag_unshard(shards), position[None, None, :, None])


def test_head_sharding_covers_every_unit_once():
    from kohakufa_cute import parallel

    for units, world in ((32, 8), (48, 8), (16, 3), (5, 8), (1, 2)):
        seen = []
        for rank in range(world):
            begin, end = parallel.shard_heads(units, 1, world, rank)
            seen.extend(range(begin, end))
            assert 0 <= end - begin <= math.ceil(units / world)
        assert seen == list(range(units))


def test_head_shard_views_keep_groups_together():
    from kohakufa_cute import parallel

    B, Hq, Hkv, S, D = 2, 8, 2, 5, 4
    q = torch.arange(B * Hq * S * D, dtype=torch.float32).reshape(B, Hq, S, D)
    k = torch.arange(B * Hkv * S * D, dtype=torch.float32).reshape(B, Hkv, S, D)
    qf, kf, vf = parallel.take_head_shard(q, k, k, 1, 3)  # units (b0,h1) and (b1,h0)
    assert qf.shape == (1, 8, S, D) and kf.shape == (1, 2, S, D)
    assert torch.equal(kf[0, 0], k[0, 1]) and torch.equal(kf[0, 1], k[1, 0])
    assert torch.equal(qf[0, :4], q[0, 4:8]) and torch.equal(qf[0, 4:], q[1, 0:4])


def _timeout_worker(rank, world, port, result):
    """A rank that never joins the exchange must surface as an error on the others, not a hang."""
    import datetime

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    try:
        from kohakufa_cute import parallel

        q = torch.zeros(1, 1, 4, 8, dtype=torch.bfloat16)
        if rank == 1:
            result[rank] = "skipped"  # injected fault: this rank drops out before the ring starts
            return
        try:
            parallel.ring_forward(q, q, q, None, 1.0, kernels=CpuBlocks)
            result[rank] = "no error"
        except Exception as error:  # noqa: BLE001 - any distributed error is the expected outcome
            result[rank] = "error: " + type(error).__name__
    finally:
        try:
            dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass


def test_a_rank_that_drops_out_is_reported_not_hung():
    manager = mp.Manager()
    result = manager.dict()
    mp.spawn(_timeout_worker, args=(2, _free_port(), result), nprocs=2, join=True)
    assert result[1] == "skipped"
    assert result[0].startswith("error"), result[0]
