"""Host logic of the multi-GPU layers, run as gloo ranks on the CPU (world size 2 and 3).

The CUDA kernels are replaced by CPU stand-ins built on the oracle, so these tests cover the
sharding arithmetic, the ring schedule (who holds which block when), the (maximum, log2-sum) merge
and the travelling FP32 gradient accumulators - not the kernels themselves.
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


# ---- CPU stand-ins with the kernels' calling convention -------------------------------------
def cpu_forward(q, k, v, mask, scale):
    out = ao.contract_reference((q, k, v), torch.zeros_like(q), mask, False, scale)[0]
    maximum, logsum = ao.forward_statistics((q, k, v), mask, False, scale)
    return out.to(q.dtype), maximum.float(), logsum.float()


def cpu_merge(acc, acc_max, acc_log, part, part_max, part_log, scale):
    c2 = abs(scale) * math.log2(math.e)
    m = torch.maximum(acc_max, part_max)
    safe = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    w0 = torch.where(torch.isinf(acc_max), torch.zeros_like(m), torch.exp2((acc_max - safe) * c2 + acc_log))
    w1 = torch.where(torch.isinf(part_max), torch.zeros_like(m), torch.exp2((part_max - safe) * c2 + part_log))
    total = w0 + w1
    inv = torch.where(total > 0, 1 / total, torch.zeros_like(total))
    acc.copy_((acc * w0[..., None] + part.float() * w1[..., None]) * inv[..., None])
    acc_max.copy_(m)
    acc_log.copy_(torch.where(total > 0, torch.log2(total), torch.zeros_like(total)))


def cpu_backward(q, k, v, mask, out, maximum, logsum, dout, scale):
    """Backward of one (query shard, key block) pair given the GLOBAL statistics."""
    group = q.shape[1] // k.shape[1]
    keys, values = k.repeat_interleave(group, 1).double(), v.repeat_interleave(group, 1).double()
    s = (q.double() @ keys.transpose(-1, -2)) * (1 if scale >= 0 else -1)
    c2 = abs(scale) * math.log2(math.e)
    p = torch.exp2((s - maximum.double()[..., None]) * c2 - logsum.double()[..., None])
    if mask is not None:
        p = p.masked_fill(~mask, 0.0)
    delta = (out.double() * dout.double()).sum(-1, keepdim=True)
    ds = p * (dout.double() @ values.transpose(-1, -2) - delta)
    dq = (ds @ keys) * scale
    dk = ((ds.transpose(-1, -2) @ q.double()) * scale).reshape(k.shape[0], k.shape[1], group, *k.shape[2:]).sum(2)
    dv = (p.transpose(-1, -2) @ dout.double()).reshape(v.shape[0], v.shape[1], group, *v.shape[2:]).sum(2)
    return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype)


def _ring_worker(rank, world, port, masked, result):
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
        n = S // world
        sl = slice(rank * n, (rank + 1) * n)
        ql, kl, vl, gl = (t[:, :, sl].contiguous() for t in (q, k, v, g))
        ml = None if mask is None else mask[..., sl].contiguous()
        out, maximum, logsum = parallel.ring_forward(ql, kl, vl, ml, scale, forward_fn=cpu_forward, merge_fn=cpu_merge)
        dq, dk, dv = parallel.ring_backward(ql, kl, vl, ml, out, maximum, logsum, gl, scale, backward_fn=cpu_backward)
        exact = ao.math_reference((q, k, v), g, mask, False, scale)
        want_max, want_log = ao.forward_statistics((q, k, v), mask, False, scale)
        errs = dict(
            out=ao.relative_error(out, exact[0][:, :, sl]), dq=ao.relative_error(dq, exact[1][:, :, sl]),
            dk=ao.relative_error(dk, exact[2][:, :, sl]), dv=ao.relative_error(dv, exact[3][:, :, sl]),
            maximum=float((maximum.double() - want_max[:, :, sl]).abs().max()),
            logsum=float((logsum.double() - want_log[:, :, sl]).abs().max()),
        )
        result[rank] = errs
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,masked", ((2, False), (2, True), (3, True)))
def test_ring_schedule_and_merge_on_cpu_ranks(world, masked):
    manager = mp.Manager()
    result = manager.dict()
    mp.spawn(_ring_worker, args=(world, _free_port(), masked, result), nprocs=world, join=True)
    assert len(result) == world
    for rank in range(world):
        errs = result[rank]
        for name in ("out", "dq", "dk", "dv"):
            assert errs[name] < 0.02, (rank, name, errs[name])
        assert errs["maximum"] < 1e-4 and errs["logsum"] < 1e-3, (rank, errs)


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
            parallel.ring_forward(q, q, q, None, 1.0, forward_fn=cpu_forward, merge_fn=cpu_merge)
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
