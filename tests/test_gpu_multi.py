"""Two-GPU tests (skipped on a single-GPU box): ring context parallelism over NCCL against the
unsharded operator, and head sharding.  NVLS is switched off for the child processes."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import kohakufa_cute
        from kohakufa_cute import parallel

        gen = torch.Generator().manual_seed(11)
        B, Hq, Hkv, S, D = 1, 4, 2, 1024, 128
        q, k, v, g = (torch.randn(B, h, S, D, generator=gen).bfloat16() for h in (Hq, Hkv, Hkv, Hq))
        mask = torch.rand(B, 1, 1, S, generator=gen) > 0.2
        n = S // world
        sl = slice(rank * n, (rank + 1) * n)
        dev = torch.device("cuda", rank)
        leaves = [t[:, :, sl].contiguous().to(dev).requires_grad_(True) for t in (q, k, v)]
        out = parallel.ring_attention(*leaves, key_mask=mask[..., sl].contiguous().to(dev))
        grads = torch.autograd.grad(out, leaves, g[:, :, sl].contiguous().to(dev))
        full = [t.to(dev).requires_grad_(True) for t in (q, k, v)]
        ref = kohakufa_cute.attention(*full, mask=mask.to(dev))
        ref_grads = torch.autograd.grad(ref, full, g.to(dev))
        def per_head(got, want):
            """Largest relative L2 error over the (batch, head) slices (the operator's own 1 % gate)."""
            diff = (got.float() - want.float()).flatten(2).norm(dim=2)
            return float((diff / want.float().flatten(2).norm(dim=2)).max())

        errs = [per_head(out, ref[:, :, sl])]
        for a, b in zip(grads, ref_grads):
            errs.append(per_head(a, b[:, :, sl]))
        # causal, zig-zag shards (the block-wise FP32 entry points underneath), relative L2 error per tensor
        shard = lambda t: parallel.zigzag_shard(t, world, rank).contiguous().to(dev)
        leaves = [shard(t).requires_grad_(True) for t in (q, k, v)]
        out = parallel.ring_attention(*leaves, causal=True)
        grads = torch.autograd.grad(out, leaves, shard(g))
        full = [t.to(dev).requires_grad_(True) for t in (q, k, v)]
        ref = kohakufa_cute.attention(*full, causal=True)
        ref_grads = torch.autograd.grad(ref, full, g.to(dev))
        for a, b in zip((out,) + tuple(grads), (ref,) + tuple(ref_grads)):
            errs.append(per_head(a, parallel.zigzag_shard(b, world, rank)))
        # head sharding: this rank's units give the same numbers as the same units of the full call
        begin, end = parallel.shard_heads(B, Hkv, world, rank)
        qs, ks, vs = parallel.take_head_shard(q.to(dev), k.to(dev), v.to(dev), begin, end)
        part = kohakufa_cute.attention(qs, ks, vs, causal=True)
        whole = kohakufa_cute.attention(q.to(dev), k.to(dev), v.to(dev), causal=True)
        group = Hq // Hkv
        same = torch.equal(part[0], whole.reshape(B * Hkv, group, S, D)[begin:end].reshape(-1, S, D))
        result[rank] = (errs, same)
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_ring_attention_and_head_sharding_on_two_gpus():
    manager = mp.Manager()
    result = manager.dict()
    mp.spawn(_worker, args=(2, _free_port(), result), nprocs=2, join=True)
    for rank in range(2):
        errs, same = result[rank]
        # masked ring, then causal ring: out, dq, dk, dv per head against the unsharded operator
        assert all(e < 0.01 for e in errs), errs
        assert same
