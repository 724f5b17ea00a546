"""The CUDA pieces of ring context parallelism on one GPU: the block-wise entry points (running FP32 state in
the forward epilogue, FP32 gradient contributions) driven through the ring schedule with all ranks emulated one
after another, and the older per-block forward + (max, log2-sum) merge; both against the unsharded operator
and the FP64 oracle."""

import pytest
import torch

from oracle import attention_oracle as ao
from tests.helpers import make_inputs

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("D,masked", ((128, False), (128, True), (64, True), (96, False)))
def test_blockwise_forward_merge_and_backward_match_the_full_operator(D, masked):
    from kohakufa_cute import native

    B, Hq, Hkv, S, blocks_n = 2, 4, 2, 512, 4
    q, k, v, dout = make_inputs(B, Hq, Hkv, S, S, D, torch.bfloat16, seed=91)
    scale = D ** -0.5
    key_mask = None
    if masked:
        key_mask = (torch.rand(B, 1, 1, S, generator=torch.Generator().manual_seed(92)) > 0.25).cuda()
        key_mask[..., 128:256] = False  # one block fully hidden
    full_mask = None if key_mask is None else key_mask.expand(B, Hq, S, S)
    out, maximum, logsum, blocks = native.forward(q, k, v, full_mask, scale, False)
    dq, dk, dv = native.backward(q, k, v, full_mask, maximum, logsum, dout, blocks, out, scale, False)

    acc = torch.zeros(B, Hq, S, D, device="cuda")
    acc_max = torch.full((B, Hq, S), float("-inf"), device="cuda")
    acc_log = torch.zeros(B, Hq, S, device="cuda")
    n = S // blocks_n
    for j in range(blocks_n):
        kb, vb = k[:, :, j * n:(j + 1) * n].contiguous(), v[:, :, j * n:(j + 1) * n].contiguous()
        mb = None if key_mask is None else key_mask[..., j * n:(j + 1) * n].contiguous().expand(B, Hq, S, n)
        part, pm, pl, _ = native.forward(q, kb, vb, mb, scale, False)
        native.merge_partial(acc, acc_max, acc_log, part, pm, pl, scale)
    torch.testing.assert_close(acc_max, maximum, atol=0, rtol=0)
    torch.testing.assert_close(acc_log, logsum, atol=2e-3, rtol=1e-4)
    assert ao.per_head_relative_error(acc.cpu(), out.float().cpu().double()) < 0.006
    merged = acc.to(q.dtype)

    dq_acc = torch.zeros_like(acc)
    dks, dvs = [], []
    for j in range(blocks_n):
        kb, vb = k[:, :, j * n:(j + 1) * n].contiguous(), v[:, :, j * n:(j + 1) * n].contiguous()
        mb = None if key_mask is None else key_mask[..., j * n:(j + 1) * n].contiguous().expand(B, Hq, S, n)
        tb = None if mb is None else native.pack_mask(q, kb, mb)
        a, b_, c = native.backward(q, kb, vb, mb, acc_max, acc_log, dout, tb, merged, scale, False)
        dq_acc += a.float()
        dks.append(b_)
        dvs.append(c)
    assert ao.per_head_relative_error(dq_acc.cpu(), dq.float().cpu().double()) < 0.01
    assert ao.per_head_relative_error(torch.cat(dks, 2).cpu(), dk.float().cpu().double()) < 0.01
    assert ao.per_head_relative_error(torch.cat(dvs, 2).cpu(), dv.float().cpu().double()) < 0.01


def _emulated_ring(q, k, v, dout, key_mask, scale, causal, world):
    """Runs the schedule of ``parallel.ring_forward`` / ``ring_backward`` for every rank on this GPU (no
    communication: the block a rank would hold in a step is taken from its owner's shard directly)."""
    from kohakufa_cute import parallel

    K = parallel.PipelineBlocks
    B, Hq = q.shape[:2]
    if causal:
        shard = lambda t, rank, dim=2: parallel.zigzag_shard(t, world, rank, dim).contiguous()
    else:
        shard = lambda t, rank, dim=2: t.narrow(dim, rank * (t.shape[dim] // world), t.shape[dim] // world).contiguous()
    outs, stats, dqs = [], [], []
    totals = [None] * world
    for rank in range(world):
        ql, gl = shard(q, rank), shard(dout, rank)
        half = ql.shape[2] // 2
        state = K.new_state(ql)
        for step in range(world):
            source = (rank - step) % world
            kb, vb = shard(k, source), shard(v, source)
            mb = None if key_mask is None else shard(key_mask, source, 3)
            rows, keys, flag = parallel._step_views(step, source, rank, causal, half)
            qs, ks = ql[:, :, rows], kb[:, :, keys]
            mask = None if mb is None else mb[..., keys].expand(B, Hq, qs.shape[2], ks.shape[2])
            K.forward_block(qs, ks, vb[:, :, keys], mask, tuple(t[:, :, rows] for t in state), scale, flag)
        out, maximum, logsum = K.finish(state, q.dtype)
        outs.append(out)
        stats.append((maximum, logsum))
        dq = torch.zeros(ql.shape, device="cuda")
        upper = (maximum[:, :, half:].contiguous(), logsum[:, :, half:].contiguous())
        for step in range(world):
            source = (rank - step) % world
            kb, vb = shard(k, source), shard(v, source)
            mb = None if key_mask is None else shard(key_mask, source, 3)
            rows, keys, flag = parallel._step_views(step, source, rank, causal, half)
            qs, ks = ql[:, :, rows], kb[:, :, keys]
            mask = None if mb is None else mb[..., keys].expand(B, Hq, qs.shape[2], ks.shape[2])
            part = [torch.full(kb.shape, float("nan"), device="cuda") for _ in range(2)]
            st = (maximum, logsum) if rows == slice(None) else upper
            K.backward_block(qs, ks, vb[:, :, keys], mask, out[:, :, rows], st[0], st[1], gl[:, :, rows], scale, flag,
                             dq[:, :, rows], part[0][:, :, keys], part[1][:, :, keys])
            if totals[source] is None:
                totals[source] = [torch.zeros(kb.shape, device="cuda") for _ in range(2)]
            totals[source][0][:, :, keys] += part[0][:, :, keys]
            totals[source][1][:, :, keys] += part[1][:, :, keys]
        dqs.append(dq)
    assert all(bool(torch.isfinite(t).all()) for pair in totals for t in pair)
    if causal:
        join = parallel.zigzag_unshard
    else:
        join = lambda parts, dim=2: torch.cat(parts, dim)
    return (join(outs), join([m for m, _ in stats]), join([l for _, l in stats]), join(dqs),
            join([t[0] for t in totals]), join([t[1] for t in totals]))


@pytest.mark.parametrize("D,masked,causal,world,S", (
    (128, False, True, 4, 1536), (128, True, False, 4, 1536), (64, False, True, 2, 1536), (96, True, True, 3, 1536),
    (128, False, False, 2, 1536),
    (128, True, False, 2, 1210), (96, False, True, 3, 1212),  # ragged shards: rows beyond the end inside a warp
))
def test_running_state_blocks_over_the_ring_schedule(D, masked, causal, world, S):
    from kohakufa_cute import native

    B, Hq, Hkv = 1, 4, 2
    q, k, v, dout = make_inputs(B, Hq, Hkv, S, S, D, torch.bfloat16, seed=95)
    scale = D ** -0.5
    key_mask = None
    if masked:
        key_mask = (torch.rand(B, 1, 1, S, generator=torch.Generator().manual_seed(96)) > 0.25).cuda()
        key_mask[..., 256:384] = False  # a whole tile of keys hidden
        key_mask[..., :2] = True
    full_mask = None if key_mask is None else key_mask.expand(B, Hq, S, S)
    out, maximum, logsum, blocks = native.forward(q, k, v, full_mask, scale, causal)
    ring = _emulated_ring(q, k, v, dout, key_mask, scale, causal, world)
    # statistics: the same exact maximum; log2-sum up to FP32 summation order
    torch.testing.assert_close(ring[1], maximum, atol=0, rtol=0)
    torch.testing.assert_close(ring[2], logsum, atol=2e-3, rtol=1e-4)
    exact = ao.math_reference((q.cpu(), k.cpu(), v.cpu()), dout.cpu(), None if full_mask is None else full_mask.cpu(),
                              causal, scale)
    # gates of the operator itself (1 % per head against FP64 mathematics): FP32 between blocks, so the
    # block-wise results are held to what a single call is held to
    for name, got, want in zip(("out", "dq", "dk", "dv"), (ring[0], ring[3], ring[4], ring[5]), exact):
        err = ao.per_head_relative_error(got.float().cpu(), want)
        assert err < 0.01, (name, err)
    # and no further from the exact values than the single-call operator is, plus a little summation noise
    dq, dk, dv = native.backward(q, k, v, full_mask, maximum, logsum, dout, blocks, out, scale, causal)
    for name, got, single, want in zip(("out", "dq", "dk", "dv"), (ring[0], ring[3], ring[4], ring[5]),
                                       (out, dq, dk, dv), exact):
        ring_err = ao.per_head_relative_error(got.float().cpu(), want)
        single_err = ao.per_head_relative_error(single.float().cpu(), want)
        assert ring_err < 1.25 * single_err + 1e-4, (name, ring_err, single_err)


def test_blockwise_entry_points_reject_other_families():
    from kohakufa_cute import native

    q, k, v, _ = make_inputs(1, 2, 2, 256, 256, 256, torch.bfloat16, seed=97)
    state = native.running_state(q)
    with pytest.raises(ValueError, match="pipeline family"):
        native.forward_running(q, k, v, None, state, 0.1)


def test_ring_attention_on_a_single_rank_equals_attention():
    import os

    import torch.distributed as dist

    import kohakufa_cute
    from kohakufa_cute import parallel

    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    created = not dist.is_initialized()
    if created:
        dist.init_process_group("gloo", rank=0, world_size=1)
    try:
        q, k, v, dout = make_inputs(1, 4, 2, 300, 300, 128, torch.bfloat16, seed=93)
        leaves = [t.clone().requires_grad_(True) for t in (q, k, v)]
        out = parallel.ring_attention(*leaves)
        grads = torch.autograd.grad(out, leaves, dout)
        ref_leaves = [t.clone().requires_grad_(True) for t in (q, k, v)]
        ref = kohakufa_cute.attention(*ref_leaves)
        ref_grads = torch.autograd.grad(ref, ref_leaves, dout)
        torch.testing.assert_close(out, ref, atol=0.01, rtol=0.01)
        for a, b in zip(grads, ref_grads):
            torch.testing.assert_close(a, b, atol=0.02, rtol=0.02)
    finally:
        if created:
            dist.destroy_process_group()
