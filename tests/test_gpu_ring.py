"""The CUDA pieces of ring context parallelism on one GPU: per-block forward + (max, log2-sum) merge,
and per-block backward against the global statistics, compared with the unsharded operator."""

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
