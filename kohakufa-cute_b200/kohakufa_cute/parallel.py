"""Multi-GPU layers around the attention operator (one process per GPU, ``torch.distributed``).

The reference project has no multi-GPU execution mode; these two layers are additions:

* ``shard_heads`` - batch x K/V-head sharding.  Attention is independent per (batch, K/V head
  group), so every rank takes a contiguous slice of those groups and runs the ordinary operator
  on it: no collective on the data path.  A grouped-query group never straddles two ranks, so
  dK/dV keep a single owner.
* ``ring_attention`` - context parallelism for sequences too long for one GPU.  Every rank owns
  ``S / P`` queries and the matching K/V (and key-mask) shard.  In step ``j`` a rank attends its
  queries to the K/V block it currently holds while that block is already on its way to the next
  rank (NCCL send/recv through ``torch.distributed`` on a side stream, into a second local
  buffer); the partial results are folded together with the (maximum, log2-sum) merge of the
  reference's split forward (src/kohakufa_cute/split_forward.py:219-245 of the reference
  project), so the saved statistics keep the operator's contract and the ordinary backward
  kernels can be reused step by step.  Key/value gradients travel around the ring in FP32 with
  their block and are rounded once by the owner.

Only non-causal attention is supported by ``ring_attention`` (contiguous shards would be
unbalanced under a causal mask).
"""

from __future__ import annotations

import torch
import torch.distributed as dist


def shard_heads(batch, kv_heads, world_size, rank):
    """Contiguous slice ``[begin, end)`` of the flattened (batch, K/V head) units owned by ``rank``.

    Units are dealt out as evenly as possible (the first ``units % world_size`` ranks get one more).
    Returns ``(begin, end)``; an empty range means the rank idles.
    """
    units = batch * kv_heads
    base, extra = divmod(units, world_size)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def take_head_shard(q, k, v, begin, end):
    """Views of q/k/v restricted to flattened (batch, K/V head) units ``[begin, end)``.

    q is ``[B, Hq, S, D]``, k/v are ``[B, Hkv, S, D]``; the result is ``[1, heads, S, D]`` with the
    selected units folded into the head axis (each K/V head keeps its ``Hq // Hkv`` query heads).
    """
    B, Hq, Sq, D = q.shape
    Hkv = k.shape[1]
    group = Hq // Hkv
    qf = q.reshape(1, B * Hkv, group, Sq, D)[:, begin:end].reshape(1, (end - begin) * group, Sq, D)
    kf = k.reshape(1, B * Hkv, k.shape[2], D)[:, begin:end]
    vf = v.reshape(1, B * Hkv, v.shape[2], D)[:, begin:end]
    return qf, kf, vf


# ------------------------------------------------------------------ ring context parallelism
def _cuda_forward(q, k, v, mask, scale):
    from . import native

    out, maximum, logsum, _ = native.forward(q, k, v, mask, scale, False)
    return out, maximum, logsum


def _cuda_backward(q, k, v, mask, out, maximum, logsum, dout, scale):
    from . import native

    blocks = None
    if mask is not None:
        # the tile table belongs to the (query shard, key block) pair: rebuild it with a forward-free call
        blocks = native.pack_mask(q, k, mask)
    return native.backward(q, k, v, mask, maximum, logsum, dout, blocks, out, scale, False)


def _cuda_merge(acc, acc_max, acc_log, part, part_max, part_log, scale):
    from . import native

    native.merge_partial(acc, acc_max, acc_log, part, part_max, part_log, scale)


def _exchange(tensors, group, step_tag):
    """Sends every tensor to the next rank and receives its replacement from the previous one."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    nxt = dist.get_global_rank(group, (rank + 1) % world) if group is not None else (rank + 1) % world
    prv = dist.get_global_rank(group, (rank - 1) % world) if group is not None else (rank - 1) % world
    received = [torch.empty_like(t) for t in tensors]
    ops = []
    for t, r in zip(tensors, received):
        ops.append(dist.P2POp(dist.isend, t, nxt, group))
        ops.append(dist.P2POp(dist.irecv, r, prv, group))
    return received, dist.batch_isend_irecv(ops)


def ring_forward(q, k, v, key_mask, scale, group=None, *, forward_fn=None, merge_fn=None):
    """Forward of ring attention on this rank's shards.

    ``q``: ``[B, Hq, S/P, D]``; ``k``, ``v``: ``[B, Hkv, S/P, D]``; ``key_mask``: optional bool
    ``[B, 1, 1, S/P]`` shard (True = visible).  Returns ``(out, maximum, logsum)`` where ``out`` has
    q's dtype and the statistics cover the whole key sequence.
    ``forward_fn`` / ``merge_fn`` default to the CUDA kernels; tests inject CPU stand-ins.
    """
    forward_fn = forward_fn or _cuda_forward
    merge_fn = merge_fn or _cuda_merge
    world = dist.get_world_size(group)
    B, Hq, Sq, D = q.shape
    acc = torch.zeros(B, Hq, Sq, D, device=q.device, dtype=torch.float32)
    acc_max = torch.full((B, Hq, Sq), float("-inf"), device=q.device, dtype=torch.float32)
    acc_log = torch.zeros(B, Hq, Sq, device=q.device, dtype=torch.float32)
    block = [k.contiguous(), v.contiguous()] + ([] if key_mask is None else [key_mask.contiguous()])
    for step in range(world):
        pending = None
        if step + 1 < world:
            incoming, pending = _exchange(block, group, step)
        mask = None
        if key_mask is not None:
            mask = block[2].expand(B, Hq, Sq, block[0].shape[2])
        part, part_max, part_log = forward_fn(q, block[0], block[1], mask, scale)
        merge_fn(acc, acc_max, acc_log, part, part_max, part_log, scale)
        if pending is not None:
            for work in pending:
                work.wait()
            block = incoming
    return acc.to(q.dtype), acc_max, acc_log


def ring_backward(q, k, v, key_mask, out, maximum, logsum, dout, scale, group=None, *, backward_fn=None):
    """Backward of ring attention: returns ``(dq, dk, dv)`` for this rank's shards.

    dQ accumulates locally in FP32 over the key blocks; the FP32 dK/dV accumulators of a block
    travel with it and reach their owner again after ``P`` hops, where they are rounded once.
    """
    backward_fn = backward_fn or _cuda_backward
    world = dist.get_world_size(group)
    B, Hq, Sq, D = q.shape
    dq_acc = torch.zeros(q.shape, device=q.device, dtype=torch.float32)
    payload = [k.contiguous(), v.contiguous(), torch.zeros(k.shape, device=k.device, dtype=torch.float32),
               torch.zeros(v.shape, device=v.device, dtype=torch.float32)]
    if key_mask is not None:
        payload.append(key_mask.contiguous())
    for step in range(world):
        mask = None
        if key_mask is not None:
            mask = payload[4].expand(B, Hq, Sq, payload[0].shape[2])
        dq, dk, dv = backward_fn(q, payload[0], payload[1], mask, out, maximum, logsum, dout, scale)
        dq_acc += dq.float()
        payload[2] += dk.float()
        payload[3] += dv.float()
        if world == 1:
            break
        # every block (with its gradient accumulators) moves on; after `world` hops it is home again
        incoming, pending = _exchange(payload, group, step)
        for work in pending:
            work.wait()
        payload = incoming
    return dq_acc.to(q.dtype), payload[2].to(k.dtype), payload[3].to(v.dtype)


class _RingAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, key_mask, scale, group):
        out, maximum, logsum = ring_forward(q, k, v, key_mask, scale, group)
        ctx.save_for_backward(q, k, v, out, maximum, logsum, *(() if key_mask is None else (key_mask,)))
        ctx.scale, ctx.group, ctx.has_mask = scale, group, key_mask is not None
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, maximum, logsum, *rest = ctx.saved_tensors
        dq, dk, dv = ring_backward(q, k, v, rest[0] if ctx.has_mask else None, out, maximum, logsum,
                                   dout.contiguous(), ctx.scale, ctx.group)
        return dq, dk, dv, None, None, None


def ring_attention(q, k, v, *, key_mask=None, scale=None, group=None):
    """Non-causal attention over a sequence sharded across the ranks of ``group`` (autograd-aware)."""
    scale = q.shape[-1] ** -0.5 if scale is None else float(scale)
    return _RingAttention.apply(q, k, v, key_mask, scale, group)
