"""Multi-GPU layers around the attention operator (one process per GPU, ``torch.distributed``).

The reference project has no multi-GPU execution mode; these two layers are additions:

* ``shard_heads`` - batch x K/V-head sharding.  Attention is independent per (batch, K/V head
  group), so every rank takes a contiguous slice of those groups and runs the ordinary operator
  on it: no collective on the data path.  A grouped-query group never straddles two ranks, so
  dK/dV keep a single owner.
* ``ring_attention`` - context parallelism for sequences too long for one GPU.  Every rank owns
  ``S / P`` queries and the matching K/V (and key-mask) shard.  In step ``j`` a rank attends its
  queries to the K/V block it currently holds while that block is already on its way to the next
  rank (send/recv through ``torch.distributed``, which NCCL runs on a stream of its own, into a
  second local buffer).  Each step is ONE kernel call that folds its block into a running FP32
  state (unnormalised accumulator, unscaled maximum, sum) with the (maximum, sum) merge of the
  reference's split forward (src/kohakufa_cute/split_forward.py:219-245 of the reference
  project) in the kernel's epilogue; one division and one rounding close the state, and the
  statistics keep the operator's contract, so the backward kernels can be reused block by block.
  They return FP32 contributions: dQ accumulates locally, the dK/dV totals of a block travel
  around the ring in FP32 one step behind the block itself (the transfer of the totals overlaps
  the next step's kernels) and are rounded once by the block's owner.

  Causal attention uses zig-zag shards (``zigzag_shard``): the sequence is cut into ``2 P`` chunks
  and rank ``r`` owns chunks ``r`` and ``2 P - 1 - r``, so every rank has the same number of visible
  (query, key) pairs in every step: the own block is an ordinary causal call, a block from a lower
  rank is seen by all local queries but only with its first chunk, a block from a higher rank is
  seen completely but only by the local second chunk.  All of these are views; nothing is copied.
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
_LOG2E = 1.4426950408889634


class PipelineBlocks:
    """Block-wise kernels of the tensor-memory pipeline family (``kfa_forward_running``,
    ``kfa_finish_running``, ``kfa_backward_partial``): FP32 between blocks, nothing rounded."""

    @staticmethod
    def new_state(q):
        from . import native

        return native.running_state(q)

    @staticmethod
    def forward_block(q, k, v, mask, state, scale, causal):
        from . import native

        native.forward_running(q, k, v, mask, state, scale, causal)

    @staticmethod
    def finish(state, dtype):
        from . import native

        return native.finish_running(state, dtype)

    @staticmethod
    def backward_block(q, k, v, mask, out, maximum, logsum, dout, scale, causal, dq, dk, dv):
        from . import native

        native.backward_partial(q, k, v, mask, maximum, logsum, dout, out, scale, causal, dq, dk, dv,
                                accumulate_dq=True, accumulate_dkv=False)


class RoundedBlocks:
    """The same interface over the ordinary forward / backward entry points, for operands the pipeline
    family does not serve (wide heads, odd head sizes): every block's 16-bit result is widened and folded
    into the FP32 state with elementwise device operations, so each block adds one rounding."""

    @staticmethod
    def new_state(q):
        acc = torch.zeros(q.shape, device=q.device, dtype=torch.float32)
        run_maximum = torch.full(q.shape[:-1], float("-inf"), device=q.device, dtype=torch.float32)
        return acc, run_maximum, torch.zeros_like(run_maximum)

    @staticmethod
    def forward_block(q, k, v, mask, state, scale, causal):
        from . import native

        out, maximum, logsum, _ = native.forward(q, k, v, mask, scale, causal)
        acc, run_maximum, run_sum = state
        c2 = abs(scale) * _LOG2E
        new = torch.maximum(run_maximum, maximum)
        zero = torch.zeros_like(new)
        w_old = torch.where(torch.isinf(run_maximum), zero, torch.exp2((run_maximum - new) * c2))
        w_blk = torch.where(torch.isinf(maximum), zero, torch.exp2((maximum - new) * c2 + logsum))
        acc.mul_(w_old[..., None]).add_(out.float() * w_blk[..., None])
        run_sum.mul_(w_old).add_(w_blk)
        run_maximum.copy_(new)

    @staticmethod
    def finish(state, dtype):
        acc, run_maximum, run_sum = state
        seen = run_sum > 0
        inv = torch.where(seen, 1 / run_sum, torch.zeros_like(run_sum))
        out = (acc * inv[..., None]).to(dtype)
        maximum = torch.where(seen, run_maximum, torch.full_like(run_maximum, float("-inf")))
        return out, maximum, torch.where(seen, torch.log2(run_sum), torch.zeros_like(run_sum))

    @staticmethod
    def backward_block(q, k, v, mask, out, maximum, logsum, dout, scale, causal, dq, dk, dv):
        from . import native

        blocks = None if mask is None else native.pack_mask(q, k, mask)
        gq, gk, gv = native.backward(q, k, v, mask, maximum.contiguous(), logsum.contiguous(), dout, blocks, out,
                                     scale, causal)
        dq.add_(gq.float())
        dk.copy_(gk)
        dv.copy_(gv)


def _pick_kernels(q, k, v, causal):
    from . import native

    return PipelineBlocks if native.selected_family(q, k, v, None, causal, True) == 1 else RoundedBlocks


def zigzag_chunks(world, rank):
    """The two chunk indices (of ``2 * world``) that ``rank`` owns under the causal layout."""
    return rank, 2 * world - 1 - rank


def zigzag_shard(x, world, rank, dim=2):
    """This rank's causal shard of a full-sequence tensor: chunks ``rank`` and ``2 world - 1 - rank``
    concatenated along ``dim`` (whose extent must be a multiple of ``2 world``)."""
    if x.shape[dim] % (2 * world):
        raise ValueError("the sequence length must be a multiple of twice the number of ranks")
    chunks = x.chunk(2 * world, dim)
    lo, hi = zigzag_chunks(world, rank)
    return torch.cat((chunks[lo], chunks[hi]), dim)


def zigzag_unshard(shards, dim=2):
    """Inverse of ``zigzag_shard``: the full-sequence tensor from every rank's shard, in rank order."""
    world = len(shards)
    chunks = [None] * (2 * world)
    for rank, shard in enumerate(shards):
        lo, hi = zigzag_chunks(world, rank)
        chunks[lo], chunks[hi] = shard.chunk(2, dim)
    return torch.cat(chunks, dim)


def _exchange(tensors, group):
    """Sends every tensor to the next rank and receives its replacement from the previous one.
    Returns the receive buffers and the pending requests; nothing is waited for here."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    nxt = dist.get_global_rank(group, (rank + 1) % world) if group is not None else (rank + 1) % world
    prv = dist.get_global_rank(group, (rank - 1) % world) if group is not None else (rank - 1) % world
    received = [torch.empty_like(t) for t in tensors]
    ops = []
    for t, r in zip(tensors, received):
        ops.append(dist.P2POp(dist.isend, t, nxt, group))
        ops.append(dist.P2POp(dist.irecv, r, prv, group))
    return received, dist.batch_isend_irecv(ops)


def _wait(pending):
    for work in pending or ():
        work.wait()


def _step_views(step, source, rank, causal, half):
    """Which part of the local queries meets which part of the resident block in this step:
    ``(query rows, key rows, causal flag)`` as slices of the local sequence axis."""
    everything = slice(None)
    if not causal:
        return everything, everything, False
    if step == 0:
        return everything, everything, True       # own block: ordinary causal attention on the two local chunks
    if source < rank:
        return everything, slice(0, half), False   # earlier block: only its first chunk lies before local queries
    return slice(half, None), everything, False    # later block: only the local second chunk lies behind it


def ring_forward(q, k, v, key_mask, scale, group=None, *, causal=False, kernels=None):
    """Forward of ring attention on this rank's shards.

    ``q``: ``[B, Hq, S/P, D]``; ``k``, ``v``: ``[B, Hkv, S/P, D]``; ``key_mask``: optional bool
    ``[B, 1, 1, S/P]`` shard (True = visible); causal calls expect zig-zag shards.  Returns
    ``(out, maximum, logsum)`` where ``out`` has q's dtype and the statistics cover the whole key
    sequence.  ``kernels`` defaults to the CUDA kernels; tests inject CPU stand-ins.
    """
    kernels = kernels or _pick_kernels(q, k, v, causal)
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    B, Hq, Sq, D = q.shape
    half = Sq // 2
    if causal and (Sq % 2 or k.shape[2] != Sq):
        raise ValueError("causal ring attention needs equal, even query and key shard lengths")
    state = kernels.new_state(q)
    block = [k.contiguous(), v.contiguous()] + ([] if key_mask is None else [key_mask.contiguous()])
    for step in range(world):
        incoming = pending = None
        if step + 1 < world:
            incoming, pending = _exchange(block, group)   # travels while this step computes
        rows, keys, flag = _step_views(step, (rank - step) % world, rank, causal, half)
        qs, ks, vs = q[:, :, rows], block[0][:, :, keys], block[1][:, :, keys]
        mask = None if key_mask is None else block[2][..., keys].expand(B, Hq, qs.shape[2], ks.shape[2])
        kernels.forward_block(qs, ks, vs, mask, tuple(t[:, :, rows] for t in state), scale, flag)
        if pending is not None:
            _wait(pending)
            block = incoming
    return kernels.finish(state, q.dtype)


def ring_backward(q, k, v, key_mask, out, maximum, logsum, dout, scale, group=None, *, causal=False, kernels=None):
    """Backward of ring attention: returns ``(dq, dk, dv)`` for this rank's shards.

    dQ accumulates locally in FP32.  The FP32 dK/dV totals of a block follow the block around the ring
    one step behind it: a rank computes its contribution to the resident block while the totals so far
    are still arriving, adds, and sends them on while the next step computes.  After ``P`` hops the totals
    are home and are rounded once.
    """
    kernels = kernels or _pick_kernels(q, k, v, causal)
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    B, Hq, Sq, D = q.shape
    half = Sq // 2
    dq = torch.zeros(q.shape, device=q.device, dtype=torch.float32)
    kv = [k.contiguous(), v.contiguous()] + ([] if key_mask is None else [key_mask.contiguous()])
    upper = None
    if causal and world > 1:
        upper = (maximum[:, :, half:].contiguous(), logsum[:, :, half:].contiguous())  # statistics are dense tensors
    totals = totals_pending = sent = None
    for step in range(world):
        kv_next = kv_pending = None
        if step + 1 < world:
            kv_next, kv_pending = _exchange(kv, group)
        rows, keys, flag = _step_views(step, (rank - step) % world, rank, causal, half)
        part = [torch.empty(k.shape, device=k.device, dtype=torch.float32) for _ in range(2)]
        ks = kv[0][:, :, keys]
        mask = None if key_mask is None else kv[2][..., keys].expand(B, Hq, q[:, :, rows].shape[2], ks.shape[2])
        stats = (maximum, logsum) if rows == slice(None) else upper
        kernels.backward_block(q[:, :, rows], ks, kv[1][:, :, keys], mask, out[:, :, rows], stats[0], stats[1],
                               dout[:, :, rows], scale, flag, dq[:, :, rows], part[0][:, :, keys], part[1][:, :, keys])
        if step == 0:
            totals = part                       # the own block: every key row was written
        else:
            _wait(totals_pending)               # the totals so far arrived while the kernels ran
            totals[0][:, :, keys] += part[0][:, :, keys]
            totals[1][:, :, keys] += part[1][:, :, keys]
        if world > 1:
            sent = totals                       # keep the buffers alive until the transfer is waited for
            totals, totals_pending = _exchange(totals, group)
        if kv_pending is not None:
            _wait(kv_pending)
            kv = kv_next
    _wait(totals_pending)                       # last hop: the totals of this rank's own block are home
    del sent
    return dq.to(q.dtype), totals[0].to(k.dtype), totals[1].to(v.dtype)


class _RingAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, key_mask, scale, group, causal):
        out, maximum, logsum = ring_forward(q, k, v, key_mask, scale, group, causal=causal)
        ctx.save_for_backward(q, k, v, out, maximum, logsum, *(() if key_mask is None else (key_mask,)))
        ctx.scale, ctx.group, ctx.has_mask, ctx.causal = scale, group, key_mask is not None, causal
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, maximum, logsum, *rest = ctx.saved_tensors
        dq, dk, dv = ring_backward(q, k, v, rest[0] if ctx.has_mask else None, out, maximum, logsum,
                                   dout.contiguous(), ctx.scale, ctx.group, causal=ctx.causal)
        return dq, dk, dv, None, None, None, None


def ring_attention(q, k, v, *, key_mask=None, scale=None, group=None, causal=False):
    """Attention over a sequence sharded across the ranks of ``group`` (autograd-aware).  Non-causal calls take
    contiguous shards; causal calls take the shards ``zigzag_shard`` makes."""
    scale = q.shape[-1] ** -0.5 if scale is None else float(scale)
    return _RingAttention.apply(q, k, v, key_mask, scale, group, bool(causal))
