"""Autograd wiring for the attention operator, eager and compiler-safe.

Two routes reach the same C-ABI calls:

* eager calls use ``torch.autograd.Function`` subclasses (least host overhead);
* under ``torch.compile`` the public API dispatches to ``torch.library`` custom operators with
  fake (shape-only) implementations so that ``fullgraph=True`` tracing and AOT autograd work.

Operator names and schemas match the reference (``kohakufa_cute::forward_v2`` and
``kohakufa_cute::backward_v2``, src/kohakufa_cute/_ops.py:16,53 of the reference project);
the statistics and the tile table are non-differentiable outputs.
"""

import torch

from . import native


def forward_impl(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mask: torch.Tensor | None, scale: float, causal: bool
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    return native.forward(q, k, v, mask, scale, causal)


forward = torch.library.custom_op("kohakufa_cute::forward_v2", mutates_args=())(forward_impl)


@forward.register_fake
def _forward_fake(q, k, v, mask, scale, causal):
    stats = torch.empty(q.shape[:-1], device=q.device, dtype=torch.float32)
    if mask is None:
        shape = (1, 1, 1, 1)
    else:
        shape = (
            1 if mask.stride(0) == 0 else q.shape[0],
            1 if mask.stride(1) == 0 else q.shape[1],
            1 if mask.stride(2) == 0 else (q.shape[2] + 63) // 64,
            1 if mask.stride(3) == 0 else (k.shape[2] + 63) // 64,
        )
    blocks = torch.empty(shape, device=q.device, dtype=torch.int32)
    return torch.empty_like(q), stats, torch.empty_like(stats), blocks


def backward_impl(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    mask: torch.Tensor | None,
    maximum: torch.Tensor,
    logsum: torch.Tensor,
    dout: torch.Tensor,
    blocks: torch.Tensor,
    out: torch.Tensor | None,
    scale: float,
    causal: bool,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    if out is None:
        raise RuntimeError("the saved forward output is required: delta is formed from the stored rounded O")
    return native.backward(q, k, v, mask, maximum, logsum, dout, blocks, out, scale, causal)


backward = torch.library.custom_op("kohakufa_cute::backward_v2", mutates_args=())(backward_impl)


@backward.register_fake
def _backward_fake(q, k, v, mask, maximum, logsum, dout, blocks, out, scale, causal):
    return torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)


def _setup_context(ctx, inputs, output):
    q, k, v, mask, ctx.scale, ctx.causal = inputs
    out, maximum, logsum, blocks = output
    ctx.has_mask = mask is not None
    ctx.save_for_backward(q, k, v, maximum, logsum, blocks, out, *(() if mask is None else (mask,)))
    ctx.mark_non_differentiable(maximum, logsum, blocks)


def _autograd_backward(ctx, dout, dmaximum, dlogsum, dblocks):
    q, k, v, maximum, logsum, blocks, out, *rest = ctx.saved_tensors
    dq, dk, dv = backward(q, k, v, rest[0] if ctx.has_mask else None, maximum, logsum, dout, blocks, out, ctx.scale,
                          ctx.causal)
    return dq, dk, dv, None, None, None


forward.register_autograd(_autograd_backward, setup_context=_setup_context)


def center_keys_impl(k: torch.Tensor) -> torch.Tensor:
    return native.center_keys(k)


center_keys_op = torch.library.custom_op("kohakufa_cute::center_keys", mutates_args=())(center_keys_impl)


@center_keys_op.register_fake
def _center_fake(k):
    return torch.empty_like(k)


def _center_backward(ctx, grad):
    # d/dk of round(f32(k) - mean_S f32(k)) applied to the stored gradient: the same projection
    return center_keys_op(grad)


center_keys_op.register_autograd(_center_backward, setup_context=lambda ctx, inputs, output: None)


def _eager_forward(q, k, v, mask, scale, causal, statistics):
    """Forward through the C ABI: the decoding kernel for a few query rows against a long cache, split over the
    keys when a short query sequence would otherwise leave most of the GPU idle, one launch otherwise."""
    if native.decode_served(q, k, v, mask, causal):
        return native.forward_decode(q, k, v, scale, statistics)
    splits = native.split_plan(q, k, causal)
    if splits:
        return native.forward_split(q, k, v, mask, scale, splits, statistics)
    return native.forward(q, k, v, mask, scale, causal, statistics)


class _EagerAttention(torch.autograd.Function):
    """Eager route: same saved-tensor set as the custom operators, without dispatcher overhead."""

    @staticmethod
    def forward(ctx, q, k, v, mask, scale, causal):
        out, maximum, logsum, blocks = _eager_forward(q, k, v, mask, scale, causal, True)
        ctx.scale, ctx.causal, ctx.has_mask = scale, causal, mask is not None
        ctx.save_for_backward(q, k, v, maximum, logsum, blocks, out, *(() if mask is None else (mask,)))
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, maximum, logsum, blocks, out, *rest = ctx.saved_tensors
        dq, dk, dv = native.backward(q, k, v, rest[0] if ctx.has_mask else None, maximum, logsum, dout, blocks, out,
                                     ctx.scale, ctx.causal)
        return dq, dk, dv, None, None, None


class _EagerCenterKeys(torch.autograd.Function):
    @staticmethod
    def forward(ctx, k):
        return native.center_keys(k)

    @staticmethod
    def backward(ctx, grad):
        return native.center_keys(grad)


def center_keys(k):
    if torch.compiler.is_compiling():
        return center_keys_op(k)
    return _EagerCenterKeys.apply(k)


def attention(q, k, v, *, mask=None, causal=False, scale=None):
    """Expands the mask, resolves the default scale and runs forward with autograd attached."""
    if mask is not None:
        mask = mask.expand(q.shape[0], q.shape[1], q.shape[2], k.shape[2])
    scale = q.shape[-1] ** -0.5 if scale is None else float(scale)
    if torch.compiler.is_compiling():
        return forward(q, k, v, mask, scale, bool(causal))[0]
    if not (torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad)):
        # nobody will differentiate this call: no row statistics, nothing saved
        return _eager_forward(q, k, v, mask, scale, bool(causal), False)[0]
    return _EagerAttention.apply(q, k, v, mask, scale, bool(causal))
