"""CPU oracle for the attention forward+backward path.  TEST INFRASTRUCTURE ONLY.

This module restates, in plain PyTorch on the CPU, the arithmetic that the
reference project specifies for its attention operator.  It exists so that the
CUDA kernels can be checked; nothing in the product package may import it.
Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark
are allowed to execute it.

Parity status: PINNED.  ``tests/test_oracle_golden.py`` compares every function
here against vectors produced by importing the reference's own pure-PyTorch
oracles (``tests/golden/make_golden.py`` is the generating script).

What each function follows in the reference project (paths inside that
project):

* ``math_reference``       – FP64 mathematics, ``benchmarks/reference.py:9-30``
* ``contract_reference``   – single-rounded P / dS contract with the output
                             the kernel actually produced feeding delta,
                             ``benchmarks/reference.py:95-138`` and
                             ``docs/precision.md:13-23``
* ``contract_columns``     – the same contract for chosen key rows only (dK, dV of long
                             sequences), streamed over query chunks; the column-restricted
                             evaluation idea of ``benchmarks/neighborhood/key_precision_reference.py:73-149``
* ``forward_statistics``   – the two saved row statistics (unscaled signed
                             row maximum, base-2 log of the normaliser),
                             ``src/kohakufa_cute/kernels.py:1286-1333,1729-1742``
* ``center_keys`` / ``center_keys_backward`` – ``src/kohakufa_cute/api.py:100-103``
* ``relative_error``       – the norm metric, ``benchmarks/reference.py:33-56``

Conventions: q is ``[B, Hq, Sq, D]``; k and v are ``[B, Hkv, Sk, D]`` with
``Hq % Hkv == 0`` (query head ``h`` reads key/value head ``h // (Hq // Hkv)``);
``mask`` is a boolean tensor broadcastable to ``[B, Hq, Sq, Sk]`` where True
means visible; ``causal`` keeps key ``c`` for query ``r`` iff ``c <= r`` (token
positions, aligned at the top-left corner also when ``Sq != Sk``).
"""

from __future__ import annotations

import math

import torch

__all__ = [
    "visible_pairs",
    "math_reference",
    "contract_reference",
    "contract_columns",
    "forward_statistics",
    "center_keys",
    "center_keys_backward",
    "relative_error",
    "per_head_relative_error",
]


def _default_scale(q, scale):
    return q.shape[-1] ** -0.5 if scale is None else float(scale)


def visible_pairs(batch, heads, sq, sk, mask=None, causal=False):
    """Boolean ``[batch, heads, sq, sk]`` visibility (a broadcast view where possible)."""
    seen = torch.ones(1, 1, sq, sk, dtype=torch.bool)
    if causal:
        rows = torch.arange(sq).view(sq, 1)
        cols = torch.arange(sk).view(1, sk)
        seen = seen & (cols <= rows)
    if mask is not None:
        m = mask.cpu()
        while m.dim() < 4:
            m = m.unsqueeze(0)
        seen = seen & m
    return seen.expand(batch, heads, sq, sk)


def _ieee_fp32_matmul(a, b):
    """FP32 product with IEEE accumulation (no TF32), as the contract prescribes."""
    return torch.matmul(a.float(), b.float())


def _heads(q, k):
    group = q.shape[1] // k.shape[1]
    if group * k.shape[1] != q.shape[1]:
        raise ValueError("query heads must be a multiple of key/value heads")
    return group


@torch.no_grad()
def math_reference(inputs, dout, mask=None, causal=False, scale=None):
    """Exact-arithmetic (FP64) attention forward and backward on the given inputs.

    The score gradient is formed from dP shifted by its value at the most
    probable key, ``c = dP - dP[argmax]``, ``dS = P (c - sum(P c))``; this is the
    same derivative as ``P (dP - sum(P dP))`` but keeps the tiny entries of a
    saturated softmax (reference: benchmarks/reference.py:22-24).
    Returns ``(out, dq, dk, dv)`` in float64.
    """
    q, k, v = (t.detach().cpu().double() for t in inputs)
    g = dout.detach().cpu().double()
    scale = _default_scale(q, scale)
    group = _heads(q, k)
    B, Hq, Sq, D = q.shape
    Sk = k.shape[2]
    seen = visible_pairs(B, Hq, Sq, Sk, mask, causal)
    out = torch.zeros_like(q)
    dq = torch.zeros_like(q)
    dk = torch.zeros_like(k)
    dv = torch.zeros_like(v)
    for b in range(B):
        for h in range(Hq):
            kv = h // group
            logits = (q[b, h] @ k[b, kv].T) * scale
            logits = logits.masked_fill(~seen[b, h], -math.inf)
            alive = seen[b, h].any(-1, keepdim=True)
            p = torch.softmax(logits.masked_fill(~alive, 0.0), -1).masked_fill(~alive, 0.0)
            p = p.masked_fill(~seen[b, h], 0.0)
            out[b, h] = p @ v[b, kv]
            dp = g[b, h] @ v[b, kv].T
            anchor = dp.gather(-1, logits.argmax(-1, keepdim=True))
            c = dp - anchor
            ds = p * (c - (p * c).sum(-1, keepdim=True))
            dq[b, h] = (ds @ k[b, kv]) * scale
            dk[b, kv] += (ds.T @ q[b, h]) * scale
            dv[b, kv] += p.T @ g[b, h]
    return out, dq, dk, dv


@torch.no_grad()
def forward_statistics(inputs, mask=None, causal=False, scale=None):
    """The two FP32 row statistics the forward pass saves for backward.

    ``maximum[b,h,r]`` is the largest visible *unscaled* score times the sign of
    ``scale``; ``logsum[b,h,r] = log2(sum_c exp((s' - maximum) * |scale|))``.  A row
    with no visible key reports ``maximum = -inf`` and ``logsum = 0``.
    Consequently ``maximum*|scale| + logsum*ln2 == logsumexp(scale * QK^T)``
    (reference: tests/test_adversarial.py:91-108).
    """
    q, k, _ = (t.detach().cpu() for t in inputs)
    scale = _default_scale(q, scale)
    sign = 1.0 if scale >= 0 else -1.0
    group = _heads(q, k)
    B, Hq, Sq, _ = q.shape
    Sk = k.shape[2]
    seen = visible_pairs(B, Hq, Sq, Sk, mask, causal)
    maximum = torch.empty(B, Hq, Sq, dtype=torch.float64)
    logsum = torch.empty(B, Hq, Sq, dtype=torch.float64)
    for b in range(B):
        for h in range(Hq):
            s = _ieee_fp32_matmul(q[b, h], k[b, h // group].T).double() * sign
            s = s.masked_fill(~seen[b, h], -math.inf)
            alive = seen[b, h].any(-1)
            m = s.amax(-1)
            w = torch.exp((s - m.masked_fill(~alive, 0.0)[:, None]) * abs(scale)).masked_fill(~seen[b, h], 0.0)
            total = w.sum(-1)
            maximum[b, h] = m
            logsum[b, h] = torch.where(alive, torch.log2(total.masked_fill(~alive, 1.0)), torch.zeros_like(total))
    return maximum, logsum


@torch.no_grad()
def contract_reference(inputs, dout, mask=None, causal=False, scale=None, *, output=None, query_rows=None):
    """Forward and backward under the operator's rounding contract.

    Rounding points (``rd`` = one round-to-nearest conversion to the input dtype):
    scores and dP are IEEE FP32 products of the stored operands; the row maximum
    is taken on the unscaled, sign-adjusted scores and subtracted *before* the
    multiplication by ``|scale|``; ``P_low = rd(P)``; ``delta = sum_d f32(O) f32(dO)``
    with O the rounded tensor the forward pass returned (``output``; when absent
    the contract's own rounded O is used); ``dS_low = rd(P_low (dP - delta))``;
    the signed scale multiplies dQ and dK after accumulation; dK and dV of one
    key/value head are summed over its group of query heads.  Final products are
    accumulated in FP64 so that only operand rounding is modelled.

    ``query_rows`` (1-D LongTensor) restricts the evaluation to those query rows:
    ``out``/``dq`` then have ``len(query_rows)`` rows and ``dk``/``dv`` hold only the
    contribution of those rows (useful for long sequences).
    Returns ``(out, dq, dk, dv)`` in float64.
    """
    q, k, v = (t.detach().cpu() for t in inputs)
    g = dout.detach().cpu()
    dtype = q.dtype
    scale = _default_scale(q, scale)
    sign = 1.0 if scale >= 0 else -1.0
    group = _heads(q, k)
    B, Hq, Sq, D = q.shape
    Sk = k.shape[2]
    seen_all = visible_pairs(B, Hq, Sq, Sk, mask, causal)
    rows = torch.arange(Sq) if query_rows is None else torch.as_tensor(query_rows, dtype=torch.long)
    given = None if output is None else output.detach().cpu()
    n = rows.numel()
    out = torch.zeros(B, Hq, n, D, dtype=torch.float64)
    dq = torch.zeros(B, Hq, n, D, dtype=torch.float64)
    dk = torch.zeros(k.shape, dtype=torch.float64)
    dv = torch.zeros(v.shape, dtype=torch.float64)
    for b in range(B):
        for h in range(Hq):
            kv = h // group
            qh, gh = q[b, h, rows], g[b, h, rows]
            seen = seen_all[b, h, rows]
            alive = seen.any(-1, keepdim=True)
            s = _ieee_fp32_matmul(qh, k[b, kv].T).double() * sign
            dp = _ieee_fp32_matmul(gh, v[b, kv].T)
            s = s.masked_fill(~seen, -math.inf)
            m = s.amax(-1, keepdim=True).masked_fill(~alive, 0.0)
            w = torch.exp((s - m) * abs(scale)).masked_fill(~seen, 0.0)
            p = w / w.sum(-1, keepdim=True).masked_fill(~alive, 1.0)
            o = p @ v[b, kv].double()
            out[b, h] = o
            o_low = (o.to(dtype) if given is None else given[b, h, rows]).float()
            delta = (o_low * gh.float()).sum(-1, keepdim=True)
            p_low = p.float().to(dtype).float()
            ds_low = (p_low * (dp - delta)).to(dtype).double()
            dq[b, h] = (ds_low @ k[b, kv].double()) * scale
            dk[b, kv] += (ds_low.T @ qh.double()) * scale
            dv[b, kv] += p_low.double().T @ gh.double()
    return out, dq, dk, dv


@torch.no_grad()
def contract_columns(inputs, dout, mask=None, causal=False, scale=None, *, output, key_rows, chunk=2048):
    """``dk`` and ``dv`` of the rounding contract for the key rows ``key_rows`` only (float64,
    ``[B, Hkv, len(key_rows), D]``), complete over all queries.

    Queries are processed in chunks: each chunk forms its full score rows (for the row maximum and the
    normaliser, exactly as ``contract_reference``) but keeps P and dS only at the chosen columns, so the
    memory stays ``chunk x Sk`` whatever the sequence length.  ``output`` is the rounded forward output.
    """
    q, k, v = (t.detach().cpu() for t in inputs)
    g, given = dout.detach().cpu(), output.detach().cpu()
    dtype = q.dtype
    scale = _default_scale(q, scale)
    sign = 1.0 if scale >= 0 else -1.0
    group = _heads(q, k)
    B, Hq, Sq, D = q.shape
    Sk = k.shape[2]
    cols = torch.as_tensor(key_rows, dtype=torch.long)
    dk = torch.zeros(B, k.shape[1], cols.numel(), D, dtype=torch.float64)
    dv = torch.zeros_like(dk)
    m4 = None
    if mask is not None:
        m4 = mask.cpu()
        while m4.dim() < 4:
            m4 = m4.unsqueeze(0)
        m4 = m4.expand(B, Hq, Sq, Sk)
    key_index = torch.arange(Sk).view(1, Sk)
    for b in range(B):
        for h in range(Hq):
            kv = h // group
            kf, vc = k[b, kv].float(), v[b, kv, cols].float()
            for r0 in range(0, Sq, chunk):
                r1 = min(Sq, r0 + chunk)
                qh, gh = q[b, h, r0:r1], g[b, h, r0:r1]
                seen = torch.ones(r1 - r0, Sk, dtype=torch.bool)
                if causal:
                    seen &= key_index <= torch.arange(r0, r1).view(-1, 1)
                if m4 is not None:
                    seen &= m4[b, h, r0:r1]
                alive = seen.any(-1, keepdim=True)
                s = (qh.float() @ kf.T).double() * sign
                s = s.masked_fill(~seen, -math.inf)
                m = s.amax(-1, keepdim=True).masked_fill(~alive, 0.0)
                total = torch.exp((s - m) * abs(scale)).masked_fill(~seen, 0.0).sum(-1, keepdim=True).masked_fill(~alive, 1.0)
                p = (torch.exp((s[:, cols] - m) * abs(scale)).masked_fill(~seen[:, cols], 0.0)) / total
                dp = gh.float() @ vc.T
                delta = (given[b, h, r0:r1].float() * gh.float()).sum(-1, keepdim=True)
                p_low = p.float().to(dtype).float()
                ds_low = (p_low * (dp - delta)).to(dtype).double()
                dk[b, kv] += (ds_low.T @ qh.double()) * scale
                dv[b, kv] += p_low.double().T @ gh.double()
    return dk, dv


def center_keys(k):
    """``rd(f32(k) - mean over the sequence axis of f32(k))`` per batch, head and channel."""
    kf = k.float()
    return (kf - kf.mean(dim=-2, keepdim=True)).to(k.dtype)


def center_keys_backward(dk_centered):
    """Gradient w.r.t. the uncentered keys: ``rd(g - mean_S g)`` with ``g = f32(dk_centered)``."""
    gf = dk_centered.float()
    return (gf - gf.mean(dim=-2, keepdim=True)).to(dk_centered.dtype)


def _stable_norm(t):
    peak = float(t.abs().max()) if t.numel() else 0.0
    return peak * float((t / peak).norm()) if peak else 0.0


def relative_error(got, want):
    """``||got - want|| / ||want||`` with norms formed after dividing by the peak magnitude.

    Returns ``None`` when ``want`` is identically zero (then compare exactly instead).
    """
    a = got.detach().cpu().double().flatten()
    b = want.detach().cpu().double().flatten()
    if not bool(torch.isfinite(a).all()):
        return math.inf
    den = _stable_norm(b)
    if den == 0:
        return None
    return _stable_norm(a - b) / den


def per_head_relative_error(got, want):
    """Largest ``relative_error`` over the (batch, head) slices; exact-zero heads must match exactly."""
    worst = 0.0
    for b in range(want.shape[0]):
        for h in range(want.shape[1]):
            e = relative_error(got[b, h], want[b, h])
            if e is None:
                e = 0.0 if float(got[b, h].detach().double().abs().max()) == 0.0 else math.inf
            worst = max(worst, e)
    return worst
