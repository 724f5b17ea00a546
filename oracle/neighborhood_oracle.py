"""CPU oracle for 2-D / 3-D neighbourhood (shifted-window) attention.  TEST INFRASTRUCTURE ONLY.

Nothing in the product package may import this module; it is executed only by
the test-suite, the smoke check and the CPU-baseline leg of the benchmark.

Parity status: PINNED by ``tests/test_oracle_golden.py`` against vectors made by
importing the reference's own neighbourhood oracles
(``tests/golden/make_golden.py``).

Reference locations restated here (paths inside the reference project):

* window geometry        – ``benchmarks/neighborhood/reference.py:12-43`` (each axis picks the
                           legal window whose anchor ``start + w//2`` is nearest the query) and
                           ``src/kohakufa_cute/neighborhood_kernels.py:193-212``
* inverse geometry       – ``src/kohakufa_cute/neighborhood_geometry.py:20-25``
* default backward       – method ``weighted_dq_reconstructed_dk`` of
                           ``benchmarks/neighborhood/key_precision_reference.py:17-69`` with
                           ``precision_reference.py:15-57``; described in ``docs/precision.md:46-80``
* 3-D two-term forward   – ``benchmarks/neighborhood/reference.py:47-69``
* sampled evaluation     – ``na_contract_sampled`` evaluates the same contract on chosen query rows (out, dQ)
                           and chosen key rows (dK, dV) only, so that grids of benchmark size can be checked;
                           the sampling protocol follows ``docs/neighborhood/reports/3d-multigpu.md:41`` and
                           the column-restricted idea of ``benchmarks/neighborhood/key_precision_reference.py:73-149``

Tokens are flattened row-major with the last spatial axis fastest.
"""

from __future__ import annotations

import itertools
import math

import torch

from .attention_oracle import math_reference

__all__ = [
    "axis_window_start",
    "query_windows",
    "inverse_axis_range",
    "neighborhood_mask",
    "na_math_reference",
    "na_contract_reference",
    "na_two_term_forward",
    "window_indices",
    "na_contract_sampled",
]


def axis_window_start(position, extent, window):
    """First key coordinate seen by a query at ``position`` on one axis."""
    return min(max(position - window // 2, 0), extent - window)


def inverse_axis_range(key, extent, window):
    """Inclusive range ``[lo, hi]`` of query coordinates on one axis whose window contains ``key``."""
    hits = [p for p in range(extent) if axis_window_start(p, extent, window) <= key < axis_window_start(p, extent, window) + window]
    return hits[0], hits[-1]


def query_windows(spatial, window):
    """For every flattened query index, the tuple of flattened key indices it attends to."""
    spatial, window = tuple(spatial), tuple(window)
    if len(spatial) not in (2, 3) or len(window) != len(spatial):
        raise ValueError("spatial shape must be 2-D or 3-D with a matching window")
    if any(w < 1 or w > e for w, e in zip(window, spatial)):
        raise ValueError("every window must fit its axis")
    pitch = [math.prod(spatial[a + 1:]) for a in range(len(spatial))]
    table = []
    for coords in itertools.product(*(range(e) for e in spatial)):
        first = [axis_window_start(p, e, w) for p, e, w in zip(coords, spatial, window)]
        keys = []
        for offs in itertools.product(*(range(w) for w in window)):
            keys.append(sum((f + o) * s for f, o, s in zip(first, offs, pitch)))
        table.append(tuple(keys))
    return tuple(table)


def neighborhood_mask(spatial, window):
    """Dense boolean ``[S, S]`` visibility; only for small grids."""
    table = query_windows(spatial, window)
    seen = torch.zeros(len(table), len(table), dtype=torch.bool)
    for r, keys in enumerate(table):
        seen[r, list(keys)] = True
    return seen


@torch.no_grad()
def na_math_reference(inputs, dout, spatial, window, scale):
    """FP64 mathematics of the windowed attention (forward and all gradients)."""
    return math_reference(inputs, dout, neighborhood_mask(spatial, window), False, scale)


def _window_terms(inputs, dout, spatial, window, scale):
    q, k, v = (t.detach().cpu() for t in inputs)
    g = dout.detach().cpu()
    seen = neighborhood_mask(spatial, window)
    s = torch.matmul(q.float(), k.float().transpose(-1, -2)).double()
    dp = torch.matmul(g.float(), v.float().transpose(-1, -2))
    if scale < 0:
        s = -s
    s = s.masked_fill(~seen, -math.inf)
    w = torch.exp((s - s.amax(-1, keepdim=True)) * abs(scale)).masked_fill(~seen, 0.0)
    return q, k, v, g, seen, w, dp


@torch.no_grad()
def na_contract_reference(inputs, dout, spatial, window, scale, output):
    """Default neighbourhood backward contract (MHA, equal Q/K/V shapes).

    With ``P32`` the FP32 probability, ``P_low = rd(P32)``, ``res = dP - delta`` and
    ``delta = sum_d f32(O) f32(dO)`` from the actual forward output:

    * query pass:   ``dS_q = rd(P32 * res)``;
      ``dQ = (dS_q K - (sum_c dS_q) * (P_low K) / (sum_c P_low)) * scale``
    * key pass:     ``t = sum_c P32 res / sum_c P32``; ``dS_k = rd(P32 * (res - t))``
      (two separate subtractions); ``dK = (dS_k^T Q) * scale``
    * value pass:   ``dV = P_low^T dO``

    Final products accumulate in FP64.  Returns ``(out, dq, dk, dv)`` in float64.
    """
    q, k, v, g, seen, w, dp = _window_terms(inputs, dout, spatial, window, scale)
    dtype = q.dtype
    p = w / w.sum(-1, keepdim=True)
    p32 = p.float()
    p_low = p32.to(dtype).float()
    delta = (output.detach().cpu().float() * g.float()).sum(-1, keepdim=True)
    res = dp - delta
    ds_q = (p32 * res).to(dtype).double()
    key_mean = (p_low.double() @ k.double()) / p_low.double().sum(-1, keepdim=True)
    dq = (ds_q @ k.double() - ds_q.sum(-1, keepdim=True) * key_mean) * scale
    t = (p32 * res).sum(-1, keepdim=True) / p32.sum(-1, keepdim=True)
    ds_k = (p32 * (res - t)).to(dtype).double()
    dk = (ds_k.transpose(-1, -2) @ q.double()) * scale
    dv = p_low.double().transpose(-1, -2) @ g.double()
    return p @ v.double(), dq, dk, dv


@torch.no_grad()
def na_two_term_forward(inputs, spatial, window, scale):
    """3-D forward with the probability split into two input-dtype terms.

    ``hi = rd(w)``, ``lo = rd(w - hi)`` for the unnormalised weight ``w`` against the
    global row maximum; ``O = (hi V + lo V) / sum_c w`` with FP64 products.
    """
    q, k, v = (t.detach().cpu() for t in inputs)
    seen = neighborhood_mask(spatial, window)
    s = torch.matmul(q.float(), k.float().transpose(-1, -2))
    if scale < 0:
        s = -s
    s = s.masked_fill(~seen, -math.inf)
    shifted = ((s - s.amax(-1, keepdim=True)) * abs(scale)).masked_fill(~seen, -math.inf)
    w = shifted.double().exp().float()
    hi = w.to(q.dtype).float()
    lo = (w - hi).to(q.dtype).float()
    num = hi.double() @ v.double() + lo.double() @ v.double()
    return num / w.sum(-1, keepdim=True).double()


def window_indices(spatial, window, rows):
    """``[len(rows), prod(window)]`` flattened key indices attended to by the given flattened queries."""
    spatial, window = tuple(int(x) for x in spatial), tuple(int(x) for x in window)
    rows = torch.as_tensor(rows, dtype=torch.long)
    pitch = [math.prod(spatial[a + 1:]) for a in range(len(spatial))]
    rest = rows.clone()
    keys = torch.zeros(rows.numel(), 1, dtype=torch.long)
    for extent, w, stride in zip(spatial, window, pitch):
        coord = rest // stride
        rest = rest % stride
        first = (coord - w // 2).clamp(0, extent - w)
        axis = (first[:, None] + torch.arange(w)[None, :]) * stride  # [n, w]
        keys = (keys[:, :, None] + axis[:, None, :]).reshape(rows.numel(), -1)
    return keys


def _queries_seeing(spatial, window, key):
    """Flattened indices of all queries whose window contains the flattened key index."""
    pitch = [math.prod(spatial[a + 1:]) for a in range(len(spatial))]
    ranges, rest = [], int(key)
    for extent, w, stride in zip(spatial, window, pitch):
        lo, hi = inverse_axis_range(rest // stride, extent, w)
        ranges.append(range(lo, hi + 1))
        rest %= stride
    return [sum(c * s for c, s in zip(coords, pitch)) for coords in itertools.product(*ranges)]


@torch.no_grad()
def na_contract_sampled(inputs, dout, spatial, window, scale, output, query_rows, key_rows, two_term=False):
    """The contract of ``na_contract_reference`` evaluated sparsely.

    Returns ``(out, dq, dk, dv)`` in float64 where ``out``/``dq`` hold the rows ``query_rows`` and
    ``dk``/``dv`` the rows ``key_rows`` (each complete: every query that sees a sampled key contributes).
    ``out`` is the plain FP64 product, or the two-term product of the 3-D forward when ``two_term``.
    """
    q, k, v = (t.detach().cpu() for t in inputs)
    g, o_given = dout.detach().cpu(), output.detach().cpu()
    dtype = q.dtype
    spatial, window = tuple(int(x) for x in spatial), tuple(int(x) for x in window)
    query_rows = torch.as_tensor(query_rows, dtype=torch.long)
    key_rows = [int(x) for x in key_rows]
    seeing = {c: _queries_seeing(spatial, window, c) for c in key_rows}
    extra = sorted({r for rows in seeing.values() for r in rows})
    rows = torch.unique(torch.cat([query_rows, torch.tensor(extra, dtype=torch.long)]))
    place = {int(r): n for n, r in enumerate(rows.tolist())}
    idx = window_indices(spatial, window, rows)  # [n, W]
    B, H, _, D = q.shape
    nq, nk = query_rows.numel(), len(key_rows)
    out = torch.zeros(B, H, nq, D, dtype=torch.float64)
    dq = torch.zeros(B, H, nq, D, dtype=torch.float64)
    dk = torch.zeros(B, H, nk, D, dtype=torch.float64)
    dv = torch.zeros(B, H, nk, D, dtype=torch.float64)
    qsel = torch.tensor([place[int(r)] for r in query_rows.tolist()], dtype=torch.long)
    for b in range(B):
        for h in range(H):
            qr, gr = q[b, h, rows], g[b, h, rows]
            kw, vw = k[b, h][idx], v[b, h][idx]  # [n, W, D]
            s = torch.bmm(kw.float(), qr.float()[:, :, None])[:, :, 0].double()
            dp = torch.bmm(vw.float(), gr.float()[:, :, None])[:, :, 0]
            if scale < 0:
                s = -s
            w = torch.exp((s - s.amax(-1, keepdim=True)) * abs(scale))
            p = w / w.sum(-1, keepdim=True)
            p32 = p.float()
            p_low = p32.to(dtype).float()
            delta = (o_given[b, h, rows].float() * gr.float()).sum(-1, keepdim=True)
            res = dp - delta
            ds_q = (p32 * res).to(dtype).double()
            kd, vd = kw.double(), vw.double()
            key_mean = torch.einsum("nw,nwd->nd", p_low.double(), kd) / p_low.double().sum(-1, keepdim=True)
            dq_all = (torch.einsum("nw,nwd->nd", ds_q, kd) - ds_q.sum(-1, keepdim=True) * key_mean) * scale
            if two_term:
                w32 = w.float()
                hi = w32.to(dtype).float()
                lo = (w32 - hi).to(dtype).float()
                out_all = (torch.einsum("nw,nwd->nd", hi.double(), vd) + torch.einsum("nw,nwd->nd", lo.double(), vd)) \
                    / w32.sum(-1, keepdim=True).double()
            else:
                out_all = torch.einsum("nw,nwd->nd", p, vd)
            out[b, h], dq[b, h] = out_all[qsel], dq_all[qsel]
            t = (p32 * res).sum(-1, keepdim=True) / p32.sum(-1, keepdim=True)
            ds_k = (p32 * (res - t)).to(dtype).double()
            for n, c in enumerate(key_rows):
                members = torch.tensor([place[r] for r in seeing[c]], dtype=torch.long)
                slot = (idx[members] == c).double()  # [m, W], one hit per row
                dk[b, h, n] = ((ds_k[members] * slot).sum(-1, keepdim=True) * qr[members].double()).sum(0) * scale
                dv[b, h, n] = ((p_low[members].double() * slot).sum(-1, keepdim=True) * gr[members].double()).sum(0)
    return out, dq, dk, dv
