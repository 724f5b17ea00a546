"""Shared helpers for the GPU parity tests: run the public API, compare with the CPU oracle."""

import math

import torch

from oracle import attention_oracle as ao

TOL = {torch.bfloat16: dict(elem=0.02, norm=0.01), torch.float16: dict(elem=0.003, norm=0.005)}
NAMES = ("out", "dq", "dk", "dv")


def make_inputs(B, Hq, Hkv, Sq, Sk, D, dtype, seed, device="cuda", q_scale=1.0):
    gen = torch.Generator().manual_seed(seed)
    q = (torch.randn(B, Hq, Sq, D, generator=gen) * q_scale).to(dtype)
    k = torch.randn(B, Hkv, Sk, D, generator=gen).to(dtype)
    v = torch.randn(B, Hkv, Sk, D, generator=gen).to(dtype)
    dout = torch.randn(B, Hq, Sq, D, generator=gen).to(dtype)
    return tuple(t.to(device) for t in (q, k, v, dout))


def run_attention(fn, q, k, v, dout, **kwargs):
    """Forward + backward through the public API; returns (out, dq, dk, dv) detached."""
    leaves = [t.detach().clone().requires_grad_(True) for t in (q, k, v)]
    out = fn(*leaves, **kwargs)
    grads = torch.autograd.grad(out, leaves, dout)
    return (out.detach(), *[g.detach() for g in grads])


def check_against_oracle(actual, q, k, v, dout, mask=None, causal=False, scale=None, norm_only=False, label=""):
    """The acceptance gates: per-head norm error against both FP64 mathematics and the rounding
    contract (conditioned on the actual forward output), element-wise closeness against the
    contract, and exact zeros where the contract is exactly zero."""
    dtype = q.dtype
    tol = TOL[dtype]
    cpu = [t.detach().cpu() for t in (q, k, v)]
    g = dout.detach().cpu()
    m = None if mask is None else mask.detach().cpu()
    exact = ao.math_reference(cpu, g, m, causal, scale)
    if k.shape[2] == 1:
        # A visible single key has P = 1 and dS = 0 exactly; two independent FP32 reductions of dP and
        # delta in the contract would invent a few-ulp gradient and reject the kernel's exact zero.
        contract = exact
    else:
        contract = ao.contract_reference(cpu, g, m, causal, scale, output=actual[0].detach().cpu())
    for name, got, want_exact, want in zip(NAMES, actual, exact, contract):
        got = got.detach().cpu()
        assert bool(torch.isfinite(got).all()), f"{label}{name}: non-finite values"
        for reference, tag in ((want_exact, "fp64"), (want, "contract")):
            err = ao.per_head_relative_error(got, reference) if float(reference.abs().max()) > 0 else (
                0.0 if float(got.abs().max()) == 0 else math.inf)
            limit = tol["norm"]
            if tag == "fp64" and float(want_exact.abs().max()) > 0:
                # On tiny heads the contract's own operand rounding can exceed the nominal gate; the
                # requirement is then "no worse than the contract itself" (with 25 % slack).
                own = ao.per_head_relative_error(want.to(dtype).double(), want_exact)
                limit = max(limit, 1.25 * own)
            assert err < limit, f"{label}{name} vs {tag}: per-head relative error {err:.3e} (limit {limit:.3e})"
        if not norm_only:
            torch.testing.assert_close(got.double(), want, atol=tol["elem"], rtol=tol["elem"],
                                       msg=lambda s: f"{label}{name} vs contract: {s}")
    return exact, contract


def strided_like_projection(t):
    """Same values, but laid out [B, S, H, D] in memory (a transposed projection view)."""
    return t.transpose(1, 2).contiguous().transpose(1, 2)
