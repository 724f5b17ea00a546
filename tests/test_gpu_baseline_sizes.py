"""The benchmark configurations at their real sizes against the CPU oracle.

Full score matrices of these sizes do not fit a test run, so the oracle is evaluated on sampled query rows
(all rows of the first and the last 128-token tile plus random rows: out, dQ) and sampled key rows (dK, dV,
each complete over every query that sees the key), the protocol of the reference's own large-grid reports
(docs/neighborhood/reports/3d-multigpu.md:41 of the reference project).  The small-shape tests elsewhere
compare every element; these make sure that nothing changes at the grid sizes, tile counts and launch
geometries of the benchmark (CTAs whose rows span several planes, 256 key tiles, split launches).
"""

import pytest
import torch

from oracle import attention_oracle as ao
from oracle import neighborhood_oracle as no
from tests.helpers import NAMES, TOL, check_against_oracle, make_inputs, run_attention

pytestmark = pytest.mark.gpu


def _sample_rows(length, seed, extra=128):
    gen = torch.Generator().manual_seed(seed)
    picked = torch.cat([torch.arange(min(128, length)), torch.arange(max(0, length - 128), length),
                        torch.randint(0, length, (extra,), generator=gen)])
    return torch.unique(picked)


def _compare_rows(name, got, want, dtype):
    """Per-head norm gate and element-wise gate on the sampled rows."""
    tol = TOL[dtype]
    got = got.detach().cpu().double()
    assert bool(torch.isfinite(got).all()), name
    err = ao.per_head_relative_error(got, want)
    assert err < tol["norm"], f"{name}: per-head relative error {err:.3e} on the sampled rows"
    torch.testing.assert_close(got, want, atol=tol["elem"], rtol=tol["elem"], msg=lambda s: f"{name}: {s}")


def test_neighborhood_3d_benchmark_grid_against_sampled_oracle():
    """Config 5: grid 16 x 32 x 32, window (3, 7, 7), FP16 - a 128-token CTA spans four image rows."""
    import kohakufa_cute
    from kohakufa_cute import native

    spatial, window, dtype = (16, 32, 32), (3, 7, 7), torch.float16
    tokens = 16 * 32 * 32
    gen = torch.Generator().manual_seed(5)
    q, k, v, dout = (torch.randn(1, 2, tokens, 64, generator=gen).to(dtype).cuda() for _ in range(4))
    leaves = [t.clone().requires_grad_(True) for t in (q, k, v)]
    native.profile_read(reset=True)
    native.profile_enable(True)
    try:
        out = kohakufa_cute.neighborhood_attention(*leaves, spatial_shape=spatial, window_size=window, scale=0.125)
        grads = torch.autograd.grad(out, leaves, dout)
        torch.cuda.synchronize()
    finally:
        native.profile_enable(False)
    assert {"na_pipeline_forward", "na_pipeline_backward_q", "na_pipeline_backward_kv"} <= set(native.profile_read())
    assert native.device_status(reset=True) == 0
    query_rows = _sample_rows(tokens, 51)
    gen = torch.Generator().manual_seed(52)
    # keys at the corners and faces of the grid (shifted windows) and in the interior
    key_rows = sorted({0, 31, 1023, 1024, tokens - 1, tokens - 1024, 5 * 1024 + 17 * 32 + 3,
                       *torch.randint(0, tokens, (40,), generator=gen).tolist()})
    cpu = tuple(t.cpu() for t in (q, k, v))
    want = no.na_contract_sampled(cpu, dout.cpu(), spatial, window, 0.125, out.detach().cpu(), query_rows, key_rows,
                                  two_term=True)
    _compare_rows("out", out[:, :, query_rows], want[0], dtype)
    _compare_rows("dq", grads[0][:, :, query_rows], want[1], dtype)
    _compare_rows("dk", grads[1][:, :, key_rows], want[2], dtype)
    _compare_rows("dv", grads[2][:, :, key_rows], want[3], dtype)


def test_key_padding_at_32768_tokens_against_sampled_oracle():
    """Config 4 (per head): S = 32768, D = 128, BF16, the last 10 % of the keys hidden: 256 key tiles, of
    which the last 25 are skipped and one is mixed."""
    import kohakufa_cute
    from kohakufa_cute import native

    S, dtype = 32768, torch.bfloat16
    q, k, v, dout = make_inputs(1, 2, 2, S, S, 128, dtype, seed=44)
    keep = S - int(S * 0.1 + 0.5)
    mask = (torch.arange(S, device="cuda") < keep)[None, None, None, :]
    assert native.selected_family(q, k, v, mask.expand(1, 2, S, S), False, backward=True) == 1
    out, dq, dk, dv = run_attention(kohakufa_cute.attention, q, k, v, dout, mask=mask)
    assert native.device_status(reset=True) == 0
    assert float(dk[:, :, keep:].abs().max()) == 0 and float(dv[:, :, keep:].abs().max()) == 0
    rows = _sample_rows(S, 45)
    cpu = tuple(t.cpu() for t in (q, k, v))
    want = ao.contract_reference(cpu, dout.cpu(), mask.cpu(), False, None, output=out.cpu(), query_rows=rows)
    _compare_rows("out", out[:, :, rows], want[0], dtype)
    _compare_rows("dq", dq[:, :, rows], want[1], dtype)
    gen = torch.Generator().manual_seed(46)
    cols = sorted({0, 127, 128, keep - 1, keep - 64, *torch.randint(0, keep, (26,), generator=gen).tolist()})
    want_dk, want_dv = ao.contract_columns(cpu, dout.cpu(), mask.cpu(), False, None, output=out.cpu(), key_rows=cols)
    _compare_rows("dk", dk[:, :, cols], want_dk, dtype)
    _compare_rows("dv", dv[:, :, cols], want_dv, dtype)


def test_wide_head_benchmark_shape_against_full_oracle():
    """Config 2 exactly: B = 1, H = 16, S = 1024, D = 512, BF16, causal (the split score launch and the merged
    gradient launch at their real grids)."""
    import kohakufa_cute
    from kohakufa_cute import native

    q, k, v, dout = make_inputs(1, 16, 16, 1024, 1024, 512, torch.bfloat16, seed=21)
    assert native.selected_family(q, k, v, None, True, backward=True) == 2
    actual = run_attention(kohakufa_cute.attention, q, k, v, dout, causal=True)
    assert native.device_status(reset=True) == 0
    check_against_oracle(actual, q, k, v, dout, causal=True, label="wide_head ")


def test_llm_gqa_benchmark_shape_with_offsets_against_sampled_oracle():
    """Config 3 at batch 1: grouped-query causal, q scaled by 8, keys with a per-head offset and centring,
    small output gradients - the regime the folded statistics of the key/value-gradient kernel must hold in."""
    import kohakufa_cute
    from kohakufa_cute import native

    S, dtype = 4096, torch.bfloat16
    gen = torch.Generator().manual_seed(3)
    q = (torch.randn(1, 8, S, 128, generator=gen) * 8).to(dtype).cuda()
    k = (torch.randn(1, 2, S, 128, generator=gen) + 2 * torch.randn(1, 2, 1, 128, generator=gen)).to(dtype).cuda()
    v = torch.randn(1, 2, S, 128, generator=gen).to(dtype).cuda()
    dout = (torch.randn(1, 8, S, 128, generator=gen) * 1e-3 ** 0.5).to(dtype).cuda()
    kc = native.center_keys(k)
    out, dq, dk, dv = run_attention(kohakufa_cute.attention, q, kc, v, dout, causal=True)
    assert native.device_status(reset=True) == 0
    rows = _sample_rows(S, 31)
    cpu = tuple(t.cpu() for t in (q, kc, v))
    want = ao.contract_reference(cpu, dout.cpu(), None, True, None, output=out.cpu(), query_rows=rows)
    _compare_rows("out", out[:, :, rows], want[0], dtype)
    _compare_rows("dq", dq[:, :, rows], want[1], dtype)
    gen = torch.Generator().manual_seed(32)
    cols = sorted({0, 1, 127, 128, S - 1, *torch.randint(0, S, (59,), generator=gen).tolist()})
    want_dk, want_dv = ao.contract_columns(cpu, dout.cpu(), None, True, None, output=out.cpu(), key_rows=cols)
    _compare_rows("dk", dk[:, :, cols], want_dk, dtype)
    _compare_rows("dv", dv[:, :, cols], want_dv, dtype)
