"""GPU parity tests: the CUDA path (through the public API and the C ABI) against the CPU oracle."""

import math

import pytest
import torch

from oracle import attention_oracle as ao
from tests.golden_io import ATTENTION_CASES, attention_case, load
from tests.helpers import (NAMES, TOL, check_against_oracle, make_inputs, run_attention, strided_like_projection)

pytestmark = pytest.mark.gpu


def api():
    import kohakufa_cute

    return kohakufa_cute


def native():
    from kohakufa_cute import native as n

    return n


@pytest.fixture(autouse=True)
def _device_status_clean():
    yield
    torch.cuda.synchronize()
    assert native().device_status(reset=True) == 0, "a kernel reported a bounded-wait timeout"


# ------------------------------------------------------------------ golden vectors
@pytest.mark.parametrize("index", ATTENTION_CASES)
def test_golden_cases(index):
    c = attention_case(index)
    q, k, v, dout = (c[n].cuda() for n in ("q", "k", "v", "dout"))
    mask = None if c["mask"] is None else c["mask"].cuda()
    actual = run_attention(api().attention, q, k, v, dout, mask=mask, causal=c["causal"], scale=c["scale"])
    check_against_oracle(actual, q, k, v, dout, mask, c["causal"], c["scale"], label=f"case{index} ")
    # the committed reference answers themselves (FP64 mathematics from the reference project)
    tol = TOL[q.dtype]["norm"]
    for name, got in zip(NAMES, actual):
        want = c[f"exact_{name}"]
        if float(want.abs().max()) > 0:
            own = ao.per_head_relative_error(c[f"rounded_{name}"].to(q.dtype).double(), want)
            assert ao.per_head_relative_error(got.cpu(), want) < max(tol, 1.25 * own), name


# ---------------------------------------------------------------- shape sweeps
PIPELINE_SHAPES = [
    # B, Hq, Hkv, Sq, Sk, D, causal
    (1, 1, 1, 128, 128, 128, False),
    (1, 2, 1, 256, 256, 128, True),
    (2, 4, 2, 129, 257, 128, False),
    (1, 2, 2, 300, 300, 128, True),
    (1, 2, 1, 1, 300, 128, False),
    (1, 4, 1, 17, 127, 64, True),
    (1, 2, 2, 513, 140, 64, True),
    (1, 2, 2, 140, 513, 64, True),
    (1, 8, 2, 640, 640, 64, False),
    (1, 2, 1, 1024, 1024, 128, True),
]


@pytest.mark.parametrize("dtype", (torch.bfloat16, torch.float16))
@pytest.mark.parametrize("shape", PIPELINE_SHAPES)
def test_pipeline_shapes(shape, dtype):
    B, Hq, Hkv, Sq, Sk, D, causal = shape
    q, k, v, dout = make_inputs(B, Hq, Hkv, Sq, Sk, D, dtype, seed=hash(shape) % 1000)
    assert native().selected_family(q, k, v, None, causal) == 1
    actual = run_attention(api().attention, q, k, v, dout, causal=causal)
    check_against_oracle(actual, q, k, v, dout, None, causal, None)


WIDE_SHAPES = [
    # B, Hq, Hkv, Sq, Sk, D, causal
    (1, 1, 1, 128, 128, 256, False),
    (1, 2, 1, 256, 256, 512, True),
    (1, 2, 2, 65, 200, 256, False),
    (1, 2, 1, 96, 96, 512, True),
    (2, 4, 2, 129, 257, 384, False),
    (1, 2, 2, 300, 300, 512, True),
    (1, 2, 1, 1, 300, 256, False),
    (1, 2, 2, 513, 140, 384, True),
    (1, 2, 2, 140, 513, 512, True),
    (1, 4, 1, 640, 640, 512, True),
]


@pytest.mark.parametrize("dtype", (torch.bfloat16, torch.float16))
@pytest.mark.parametrize("shape", WIDE_SHAPES)
def test_wide_head_shapes(shape, dtype):
    """Heads of 256/384/512 channels run on the tensor-memory kernels for wide heads (family 2)."""
    B, Hq, Hkv, Sq, Sk, D, causal = shape
    q, k, v, dout = make_inputs(B, Hq, Hkv, Sq, Sk, D, dtype, seed=hash(shape) % 1000)
    assert native().selected_family(q, k, v, None, causal) == 2
    assert native().selected_family(q, k, v, None, causal, backward=True) == 2
    actual = run_attention(api().attention, q, k, v, dout, causal=causal)
    check_against_oracle(actual, q, k, v, dout, None, causal, None)


@pytest.mark.parametrize("scale", (-0.05, 0.2))
@pytest.mark.parametrize("name", ("keys", "key_padding", "all_false", "full2d", "per_head"))
def test_wide_head_masks_and_scales(name, scale):
    B, Hq, Hkv, Sq, Sk, D = 2, 4, 2, 150, 330, 256
    gen = torch.Generator().manual_seed(77)
    mask = _mask_variants(B, Hq, Sq, Sk, gen)[name].cuda()
    q, k, v, dout = make_inputs(B, Hq, Hkv, Sq, Sk, D, torch.bfloat16, seed=78)
    expanded = mask.expand(B, Hq, Sq, Sk)
    assert native().selected_family(q, k, v, expanded, True) == 2   # every mask shape stays on the wide-head kernels
    assert native().selected_family(q, k, v, expanded, True, backward=True) == 2
    actual = run_attention(api().attention, q, k, v, dout, mask=mask, causal=True, scale=scale)
    check_against_oracle(actual, q, k, v, dout, mask, True, scale)
    if name in ("full2d", "per_head"):
        seen = ao.visible_pairs(B, Hq, Sq, Sk, mask.cpu(), True)
        hidden = ~seen.any(-1)
        if bool(hidden.any()):  # all-hidden rows give exactly zero output and zero dQ
            assert float(actual[0].cpu()[hidden].abs().max()) == 0
            assert float(actual[1].cpu()[hidden].abs().max()) == 0
    elif name != "all_false":
        hidden_keys = ~mask.expand(B, 1, 1, Sk)[:, 0, 0].cpu()
        for grad in actual[2:]:
            assert float(grad.cpu()[hidden_keys[:, None, :].expand(B, Hkv, Sk)].abs().max()) == 0


def test_wide_head_backward_in_head_group_passes(monkeypatch):
    """With a small cap on the stored matrices the backward runs batch element by batch element and
    K/V-head group by group over one reused workspace; results do not change."""
    B, Hq, Hkv, S, D = 2, 4, 2, 300, 256
    q, k, v, dout = make_inputs(B, Hq, Hkv, S, S, D, torch.bfloat16, seed=80)
    whole = run_attention(api().attention, q, k, v, dout, causal=True)
    one_group = 2 * S * 384 * 2  # two query heads x S rows x ceil128(S) columns x 2 bytes
    monkeypatch.setenv("KFA_WIDE_MATRIX_BYTES", str(one_group + 256))
    assert native().selected_family(q, k, v, None, True, backward=True) == 2
    split = run_attention(api().attention, q, k, v, dout, causal=True)
    for a, b in zip(whole, split):
        assert torch.equal(a, b)
    check_against_oracle(split, q, k, v, dout, None, True, None)
    # not even one group fits: passes over key ranges of a group, dQ summed over the ranges in FP32
    for limit in (one_group - 256, 1):  # two ranges (256 + 44 keys) and three (128 + 128 + 44)
        monkeypatch.setenv("KFA_WIDE_MATRIX_BYTES", str(limit))
        assert native().selected_family(q, k, v, None, True, backward=True) == 2
        ranged = run_attention(api().attention, q, k, v, dout, causal=True)
        assert torch.equal(ranged[0], whole[0])
        assert torch.equal(ranged[2], whole[2]) and torch.equal(ranged[3], whole[3])  # key owners: same sums
        torch.testing.assert_close(ranged[1], whole[1], atol=2e-3, rtol=2e-2)
        check_against_oracle(ranged, q, k, v, dout, None, True, None)
    # the same with a per-head mask (the tile table and the mask are addressed from the range's first key) and
    # with more keys than queries (the last range is hidden from every query under the causal mask)
    B, Hq, Hkv, Sq, Sk = 1, 2, 1, 200, 450
    gen = torch.Generator().manual_seed(81)
    q, k, v, dout = make_inputs(B, Hq, Hkv, Sq, Sk, D, torch.float16, seed=82)
    for mask, causal in ((torch.rand(B, Hq, Sq, Sk, generator=gen) > 0.4, False), (None, True),
                         ((torch.arange(Sk)[None, :] // 150 == torch.arange(Sq)[:, None] // 100)[None, None], False)):
        mask = None if mask is None else mask.cuda()
        monkeypatch.setenv("KFA_WIDE_MATRIX_BYTES", "1")
        ranged = run_attention(api().attention, q, k, v, dout, mask=mask, causal=causal)
        monkeypatch.delenv("KFA_WIDE_MATRIX_BYTES")
        check_against_oracle(ranged, q, k, v, dout, mask, causal, None)


def test_wide_head_projection_layout():
    """[B, S, H, D] memory behind a [B, H, S, D] view is addressed through the tensor maps, no copy."""
    q, k, v, dout = make_inputs(1, 4, 2, 200, 200, 512, torch.bfloat16, seed=79)
    q, k, v = (strided_like_projection(t) for t in (q, k, v))
    assert native().selected_family(q, k, v, None, True) == 2
    actual = run_attention(api().attention, q, k, v, dout, causal=True)
    check_against_oracle(actual, q, k, v, dout, None, True, None)


GENERAL_SHAPES = [
    (1, 2, 1, 33, 49, 1, False),
    (1, 2, 2, 70, 65, 17, True),
    (1, 4, 2, 64, 96, 80, False),
    (1, 2, 1, 130, 130, 96, True),
    (1, 2, 2, 65, 200, 256, False),
    (1, 2, 1, 96, 96, 512, True),
    (1, 1, 1, 40, 40, 257, False),
]


@pytest.mark.parametrize("dtype", (torch.bfloat16, torch.float16))
@pytest.mark.parametrize("shape", GENERAL_SHAPES)
def test_general_head_dims(shape, dtype):
    B, Hq, Hkv, Sq, Sk, D, causal = shape
    q, k, v, dout = make_inputs(B, Hq, Hkv, Sq, Sk, D, dtype, seed=D)
    actual = run_attention(api().attention, q, k, v, dout, causal=causal)
    check_against_oracle(actual, q, k, v, dout, None, causal, None)


def test_odd_head_dims_and_unaligned_rows_reach_the_tensor_core_kernels():
    """Head sizes that are not multiples of 8 are padded with zero channels by the host layer, operands whose rows
    are not 16-byte addressable are copied densely; either way the tensor-memory kernels do the work (the launch
    statistics show which kernels ran) and the outputs keep the layout of their inputs."""
    def launched(run):
        before = native().launch_stats()
        result = run()
        after = native().launch_stats()
        return result, {name: after[name] - before.get(name, 0) for name in after if after[name] != before.get(name, 0)}

    for D, family in ((17, "pipeline"), (1, "pipeline"), (129, "wide"), (257, "wide")):
        q, k, v, dout = make_inputs(1, 2, 1, 150, 200, D, torch.bfloat16, seed=300 + D)
        actual, ran = launched(lambda: run_attention(api().attention, q, k, v, dout, causal=True))
        assert any(name.startswith(family) for name in ran), (D, ran)
        assert not any(name.startswith("general") for name in ran), (D, ran)
        check_against_oracle(actual, q, k, v, dout, None, True, None)
        assert all(a.shape == b.shape and a.stride() == b.stride() for a, b in zip(actual, (q, q, k, v)))
    # rows that start at odd addresses: a channel offset of one element into a wider buffer
    q, k, v, dout = make_inputs(1, 2, 2, 130, 130, 64, torch.float16, seed=333)
    views = []
    for t in (q, k, v):
        big = torch.full((*t.shape[:-1], t.shape[-1] + 3), float("nan"), device=t.device, dtype=t.dtype)
        big[..., 1:65] = t
        views.append(big[..., 1:65])
    actual, ran = launched(lambda: run_attention(api().attention, *views, dout, causal=False))
    assert any(name.startswith("pipeline") for name in ran) and not any(name.startswith("general") for name in ran), ran
    check_against_oracle(actual, q, k, v, dout, None, False, None)
    # outputs are laid out like empty_like of their inputs (dense here: the views have gaps between rows)
    assert actual[0].stride() == torch.empty_like(views[0]).stride() and actual[2].stride() == torch.empty_like(views[1]).stride()


PADDED_HEAD_SHAPES = [
    # B, Hq, Hkv, Sq, Sk, D, causal: head dims that are multiples of 8 run on the tensor-memory pipeline as 64 or
    # 128 channels (the loads zero-fill the rest, the stores drop it)
    (1, 4, 2, 300, 300, 80, True),
    (2, 2, 2, 129, 257, 96, False),
    (1, 2, 1, 513, 140, 8, True),
    (1, 4, 1, 640, 640, 120, True),
    (1, 2, 2, 70, 330, 40, False),
    (1, 2, 1, 260, 260, 72, True),
]


@pytest.mark.parametrize("dtype", (torch.bfloat16, torch.float16))
@pytest.mark.parametrize("shape", PADDED_HEAD_SHAPES)
def test_head_dims_padded_by_the_tiled_loads(shape, dtype):
    B, Hq, Hkv, Sq, Sk, D, causal = shape
    q, k, v, dout = make_inputs(B, Hq, Hkv, Sq, Sk, D, dtype, seed=D + Sq)
    assert native().selected_family(q, k, v, None, causal) == 1
    assert native().selected_family(q, k, v, None, causal, backward=True) == 1
    # poison behind every row end would show a store or load that runs past the head's channels
    wide = [torch.full((*t.shape[:-1], t.shape[-1] + 8), float("nan"), device=t.device, dtype=t.dtype) for t in (q, k, v)]
    for big, t in zip(wide, (q, k, v)):
        big[..., :D] = t
    views = [big[..., :D] for big in wide]
    assert native().selected_family(*views, None, causal, backward=True) == 1
    actual = run_attention(api().attention, *views, dout, causal=causal)
    check_against_oracle(actual, q, k, v, dout, None, causal, None)
    plain = run_attention(api().attention, q, k, v, dout, causal=causal)
    for a, b in zip(actual, plain):
        assert torch.equal(a, b)
    # a key-padding mask together with the padded channels
    mask = (torch.arange(Sk, device="cuda") < Sk - 37)[None, None, None, :]
    masked = run_attention(api().attention, q, k, v, dout, mask=mask, causal=causal)
    check_against_oracle(masked, q, k, v, dout, mask, causal, None)


@pytest.mark.parametrize("scale", (0.0, -0.125, 0.3))
@pytest.mark.parametrize("D", (64, 96))
def test_signed_and_zero_scale(scale, D):
    q, k, v, dout = make_inputs(1, 2, 1, 150, 170, D, torch.bfloat16, seed=11)
    actual = run_attention(api().attention, q, k, v, dout, scale=scale, causal=True)
    check_against_oracle(actual, q, k, v, dout, None, True, scale)
    if scale == 0.0:
        assert float(actual[1].abs().max()) == 0 and float(actual[2].abs().max()) == 0


# ------------------------------------------------------------------------ masks
def _mask_variants(B, Hq, Sq, Sk, gen):
    full = torch.rand(Sq, Sk, generator=gen) > 0.3
    full[0] = False
    return {
        "keys": torch.rand(Sk, generator=gen) > 0.3,
        "key_padding": (torch.arange(Sk)[None, None, None, :] < torch.tensor([Sk - 37, Sk // 2])[:B, None, None, None]),
        "full2d": full,
        "full4d_one": full[None, None],
        "per_head": torch.rand(B, Hq, Sq, Sk, generator=gen) > 0.5,
        "all_true": torch.ones(1, 1, 1, 1, dtype=torch.bool),
        "all_false": torch.zeros(1, 1, 1, 1, dtype=torch.bool),
    }


@pytest.mark.parametrize("D", (64, 128, 80))
@pytest.mark.parametrize("causal", (False, True))
@pytest.mark.parametrize("name", ("keys", "key_padding", "full2d", "full4d_one", "per_head", "all_true", "all_false"))
def test_boolean_masks(name, causal, D):
    B, Hq, Hkv, Sq, Sk = 2, 4, 2, 150, 330
    gen = torch.Generator().manual_seed(31)
    mask = _mask_variants(B, Hq, Sq, Sk, gen)[name].cuda()
    q, k, v, dout = make_inputs(B, Hq, Hkv, Sq, Sk, D, torch.bfloat16, seed=32)
    if D in (64, 128):
        # every mask shape, full per-head 4-D masks included, runs on the tensor-memory kernels
        expanded = mask.expand(B, Hq, Sq, Sk)
        assert native().selected_family(q, k, v, expanded, causal) == 1
        assert native().selected_family(q, k, v, expanded, causal, backward=True) == 1
    actual = run_attention(api().attention, q, k, v, dout, mask=mask, causal=causal)
    _, contract = check_against_oracle(actual, q, k, v, dout, mask, causal, None)
    # all-hidden rows give exactly zero output and zero dQ
    seen = ao.visible_pairs(B, Hq, Sq, Sk, mask.cpu(), causal)
    hidden = ~seen.any(-1)
    if bool(hidden.any()):
        assert float(actual[0].cpu()[hidden].abs().max()) == 0
        assert float(actual[1].cpu()[hidden].abs().max()) == 0


@pytest.mark.parametrize("D", (128, 256))
def test_block_sparse_full_mask_long_sequence(D):
    """A full [Sq, Sk] mask with hidden, mixed and visible 128x128 blocks (a banded document mask with ragged
    edges) at a length where tile skipping matters; per-head variation through a second, shifted band."""
    B, H, S = 1, 2, 1536
    q, k, v, dout = make_inputs(B, H, H, S, S, D, torch.bfloat16, seed=6)
    idx = torch.arange(S)
    band0 = (idx[:, None] // 200 == idx[None, :] // 200)           # documents of 200 tokens
    band1 = ((idx[:, None] - idx[None, :]).abs() < 333)            # a sliding band
    mask = torch.stack([band0, band1])[None].cuda()                # [1, H, S, S]
    assert native().selected_family(q, k, v, mask, True) == (1 if D == 128 else 2)
    actual = run_attention(api().attention, q, k, v, dout, mask=mask, causal=True)
    check_against_oracle(actual, q, k, v, dout, mask, True, None)


def test_key_padding_long_sequence_skips_hidden_tiles():
    B, H, S, D = 2, 2, 2048, 128
    q, k, v, dout = make_inputs(B, H, H, S, S, D, torch.bfloat16, seed=5)
    mask = (torch.arange(S) < int(S * 0.9))[None, None, None, :].expand(B, 1, 1, S).cuda()
    assert native().selected_family(q, k, v, mask.expand(B, H, S, S), False) == 1
    actual = run_attention(api().attention, q, k, v, dout, mask=mask)
    check_against_oracle(actual, q, k, v, dout, mask, False, None)
    assert float(actual[2][:, :, int(S * 0.9):].abs().max()) == 0
    assert float(actual[3][:, :, int(S * 0.9):].abs().max()) == 0


# ---------------------------------------------------------- layouts and strides
@pytest.mark.parametrize("D", (64, 128, 96))
def test_projection_layout_preserves_strides(D):
    q, k, v, dout = make_inputs(2, 4, 2, 200, 260, D, torch.bfloat16, seed=41)
    qs, ks, vs = (strided_like_projection(t) for t in (q, k, v))
    leaves = [t.detach().requires_grad_(True) for t in (qs, ks, vs)]
    out = api().attention(*leaves, causal=True)
    assert out.stride() == qs.stride()
    grads = torch.autograd.grad(out, leaves, dout)
    for g, t in zip(grads, (qs, ks, vs)):
        assert g.stride() == t.stride()
    check_against_oracle((out.detach(), *grads), q, k, v, dout, None, True, None)


def test_cache_slices_ignore_poison_beyond_the_view():
    B, H, S, D, cap = 1, 2, 150, 128, 256
    q, k, v, dout = make_inputs(B, H, H, S, S, D, torch.bfloat16, seed=43)
    big_k = torch.full((B, H, cap, D), float("nan"), device="cuda", dtype=torch.bfloat16)
    big_v = torch.full((B, H, cap, D), 1234.0, device="cuda", dtype=torch.bfloat16)
    big_k[:, :, :S], big_v[:, :, :S] = k, v
    actual = run_attention(api().attention, q, big_k[:, :, :S], big_v[:, :, :S], dout)
    check_against_oracle(actual, q, k, v, dout)


def test_expanded_and_offset_output_gradients():
    q, k, v, _ = make_inputs(1, 2, 2, 140, 140, 128, torch.bfloat16, seed=44)
    leaves = [t.detach().requires_grad_(True) for t in (q, k, v)]
    out = api().attention(*leaves, causal=True)
    out.sum().backward()  # dO is an expanded (all strides zero) tensor of ones
    actual = (out.detach(), leaves[0].grad, leaves[1].grad, leaves[2].grad)
    check_against_oracle(actual, q, k, v, torch.ones_like(q), None, True, None)


def test_singleton_key_is_exact():
    q, k, v, dout = make_inputs(2, 4, 2, 70, 1, 64, torch.bfloat16, seed=45)
    out, dq, dk, dv = run_attention(api().attention, q, k, v, dout)
    assert torch.equal(out, v.repeat_interleave(2, 1).expand_as(out))
    assert float(dq.abs().max()) == 0 and float(dk.abs().max()) == 0
    want = dout.float().reshape(2, 2, 2, 70, 64).sum((2, 3))[:, :, None]
    torch.testing.assert_close(dv.float(), want, atol=0.02, rtol=0.02)


# ------------------------------------------------------------------- statistics
@pytest.mark.parametrize("D,Sq,Sk,causal", ((128, 300, 300, True), (64, 1, 300, False), (80, 33, 49, False)))
def test_saved_statistics(D, Sq, Sk, causal):
    q, k, v, _ = make_inputs(1, 4, 2, Sq, Sk, D, torch.bfloat16, seed=51, q_scale=4.0)
    scale = -0.2
    out, maximum, logsum, _ = native().forward(q, k, v, None, scale, causal)
    want_max, want_log = ao.forward_statistics((q.cpu(), k.cpu(), v.cpu()), None, causal, scale)
    torch.testing.assert_close(maximum.cpu().double(), want_max, atol=1e-3, rtol=1e-5)
    torch.testing.assert_close(logsum.cpu().double(), want_log, atol=2e-3, rtol=1e-4)
    keys = k.cpu().double().repeat_interleave(2, 1)
    logits = (q.cpu().double() @ keys.transpose(-1, -2)) * scale
    if causal:
        logits = logits.masked_fill(~ao.visible_pairs(1, 4, Sq, Sk, None, True), -math.inf)
    combined = maximum.cpu().double() * abs(scale) + logsum.cpu().double() * math.log(2)
    torch.testing.assert_close(combined, torch.logsumexp(logits, -1), atol=2e-3, rtol=1e-4)


# ------------------------------------------------------------ directed fixtures
def test_saturated_pair_keeps_a_nonzero_query_gradient():
    c = load("saturated_pair")
    q, k, v, dout = (c[n].cuda() for n in ("q", "k", "v", "dout"))
    out, dq, dk, dv = run_attention(api().attention, q, k, v, dout, scale=1.0)
    assert abs(float(dv[0, 0, 0, 0]) - 1.0) < 0.02
    want = float(c["rounded_dk"][0, 0, 1, 0])
    assert want != 0 and abs(float(dk[0, 0, 1, 0]) / want - 1) < 0.03


@pytest.mark.parametrize("dimension", (16, 128))
def test_key_cancellation_fixture(dimension):
    c = load(f"key_cancellation_d{dimension}")
    q, k, v, dout = (c[n].cuda() for n in ("q", "k", "v", "dout"))
    actual = run_attention(api().attention, q, k, v, dout)
    check_against_oracle(actual, q, k, v, dout)


def test_large_logits_stay_finite_and_accurate():
    # clustered unit directions scaled so that scaled logits reach ~1e5: needs the shifted score
    gen = torch.Generator().manual_seed(61)
    H, S, D = 2, 384, 128
    centers = torch.randn(1, H, 16, D, generator=gen)
    centers = centers / centers.norm(dim=-1, keepdim=True)
    pick = torch.randint(16, (1, H, S), generator=gen)
    base = centers.gather(2, pick[..., None].expand(-1, -1, -1, D))
    radius = math.sqrt(1e5 * math.sqrt(D))
    q, k = ((radius * (base + 0.03 * torch.randn(base.shape, generator=gen))).to(torch.bfloat16).cuda() for _ in range(2))
    v, dout = (torch.randn(base.shape, generator=gen).to(torch.bfloat16).cuda() for _ in range(2))
    actual = run_attention(api().attention, q, k, v, dout, causal=True)
    exact = ao.math_reference((q.cpu(), k.cpu(), v.cpu()), dout.cpu(), None, True, None)
    for name, got, want in zip(NAMES, actual, exact):
        assert bool(torch.isfinite(got).all()), name
    got, want = actual[3].cpu().double().flatten(), exact[3].flatten()
    assert float(torch.dot(got, want) / (got.norm() * want.norm())) > 0.9999
    got, want = actual[0].cpu().double().flatten(), exact[0].flatten()
    assert float(torch.dot(got, want) / (got.norm() * want.norm())) > 0.9999


# ------------------------------------------------------------------ SDPA wrappers
def test_sdpa_wrappers_and_errors():
    K = api()
    q, k, v, dout = make_inputs(1, 4, 2, 130, 130, 64, torch.bfloat16, seed=71)
    out = K.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
    torch.testing.assert_close(out, K.attention(q, k, v, causal=True), atol=0, rtol=0)
    torch.testing.assert_close(K.automatic_scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True), out,
                               atol=0, rtol=0)
    mask = torch.ones(130, 130, dtype=torch.bool, device="cuda")
    for kwargs, pattern in (
        (dict(dropout_p=0.1), "dropout"),
        (dict(attn_mask=mask, is_causal=True, enable_gqa=True), "folded"),
        (dict(attn_mask=mask.float(), enable_gqa=True), "boolean"),
        (dict(), "enable_gqa"),
    ):
        with pytest.raises(ValueError, match=pattern):
            K.scaled_dot_product_attention(q, k, v, **kwargs)
    with pytest.raises(ValueError, match="FP32"):
        K.attention(q.float(), k.float(), v.float())
    with pytest.raises(ValueError, match="CUDA"):
        K.attention(q.cpu(), k.cpu(), v.cpu())
    with pytest.raises(ValueError, match="4D"):
        K.attention(q[0], k[0], v[0])
    with pytest.raises(ValueError, match="K/V shapes"):
        K.attention(q, k, v[:, :, :-1])
    with pytest.raises(ValueError, match="nonempty"):
        K.attention(q[:, :, :0], k, v)
    # unsupported inputs of the automatic entry point go to native SDPA unchanged
    qf, kf, vf = q.float(), k.float()[:, :1].expand(-1, 4, -1, -1), v.float()[:, :1].expand(-1, 4, -1, -1)
    want = torch.nn.functional.scaled_dot_product_attention(qf, kf, vf)
    torch.testing.assert_close(K.automatic_scaled_dot_product_attention(qf, kf, vf), want, atol=0, rtol=0)


# ------------------------------------------------------------------ key centering
@pytest.mark.parametrize("dtype", (torch.bfloat16, torch.float16))
def test_center_keys_kernel_matches_the_contract(dtype):
    c = load("center_keys_bf16" if dtype == torch.bfloat16 else "center_keys_fp16")
    got = native().center_keys(c["k"].cuda())
    # FP32 means may differ in the last bit by summation order: allow one ulp of the 16-bit type
    diff = (got.cpu().float() - c["centered"].float()).abs()
    assert float(diff.max()) <= float(c["centered"].float().abs().max()) * 2 ** (-7 if dtype == torch.bfloat16 else -10)
    keys = (c["k"].transpose(1, 2).contiguous().transpose(1, 2)).cuda()
    torch.testing.assert_close(native().center_keys(keys), got, atol=0, rtol=0)
    back = native().center_keys(c["grad"].cuda())
    assert float(back.float().sum(-2).abs().max()) < 0.1


@pytest.mark.parametrize("shape", ((4, 8, 4096, 128), (1, 3, 1000, 64), (2, 2, 65, 512), (1, 2, 777, 256),
                                   (6, 8, 4096, 128), (1, 2, 40001, 64)))
@pytest.mark.parametrize("dtype", (torch.bfloat16, torch.float16))
def test_center_keys_cluster_kernel(shape, dtype):
    """Tensors of up to 40 MB (any sequence length: the rows are read a second time from L2) and larger ones whose
    slab of S/8 rows fits in shared memory (the 50 MB case) are centred by one launch over thread-block clusters:
    same values as the FP32 definition (to one rounding of the mean), bitwise reproducible, any 16-byte row layout."""
    B, H, S, D = shape
    gen = torch.Generator().manual_seed(S + D)
    k = (torch.randn(B, H, S, D, generator=gen) + 3 * torch.randn(B, H, 1, D, generator=gen)).to(dtype).cuda()
    _, names = _launched(lambda: native().center_keys(k))
    assert names == {"center_keys"}
    got = native().center_keys(k)
    want = (k.float() - k.float().mean(dim=2, keepdim=True)).to(dtype)
    ulp = 2 ** (-7 if dtype == torch.bfloat16 else -10)
    assert float((got.float() - want.float()).abs().max()) <= float(want.float().abs().max()) * ulp
    torch.testing.assert_close(native().center_keys(k), got, atol=0, rtol=0)
    strided = strided_like_projection(k)
    torch.testing.assert_close(native().center_keys(strided), got, atol=0, rtol=0)
    # the column sums that are left: those of the definition (rounding k - mean to 16 bits is biased when the keys
    # sit on a coarse grid around a large offset), up to the elements whose rounding the last bit of the mean flips
    left = (got.float().sum(2) - want.float().sum(2)).abs().max()
    assert float(left) < 0.02 * S ** 0.5 * float(want.float().abs().max()) + 0.1


def _launched(fn):
    native().profile_read(reset=True)
    native().profile_enable(True)
    try:
        result = fn()
        torch.cuda.synchronize()
    finally:
        native().profile_enable(False)
    return result, set(native().profile_read(reset=True))


@pytest.mark.parametrize("causal,masked", ((False, False), (True, False), (False, True), (True, True)))
def test_centered_attention_matches_fp64(causal, masked):
    gen = torch.Generator().manual_seed(44)
    q = torch.randn(2, 4, 33, 64, generator=gen).bfloat16().cuda()
    k = (torch.randn(2, 2, 49, 64, generator=gen) + 4).bfloat16().cuda()
    v = torch.randn(2, 2, 49, 64, generator=gen).bfloat16().cuda()
    dout = torch.randn(2, 4, 33, 64, generator=gen).bfloat16().cuda()
    mask = None
    if masked:
        mask = (torch.rand(33, 49, generator=gen) > 0.2)
        mask[0] = False
        mask = mask.cuda()
    actual = run_attention(api().attention, q, k, v, dout, mask=mask, causal=causal, scale=-0.125, center_keys=True)
    exact = ao.math_reference((q.cpu(), k.cpu(), v.cpu()), dout.cpu(), None if mask is None else mask.cpu(), causal,
                              -0.125)
    for name, got, want in zip(NAMES, actual, exact):
        assert ao.relative_error(got.cpu(), want) < 0.04, name
    assert float(actual[2].float().sum(-2).abs().max()) < 0.05


# ------------------------------------------------- torch.compile and CUDA graphs
def test_compiled_attention_matches_eager():
    K = api()
    q, k, v, dout = make_inputs(1, 4, 2, 200, 200, 128, torch.bfloat16, seed=81)
    compiled = torch.compile(K.attention, fullgraph=True)
    eager = run_attention(K.attention, q, k, v, dout, causal=True)
    traced = run_attention(compiled, q, k, v, dout, causal=True)
    for a, b in zip(eager, traced):
        torch.testing.assert_close(a, b, atol=0, rtol=0)
    eager = run_attention(K.attention, q, k, v, dout, center_keys=True)
    traced = run_attention(compiled, q, k, v, dout, center_keys=True)
    for a, b in zip(eager, traced):
        torch.testing.assert_close(a, b, atol=0, rtol=0)


def test_cuda_graph_replay_with_changed_inputs_and_mask():
    K = api()
    q, k, v, dout = make_inputs(1, 2, 2, 260, 260, 128, torch.bfloat16, seed=82)
    mask = (torch.arange(260) < 200)[None, None, None, :].cuda().clone()
    leaves = [t.clone().requires_grad_(True) for t in (q, k, v)]
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        for _ in range(3):
            out = K.attention(*leaves, mask=mask, center_keys=True)
            torch.autograd.grad(out, leaves, dout)
    torch.cuda.current_stream().wait_stream(stream)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        out = K.attention(*leaves, mask=mask, center_keys=True)
        grads = torch.autograd.grad(out, leaves, dout)
    # new values in the same storage, including a different mask, then replay
    q2, k2, v2, dout2 = make_inputs(1, 2, 2, 260, 260, 128, torch.bfloat16, seed=83)
    with torch.no_grad():
        for leaf, new in zip(leaves, (q2, k2 + 3, v2)):
            leaf.copy_(new)
        dout.copy_(dout2)
        mask.copy_((torch.arange(260) < 131)[None, None, None, :])
        out.fill_(float("nan"))
    graph.replay()
    torch.cuda.synchronize()
    want = run_attention(K.attention, leaves[0].detach(), leaves[1].detach(), leaves[2].detach(), dout, mask=mask,
                         center_keys=True)
    for got, ref in zip((out, *grads), want):
        torch.testing.assert_close(got, ref, atol=0, rtol=0)


@pytest.mark.parametrize("kind", ("wide_head", "neighborhood"))
def test_cuda_graph_replay_of_the_other_tensor_core_families(kind):
    """Forward + backward of the wide-head and neighbourhood families captured once and replayed on new data."""
    K = api()
    gen = torch.Generator().manual_seed(84)
    if kind == "wide_head":
        shape_q, shape_k, dtype = (1, 4, 200, 512), (1, 2, 200, 512), torch.bfloat16

        def call(q, k, v):
            return K.attention(q, k, v, causal=True)
    else:
        shape_q = shape_k = (1, 2, 4 * 10 * 12, 64)
        dtype = torch.float16

        def call(q, k, v):
            return K.neighborhood_attention(q, k, v, spatial_shape=(4, 10, 12), window_size=(3, 5, 7), scale=0.125)

    def fresh():
        q = torch.randn(shape_q, generator=gen).to(dtype).cuda()
        k = torch.randn(shape_k, generator=gen).to(dtype).cuda()
        v = torch.randn(shape_k, generator=gen).to(dtype).cuda()
        g = torch.randn(shape_q, generator=gen).to(dtype).cuda()
        return q, k, v, g

    q, k, v, dout = fresh()
    leaves = [t.clone().requires_grad_(True) for t in (q, k, v)]
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        for _ in range(2):
            torch.autograd.grad(call(*leaves), leaves, dout)
    torch.cuda.current_stream().wait_stream(stream)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        out = call(*leaves)
        grads = torch.autograd.grad(out, leaves, dout)
    q2, k2, v2, dout2 = fresh()
    with torch.no_grad():
        for leaf, new in zip(leaves, (q2, k2, v2)):
            leaf.copy_(new)
        dout.copy_(dout2)
        out.fill_(float("nan"))
    graph.replay()
    torch.cuda.synchronize()
    again = [t.detach().clone().requires_grad_(True) for t in leaves]
    ref_out = call(*again)
    ref = (ref_out.detach(), *torch.autograd.grad(ref_out, again, dout))
    for got, want in zip((out, *grads), ref):
        torch.testing.assert_close(got, want, atol=0, rtol=0)
    assert native().device_status(reset=True) == 0


def test_activation_checkpointing_and_prescaled_queries():
    """The caller patterns of the reference's integration notes: a [B, S, H, D] projection layout, queries
    that already carry the softmax scale (scale = 1.0), and recomputation under torch.utils.checkpoint."""
    from torch.utils.checkpoint import checkpoint

    K = api()
    q, k, v, dout = make_inputs(2, 4, 2, 384, 384, 128, torch.bfloat16, seed=85)
    q = (q.float() * 128 ** -0.5).to(torch.bfloat16)
    q, k, v = (strided_like_projection(t) for t in (q, k, v))

    def block(q_, k_, v_):
        return K.attention(q_, k_, v_, causal=True, scale=1.0)

    plain = [t.detach().clone().requires_grad_(True) for t in (q, k, v)]
    out_plain = block(*plain)
    grads_plain = torch.autograd.grad(out_plain, plain, dout)
    again = [t.detach().clone().requires_grad_(True) for t in (q, k, v)]
    out_ckpt = checkpoint(block, *again, use_reentrant=False)
    grads_ckpt = torch.autograd.grad(out_ckpt, again, dout)
    for a, b in zip((out_plain, *grads_plain), (out_ckpt, *grads_ckpt)):
        torch.testing.assert_close(a, b, atol=0, rtol=0)
    check_against_oracle((out_plain.detach(), *grads_plain), q, k, v, dout, None, True, 1.0)


def test_two_streams_give_identical_results():
    import threading

    K = api()
    q, k, v, dout = make_inputs(1, 4, 2, 300, 300, 128, torch.bfloat16, seed=84)
    results = [None, None]

    def work(slot):
        stream = torch.cuda.Stream()
        with torch.cuda.stream(stream):
            results[slot] = run_attention(K.attention, q, k, v, dout, causal=True)
        stream.synchronize()

    threads = [threading.Thread(target=work, args=(i,)) for i in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    for a, b in zip(*results):
        torch.testing.assert_close(a, b, atol=0, rtol=0)
    assert native().cache_size() <= 128


# --------------------------------------------------------- full-size properties
def test_llm_gqa_config_row_sampled():
    """The default benchmark shape at batch 1: q scaled by 8, keys offset per head, tiny dO; checks sampled rows."""
    gen = torch.Generator().manual_seed(3)
    B, Hq, Hkv, S, D = 1, 8, 2, 4096, 128
    q = (8 * torch.randn(B, Hq, S, D, generator=gen)).bfloat16().cuda()
    k = (torch.randn(B, Hkv, S, D, generator=gen) + 2 * torch.randn(B, Hkv, 1, D, generator=gen)).bfloat16().cuda()
    v = torch.randn(B, Hkv, S, D, generator=gen).bfloat16().cuda()
    dout = (math.sqrt(1e-3) * torch.randn(B, Hq, S, D, generator=gen)).bfloat16().cuda()
    out, dq, dk, dv = run_attention(api().attention, q, k, v, dout, causal=True)
    rows = torch.cat([torch.arange(0, 128), torch.arange(S - 128, S), torch.randint(128, S - 128, (128,), generator=gen)])
    heads = [0, 5]
    for h in heads:
        sel = (q[:, h:h + 1].cpu(), k[:, h // 4:h // 4 + 1].cpu(), v[:, h // 4:h // 4 + 1].cpu())
        part = ao.contract_reference(sel, dout[:, h:h + 1].cpu(), None, True, None, output=out[:, h:h + 1].cpu(),
                                     query_rows=rows)
        assert ao.relative_error(out[:, h:h + 1, rows].cpu(), part[0]) < 0.01
        assert ao.relative_error(dq[:, h:h + 1, rows].cpu(), part[1]) < 0.01
    # dK/dV of one K/V head need every query row of its four query heads
    sel = (q[:, :4].cpu(), k[:, :1].cpu(), v[:, :1].cpu())
    full = ao.contract_reference(sel, dout[:, :4].cpu(), None, True, None, output=out[:, :4].cpu())
    assert ao.relative_error(dk[:, :1].cpu(), full[2]) < 0.01
    assert ao.relative_error(dv[:, :1].cpu(), full[3]) < 0.01
    # centered run: same output within the looser centering gate, sum_S dK == 0
    outc, dqc, dkc, dvc = run_attention(api().attention, q, k, v, dout, causal=True, center_keys=True)
    assert ao.relative_error(outc[:, :4].cpu(), full[0]) < 0.04
    assert ao.relative_error(dvc[:, :1].cpu(), full[3]) < 0.04
    assert float(dkc.float().sum(-2).abs().max()) < 0.05 * float(dkc.float().abs().max()) * math.sqrt(S)


# ------------------------------------------------------------------ randomised sweep
def _random_case(index):
    gen = torch.Generator().manual_seed(9000 + index)

    def pick(options):
        return options[int(torch.randint(len(options), (1,), generator=gen))]

    D = pick((64, 128, 128, 256, 512))
    group = pick((1, 2, 4))
    Hkv = pick((1, 2))
    B = pick((1, 2))
    Sq = int(torch.randint(1, 420, (1,), generator=gen))
    Sk = int(torch.randint(2, 420, (1,), generator=gen))
    causal = bool(torch.randint(2, (1,), generator=gen))
    kind = pick(("none", "none", "keys", "full2d", "per_head", "banded"))
    dtype = pick((torch.bfloat16, torch.float16))
    scale = pick((None, None, -0.11, 0.3))
    return B, Hkv * group, Hkv, Sq, Sk, D, causal, kind, dtype, scale, gen


@pytest.mark.parametrize("index", range(36))
def test_random_shapes_masks_and_scales(index):
    """Seeded random shapes (ragged lengths, GQA, every mask kind, both dtypes, signed scales) through whichever
    tensor-core family serves them, against the oracle."""
    B, Hq, Hkv, Sq, Sk, D, causal, kind, dtype, scale, gen = _random_case(index)
    q, k, v, dout = make_inputs(B, Hq, Hkv, Sq, Sk, D, dtype, seed=9100 + index)
    mask = None
    if kind == "keys":
        mask = (torch.rand(B, 1, 1, Sk, generator=gen) > 0.3)
    elif kind == "full2d":
        mask = torch.rand(Sq, Sk, generator=gen) > 0.4
    elif kind == "per_head":
        mask = torch.rand(B, Hq, Sq, Sk, generator=gen) > 0.5
    elif kind == "banded":
        idx_q, idx_k = torch.arange(Sq)[:, None], torch.arange(Sk)[None, :]
        mask = ((idx_q - idx_k).abs() < 70)[None, None]
    if mask is not None:
        mask = mask.cuda()
    expanded = None if mask is None else mask.expand(B, Hq, Sq, Sk)
    assert native().selected_family(q, k, v, expanded, causal) == (1 if D <= 128 else 2)
    actual = run_attention(api().attention, q, k, v, dout, mask=mask, causal=causal, scale=scale)
    check_against_oracle(actual, q, k, v, dout, mask, causal, scale, label=f"random{index} ")
    assert native().device_status(reset=True) == 0
