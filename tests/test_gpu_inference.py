"""Forward passes nobody differentiates (no row statistics) and the forward split over the key axis for short
query sequences (decode shapes), against the oracle and against the ordinary path."""

import math

import pytest
import torch

from oracle import attention_oracle as ao
from tests.helpers import TOL, check_against_oracle, make_inputs, run_attention

pytestmark = pytest.mark.gpu


def api():
    import kohakufa_cute

    return kohakufa_cute


def native():
    from kohakufa_cute import native as module

    return module


@pytest.mark.parametrize("shape", ((1, 4, 2, 300, 300, 128, True), (2, 2, 2, 129, 257, 64, False),
                                   (1, 2, 1, 96, 96, 512, True), (1, 2, 2, 70, 65, 17, True)))
def test_forward_without_gradients_keeps_no_statistics_and_equals_the_training_forward(shape):
    B, Hq, Hkv, Sq, Sk, D, causal = shape
    q, k, v, _ = make_inputs(B, Hq, Hkv, Sq, Sk, D, torch.bfloat16, seed=Sq + D)
    with torch.no_grad():
        inference = api().attention(q, k, v, causal=causal)
    with torch.inference_mode():
        inference2 = api().attention(q, k, v, causal=causal)
    training = api().attention(q.clone().requires_grad_(True), k, v, causal=causal)
    assert torch.equal(inference, training.detach()) and torch.equal(inference2, inference)
    out, maximum, logsum, _ = native().forward(q, k, v, None, D ** -0.5, causal, statistics=False)
    assert maximum is None and logsum is None and torch.equal(out, inference)
    assert native().device_status(reset=True) == 0


DECODE_SHAPES = (
    # B, Hq, Hkv, Sq, Sk, D
    (1, 8, 2, 1, 8192, 128),
    (1, 32, 8, 1, 16384, 128),
    (2, 8, 2, 16, 8192, 64),
    (1, 4, 4, 200, 9000, 128),   # a remainder range
    (1, 16, 2, 1, 4096 + 300, 80),
)


@pytest.mark.parametrize("dtype", (torch.bfloat16, torch.float16))
@pytest.mark.parametrize("shape", DECODE_SHAPES)
def test_split_forward_matches_the_oracle_and_its_statistics_serve_the_backward(shape, dtype):
    B, Hq, Hkv, Sq, Sk, D = shape
    q, k, v, dout = make_inputs(B, Hq, Hkv, Sq, Sk, D, dtype, seed=Sk % 997)
    scale = D ** -0.5
    splits = native().split_plan(q, k, False)
    assert splits >= 2
    out, maximum, logsum, _ = native().forward_split(q, k, v, None, scale, splits)
    whole, whole_max, whole_log, _ = native().forward(q, k, v, None, scale, False)
    assert torch.equal(maximum, whole_max)  # the exact row maximum either way
    # maximum * scale + logsum * ln 2 == logsumexp(scale * Q K^T)
    want = torch.logsumexp(scale * torch.einsum("bhqd,bhkd->bhqk", q.float(),
                                                k.float().repeat_interleave(Hq // Hkv, dim=1)), dim=-1)
    torch.testing.assert_close(maximum * scale + logsum * math.log(2.0), want, atol=1e-3, rtol=1e-4)
    torch.testing.assert_close(logsum, whole_log, atol=2e-3, rtol=0)
    # the public API takes the decoding kernel for a few rows per K/V head and the split path for the other
    # shapes, with and without gradients
    decode = native().decode_served(q, k, v, None, False)
    name = "decode_forward" if decode else "merge_splits"
    names_before = native().launch_stats().get(name, 0)
    actual = run_attention(api().attention, q, k, v, dout)
    with torch.no_grad():
        inference = api().attention(q, k, v)
    assert native().launch_stats().get(name, 0) >= names_before + 2 * (1 if decode else B)
    assert torch.equal(inference, actual[0])
    if decode:
        torch.testing.assert_close(actual[0].float(), out.float(), atol=0.01, rtol=0.02)
    else:
        assert torch.equal(actual[0], out)
    check_against_oracle(actual, q, k, v, dout, None, False, None)
    assert native().device_status(reset=True) == 0


def test_split_forward_with_key_padding_and_hidden_ranges():
    B, Hq, Hkv, Sq, Sk, D = 1, 8, 2, 4, 8192, 128
    q, k, v, dout = make_inputs(B, Hq, Hkv, Sq, Sk, D, torch.bfloat16, seed=5)
    mask = (torch.arange(Sk, device="cuda") < 5000)[None, None, None, :]  # whole key ranges are hidden
    actual = run_attention(api().attention, q, k, v, dout, mask=mask)
    check_against_oracle(actual, q, k, v, dout, mask, False, None)
    assert float(actual[2][:, :, 5000:].abs().max()) == 0 and float(actual[3][:, :, 5000:].abs().max()) == 0
    nothing = torch.zeros(1, 1, 1, Sk, dtype=torch.bool, device="cuda")
    hidden = run_attention(api().attention, q, k, v, dout, mask=nothing)
    assert all(float(t.abs().max()) == 0 for t in hidden)


@pytest.mark.parametrize("heads", ((8, 2), (32, 8)))
def test_single_query_row_with_grouped_heads(heads):
    """One query row against 300 keys, 8/2 and 32/8 heads (a shape the reference pins,
    tests/test_tracker_regressions.py:135-165 of the reference project): too short to split."""
    Hq, Hkv = heads
    q, k, v, dout = make_inputs(1, Hq, Hkv, 1, 300, 128, torch.bfloat16, seed=Hq)
    assert native().split_plan(q, k, False) == 0
    actual = run_attention(api().attention, q, k, v, dout)
    check_against_oracle(actual, q, k, v, dout, None, False, None)
    scale = 128 ** -0.5
    _, maximum, logsum, _ = native().forward(q, k, v, None, scale, False)
    want = torch.logsumexp(scale * torch.einsum("bhqd,bhkd->bhqk", q.float(), k.float().repeat_interleave(Hq // Hkv, dim=1)), -1)
    torch.testing.assert_close(maximum * scale + logsum * math.log(2.0), want, atol=1e-3, rtol=1e-4)


DECODE_KERNEL_SHAPES = (
    # B, Hq, Hkv, Sq, Sk, D: query positions x grouped heads <= 8 rows per K/V head
    (1, 32, 8, 1, 32768, 128),
    (2, 8, 8, 1, 4097, 64),
    (1, 16, 2, 1, 5000, 128),     # eight rows per K/V head
    (3, 4, 2, 4, 777, 64),        # four positions x two heads, a ragged key count
    (1, 6, 2, 2, 12345, 128),     # six rows: a row count that is not a power of two
)


@pytest.mark.parametrize("dtype", (torch.bfloat16, torch.float16))
@pytest.mark.parametrize("shape", DECODE_KERNEL_SHAPES)
def test_decoding_kernel_matches_the_oracle_and_the_tensor_core_forward(shape, dtype):
    B, Hq, Hkv, Sq, Sk, D = shape
    q, k, v, dout = make_inputs(B, Hq, Hkv, Sq, Sk, D, dtype, seed=Sk % 991)
    assert native().decode_served(q, k, v, None, False)
    for scale in (D ** -0.5, -0.07):
        out, maximum, logsum, _ = native().forward_decode(q, k, v, scale)
        whole, whole_max, whole_log, _ = native().forward(q, k, v, None, scale, False)
        # the row maximum of the scores as this kernel sums them (FMA chains and a shuffle tree, not the tensor core's
        # order): equal up to FP32 summation order, and consistent with its own log-sum
        torch.testing.assert_close(maximum, whole_max, atol=1e-4, rtol=1e-5)
        c2 = abs(scale) * math.log2(math.e)
        torch.testing.assert_close(maximum * c2 + logsum, whole_max * c2 + whole_log, atol=2e-3, rtol=0)
        torch.testing.assert_close(out.float(), whole.float(), atol=0.01, rtol=0.02)
        bare, no_max, no_log, _ = native().forward_decode(q, k, v, scale, statistics=False)
        assert no_max is None and no_log is None and torch.equal(bare, out)
    actual = run_attention(api().attention, q, k, v, dout)
    check_against_oracle(actual, q, k, v, dout, None, False, None)
    # views of a larger cache (the usual decoding layout): rows stay 8-byte addressable
    cache_k = torch.randn(B, Hkv, Sk + 64, D, device="cuda").to(dtype)
    cache_v = torch.randn(B, Hkv, Sk + 64, D, device="cuda").to(dtype)
    cache_k[:, :, :Sk], cache_v[:, :, :Sk] = k, v
    sliced = run_attention(api().attention, q, cache_k[:, :, :Sk], cache_v[:, :, :Sk], dout)
    assert torch.equal(sliced[0], actual[0])
    assert native().device_status(reset=True) == 0


def test_decoding_kernel_refuses_other_shapes():
    q, k, v, _ = make_inputs(1, 16, 1, 1, 4096, 128, torch.bfloat16, seed=3)  # sixteen rows per K/V head
    assert not native().decode_served(q, k, v, None, False)
    with pytest.raises(ValueError, match="at most 8 query rows"):
        native().forward_decode(q, k, v, 0.1)

