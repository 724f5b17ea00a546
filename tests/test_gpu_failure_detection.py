"""Failure detection on the GPU without any fault: a bounded wait that runs out is reported through the
status word, stops the rest of the launch, keeps later kernels idle until it is acknowledged, and leaves
the context usable."""

import pytest
import torch

from oracle import attention_oracle as ao
from tests.helpers import make_inputs

pytestmark = pytest.mark.gpu


def test_bounded_wait_runs_out_is_reported_and_cleared():
    import kohakufa_cute
    from kohakufa_cute import native

    native.device_status(reset=True)
    ctas = 20000  # several waves of 64-thread CTAs: the later ones start after the first ones gave up
    skipped = native.self_test_wait(2_000_000, ctas)  # about a millisecond per wait
    assert 0 < skipped < ctas
    assert native.device_status(reset=False) == 9001

    # until the condition is acknowledged no entry point launches (nobody is handed unwritten outputs)
    q, k, v, dout = make_inputs(1, 2, 2, 256, 256, 128, torch.bfloat16, seed=91)
    before = native.launch_count()
    with pytest.raises(native.DeviceTimeoutError, match="ran out"):
        kohakufa_cute.attention(q, k, v, causal=True)
    with pytest.raises(native.DeviceTimeoutError):
        kohakufa_cute.neighborhood_attention(q[..., :64].contiguous(), k[..., :64].contiguous(), v[..., :64].contiguous(),
                                             spatial_shape=(16, 16), window_size=3)
    assert native.launch_count() == before
    assert native.device_status(reset=True) == 9001

    # acknowledged: the same call works and matches the oracle
    out = kohakufa_cute.attention(q, k, v, causal=True)
    torch.cuda.synchronize()
    assert native.device_status(reset=True) == 0
    want = ao.math_reference([t.cpu() for t in (q, k, v)], dout.cpu(), None, True, None)[0]
    assert ao.per_head_relative_error(out.cpu(), want) < 0.01


def test_self_test_rejects_unbounded_limits():
    from kohakufa_cute import native

    with pytest.raises(ValueError):
        native.self_test_wait(10**12, 1)
    with pytest.raises(ValueError):
        native.self_test_wait(1000, 0)
