"""GPU parity tests for 2-D / 3-D neighbourhood attention against the CPU oracle."""

import pytest
import torch

from oracle import attention_oracle as ao
from oracle import neighborhood_oracle as no
from tests.golden_io import NEIGHBORHOOD_CASES, load
from tests.helpers import NAMES, TOL

pytestmark = pytest.mark.gpu


def api():
    import kohakufa_cute

    return kohakufa_cute


def run(q, k, v, dout, spatial, window, scale):
    leaves = [t.detach().clone().requires_grad_(True) for t in (q, k, v)]
    out = api().neighborhood_attention(*leaves, spatial_shape=spatial, window_size=window, scale=scale)
    grads = torch.autograd.grad(out, leaves, dout)
    return (out.detach(), *grads)


def gate(actual, q, k, v, dout, spatial, window, scale):
    tol = TOL[q.dtype]
    cpu = tuple(t.cpu() for t in (q, k, v))
    exact = no.na_math_reference(cpu, dout.cpu(), spatial, window, scale)
    policy = no.na_contract_reference(cpu, dout.cpu(), spatial, window, scale, actual[0].cpu())
    for name, got, want_exact, want in zip(NAMES, actual, exact, policy):
        got = got.cpu()
        assert bool(torch.isfinite(got).all()), name
        for reference in (want_exact, want):
            if float(reference.abs().max()) > 0:
                assert ao.per_head_relative_error(got, reference) < tol["norm"], name
            else:
                assert float(got.abs().max()) == 0, name
        torch.testing.assert_close(got.double(), want, atol=tol["elem"], rtol=tol["elem"])


@pytest.mark.parametrize("index", NEIGHBORHOOD_CASES)
def test_golden_cases(index):
    c = load(f"neighborhood_case{index}")
    spatial = tuple(int(x) for x in c["spatial"])
    window = tuple(int(x) for x in c["window"])
    q, k, v, dout = (c[n].cuda() for n in ("q", "k", "v", "dout"))
    actual = run(q, k, v, dout, spatial, window, c["scale"])
    gate(actual, q, k, v, dout, spatial, window, c["scale"])
    tol = TOL[q.dtype]["norm"]
    for name, got in zip(NAMES, actual):
        want = c[f"exact_{name}"]
        if float(want.abs().max()) > 0:
            assert ao.per_head_relative_error(got.cpu(), want) < tol, name
    if len(spatial) == 3:
        assert ao.relative_error(actual[0].cpu(), c["two_term"]) < tol


@pytest.mark.parametrize("dtype", (torch.float16, torch.bfloat16))
@pytest.mark.parametrize("spatial,window", (((9, 11), (3, 5)), ((8, 8), (4, 6)), ((3, 7, 9), (3, 5, 5)),
                                            ((2, 6, 5), (2, 2, 4)), ((1, 1, 70), (1, 1, 7))))
def test_random_grids(spatial, window, dtype):
    gen = torch.Generator().manual_seed(sum(spatial) * 7 + sum(window))
    tokens = 1
    for n in spatial:
        tokens *= n
    q, k, v, dout = (torch.randn(2, 3, tokens, 64, generator=gen).to(dtype).cuda() for _ in range(4))
    for scale in (0.125, -0.125):
        actual = run(q, k, v, dout, spatial, window, scale)
        gate(actual, q, k, v, dout, spatial, window, scale)


def test_shifted_border_counts_are_exact():
    # 1x5 grid, window 3, zero scores: P = 1/3 everywhere, so dV counts how many queries see each key
    q = torch.zeros(1, 1, 5, 64, device="cuda", dtype=torch.float16)
    dout = torch.ones_like(q)
    out, dq, dk, dv = run(q, q.clone(), torch.ones_like(q), dout, (1, 5), (1, 3), 0.125)
    third = float(torch.tensor(1 / 3).half())
    want = torch.tensor([2, 3, 5, 3, 2], dtype=torch.float32) * third
    torch.testing.assert_close(dv[0, 0, :, 0].float().cpu(), want, atol=2e-3, rtol=2e-3)
    assert float(dq.abs().max()) == 0 and float(dk.abs().max()) == 0


def test_video_layout_adapter():
    K = api()
    gen = torch.Generator().manual_seed(9)
    shape = (1, 3, 6, 5, 2, 64)
    q, k, v, dout = (torch.randn(shape, generator=gen).half().cuda() for _ in range(4))
    leaves = [t.clone().requires_grad_(True) for t in (q, k, v)]
    out = K.neighborhood_attention_3d(*leaves, (11, 3, 5), None, 0.125)  # 11-frame window clipped to 3
    assert out.shape == shape
    flat = [t.flatten(1, 3).transpose(1, 2) for t in (q, k, v)]
    ref = K.neighborhood_attention(*flat, spatial_shape=(3, 6, 5), window_size=(3, 3, 5), scale=0.125)
    torch.testing.assert_close(out, ref.transpose(1, 2).reshape(shape), atol=0, rtol=0)
    grads = torch.autograd.grad(out, leaves, dout)
    fl = [t.flatten(1, 3).transpose(1, 2) for t in (q, k, v, dout)]
    actual = (ref, *[g.flatten(1, 3).transpose(1, 2) for g in grads])
    gate(actual, *fl, (3, 6, 5), (3, 3, 5), 0.125)
    for bad in (True, (False, True, False)):
        with pytest.raises(ValueError, match="noncausal"):
            K.neighborhood_attention_3d(q, k, v, 3, bad)
    with pytest.raises(ValueError, match="window_size"):
        K.neighborhood_attention(*flat, spatial_shape=(3, 6, 5), window_size=(4, 3, 5))


def test_compiled_neighborhood_with_equal_length_different_geometry():
    K = api()
    gen = torch.Generator().manual_seed(10)
    q, k, v = (torch.randn(1, 2, 60, 64, generator=gen).half().cuda() for _ in range(3))

    def fn(q, k, v, spatial, window):
        return K.neighborhood_attention(q, k, v, spatial_shape=spatial, window_size=window)

    compiled = torch.compile(fn)
    for spatial, window in (((6, 10), (3, 3)), ((10, 6), (3, 3)), ((3, 4, 5), (3, 3, 3))):
        torch.testing.assert_close(compiled(q, k, v, spatial, window), fn(q, k, v, spatial, window), atol=0, rtol=0)


# ------------------------------------------------ tensor-core family against the window-enumerating family
def _kernel_names(fn):
    from kohakufa_cute import native

    native.profile_read(reset=True)
    native.profile_enable(True)
    try:
        result = fn()
        torch.cuda.synchronize()
    finally:
        native.profile_enable(False)
    return result, set(native.profile_read(reset=True))


def _run_misaligned(q, k, v, dout, spatial, window, scale):
    """Same values behind views whose rows start 8 bytes off a 16-byte boundary: the tensor-memory
    kernels cannot address them, so the exact-window CUDA-core kernels run."""
    wides = []
    for t in (q, k, v):
        wide = torch.zeros(*t.shape[:-1], t.shape[-1] + 8, device=t.device, dtype=t.dtype)
        wide[..., 4:4 + t.shape[-1]] = t
        wides.append(wide.requires_grad_(True))
    views = [w[..., 4:4 + q.shape[-1]] for w in wides]
    out = api().neighborhood_attention(*views, spatial_shape=spatial, window_size=window, scale=scale)
    grads = torch.autograd.grad(out, wides, dout)
    return (out.detach(), *[g[..., 4:4 + q.shape[-1]] for g in grads])


@pytest.mark.parametrize("spatial,window,dtype", (((16, 32, 32), (3, 7, 7), torch.float16),
                                                  ((5, 32, 32), (3, 7, 7), torch.bfloat16),
                                                  ((64, 64), (7, 7), torch.bfloat16),
                                                  ((3, 17, 29), (3, 5, 9), torch.float16)))
def test_tensor_core_family_matches_window_enumeration_at_full_size(spatial, window, dtype):
    """The benchmark's 16x32x32 / (3,7,7) grid (and the reference's published shapes): the dense-tile
    tensor-core kernels and the exact-window kernels follow one arithmetic contract, so their results
    agree to accumulation-order noise; the small-grid tests pin both to the oracle."""
    gen = torch.Generator().manual_seed(len(spatial) * 100 + spatial[-1])
    tokens = 1
    for n in spatial:
        tokens *= n
    heads = 4 if tokens > 8192 else 2
    q, k, v, dout = (torch.randn(1, heads, tokens, 64, generator=gen).to(dtype).cuda() for _ in range(4))
    fast, fast_names = _kernel_names(lambda: run(q, k, v, dout, spatial, window, 0.125))
    slow, slow_names = _kernel_names(lambda: _run_misaligned(q, k, v, dout, spatial, window, 0.125))
    assert {"na_pipeline_forward", "na_pipeline_backward_q", "na_pipeline_backward_kv"} <= fast_names
    assert {"neighborhood_forward", "neighborhood_backward_q", "neighborhood_backward_kv"} <= slow_names
    from kohakufa_cute import native

    assert native.device_status(reset=True) == 0
    for name, a, b in zip(NAMES, fast, slow):
        assert bool(torch.isfinite(a).all()), name
        # two roundings to the 16-bit type of (almost) the same FP32 value differ by at most one ulp
        assert ao.per_head_relative_error(a.cpu(), b.cpu().double()) < 0.5 * TOL[dtype]["norm"], name
        torch.testing.assert_close(a.float(), b.float(), atol=TOL[dtype]["elem"], rtol=TOL[dtype]["elem"])


def _random_geometry(index):
    gen = torch.Generator().manual_seed(7000 + index)

    def rand(lo, hi):
        return int(torch.randint(lo, hi + 1, (1,), generator=gen))

    nd = 2 if index % 3 == 0 else 3
    while True:
        spatial = tuple(rand(1, 14 if nd == 3 else 40) for _ in range(nd))
        tokens = 1
        for n in spatial:
            tokens *= n
        if 2 <= tokens <= 1600:
            break
    while True:
        window = tuple(rand(1, min(n, 11)) for n in spatial)
        seen = 1
        for w in window:
            seen *= w
        if seen >= 2:  # a window of one key has P = 1 and zero score gradients: nothing to compare relatively
            break
    dtype = torch.float16 if index % 2 else torch.bfloat16
    scale = (0.125, -0.125, 0.3)[index % 3]
    return spatial, window, dtype, scale, tokens


@pytest.mark.parametrize("index", range(24))
def test_random_grids_and_windows(index):
    """Seeded random grids and windows (windows equal to the extent, windows of one, extents of one, odd sizes)
    through the tensor-core family, against the oracle."""
    spatial, window, dtype, scale, tokens = _random_geometry(index)
    gen = torch.Generator().manual_seed(7100 + index)
    q, k, v, dout = (torch.randn(1, 2, tokens, 64, generator=gen).to(dtype).cuda() for _ in range(4))
    actual, names = _kernel_names(lambda: run(q, k, v, dout, spatial, window, scale))
    assert "na_pipeline_forward" in names and "na_pipeline_backward_kv" in names
    gate(actual, q, k, v, dout, spatial, window, scale)
    from kohakufa_cute import native

    assert native.device_status(reset=True) == 0
