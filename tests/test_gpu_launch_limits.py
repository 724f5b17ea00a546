"""Large batch x head grids keep exact singleton-key results, and key centring has no grid limit.

One visible key makes the answer exact without any score matrix: O = V, dQ = dK = 0, dV = sum of dO
(the reference pins the same shapes: tests/test_launch_limits.py:19-61 of the reference project).
"""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(q, k, v, dout, mask=None):
    import kohakufa_cute

    leaves = [t.detach().requires_grad_(True) for t in (q, k, v)]
    out = kohakufa_cute.attention(*leaves, mask=mask)
    grads = torch.autograd.grad(out, leaves, dout)
    return (out.detach(), *grads)


@pytest.mark.parametrize("batch,heads,queries,dim", ((1, 65534, 1, 64), (1, 65535, 1, 64), (1, 65536, 1, 64),
                                                     (256, 256, 1, 64), (65536, 1, 1, 64), (1, 65536, 129, 8),
                                                     (256, 256, 1, 257)))
def test_singleton_key_is_exact_across_grid_limits(batch, heads, queries, dim):
    gen = torch.Generator(device="cuda").manual_seed(batch + heads + dim)
    q = torch.randn(batch, heads, queries, dim, device="cuda", dtype=torch.float16, generator=gen)
    k = torch.randn(batch, heads, 1, dim, device="cuda", dtype=torch.float16, generator=gen)
    v = torch.randn(batch, heads, 1, dim, device="cuda", dtype=torch.float16, generator=gen)
    dout = torch.ones_like(q)
    out, dq, dk, dv = _run(q, k, v, dout)
    torch.testing.assert_close(out, v.expand_as(out), atol=0, rtol=0)
    assert int(dq.count_nonzero()) == 0 and int(dk.count_nonzero()) == 0
    torch.testing.assert_close(dv, dout.sum(2, keepdim=True), atol=0, rtol=0)


def test_query_and_key_launches_on_opposite_sides_of_the_limit():
    gen = torch.Generator(device="cuda").manual_seed(7)
    q = torch.randn(256, 256, 1, 64, device="cuda", dtype=torch.float16, generator=gen)
    k, v = (torch.randn(256, 1, 1, 64, device="cuda", dtype=torch.float16, generator=gen) for _ in range(2))
    out, dq, dk, dv = _run(q, k, v, torch.ones_like(q))
    torch.testing.assert_close(out, v.expand_as(q), atol=0, rtol=0)
    assert int(dq.count_nonzero()) == 0 and int(dk.count_nonzero()) == 0
    torch.testing.assert_close(dv, torch.full_like(v, 256), atol=0, rtol=0)


def test_masked_grid_limits():
    batch, heads = 256, 256
    gen = torch.Generator(device="cuda").manual_seed(8)
    q, k, v = (torch.randn(batch, heads, 1, 64, device="cuda", dtype=torch.float16, generator=gen) for _ in range(3))
    mask = (torch.arange(batch * heads, device="cuda").reshape(batch, heads, 1, 1) % 2) == 0
    dout = torch.ones_like(q)
    out, dq, dk, dv = _run(q, k, v, dout, mask=mask)
    torch.testing.assert_close(out, v.masked_fill(~mask, 0), atol=0, rtol=0)
    assert int(dq.count_nonzero()) == 0 and int(dk.count_nonzero()) == 0
    torch.testing.assert_close(dv, dout.masked_fill(~mask, 0), atol=0, rtol=0)


@pytest.mark.parametrize("shape", ((1, 65537, 8, 16), (256, 257, 64, 64), (2, 40000, 3, 24)))
def test_key_centering_beyond_65535_batch_heads(shape):
    """Both centring paths (the cluster kernel for 64 channels and 64 rows, the three-kernel path otherwise)
    index batch x heads on the first grid axis, which has no 65535 limit."""
    from kohakufa_cute import native

    gen = torch.Generator(device="cuda").manual_seed(shape[1])
    k = (torch.randn(shape, device="cuda", generator=gen) + 3).to(torch.bfloat16)
    got = native.center_keys(k)
    kf = k.float()
    want = (kf - kf.mean(dim=-2, keepdim=True)).to(k.dtype)
    torch.testing.assert_close(got.float(), want.float(), atol=2 ** -6, rtol=2 ** -7)
    assert float(got.float().sum(-2).abs().max()) < 0.5
