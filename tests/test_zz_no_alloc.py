"""The allocation-free key-centring entry point (``kfa_center_keys_static``) against the ordinary one.

Some hosts of the library cannot allocate device memory while they run (a server with a fixed
arena, a C plugin host that owns only the tensors it passes in), so this entry point takes its
scratch from a fixed array inside the library.  The test calls it through the C ABI twice in a row,
with different shapes so that the second call meets the first call's leftovers in the shared array,
and requires bit-identical results to ``kfa_center_keys`` (same kernels, same summation order).
It lives in a file that sorts last so that a run stopping at the first failure has already run
everything else; it must also pass alone in a fresh process.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_static_scratch_entry_point_matches_caller_scratch_twice_in_a_row():
    from kohakufa_cute import native

    lib = native.library()
    gen = torch.Generator().manual_seed(123)
    shapes = [((2, 3, 700, 128), torch.bfloat16), ((1, 2, 130, 64), torch.float16)]
    for shape, dtype in shapes:
        k = (torch.randn(shape, generator=gen) + 4).to(dtype).cuda()
        want = native.center_keys(k)
        got = torch.full_like(k, float("nan"))
        rk, ro = native.describe(k), native.describe(got)
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        code = lib.kfa_center_keys_static(ctypes.byref(rk), ctypes.byref(ro), stream)
        assert code == 0, lib.kfa_last_error()
        torch.cuda.synchronize()
        torch.testing.assert_close(got, want, atol=0, rtol=0)
        # strided (projection-layout) input through the Python wrapper
        ks = k.transpose(1, 2).contiguous().transpose(1, 2)
        torch.testing.assert_close(native.center_keys_static(ks), want, atol=0, rtol=0)
    assert native.device_status(reset=True) == 0


def test_static_scratch_entry_point_rejects_sizes_beyond_its_capacity():
    from kohakufa_cute import native

    limit = native.library().kfa_center_keys_static_limit()
    assert limit == 16384
    k = torch.zeros(1, limit // 128 + 1, 8, 128, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="exceeds the fixed scratch capacity"):
        native.center_keys_static(k)
