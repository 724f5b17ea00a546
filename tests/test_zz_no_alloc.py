"""The allocation-free key-centring entry point (``kfa_center_keys_static``) against the ordinary one.

Some hosts of the library cannot allocate device memory while they run (a server with a fixed
arena, a C plugin host that owns only the tensors it passes in), so this entry point takes its
scratch from a fixed array inside the library.  The test calls it through the C ABI several times in a
row on shapes that really go through that array (fewer than 64 rows, a channel count or a tensor
size the one-launch cluster kernel does not take), a many-split shape followed by few-split ones so that
the later calls meet the earlier calls' leftovers, and requires bit-identical results to
``kfa_center_keys`` (same kernels, same summation order).  It also covers a shape the cluster kernel
serves, for which the array is not touched at all.  The file sorts last so that a run stopping at the
first failure has already run everything else; it must also pass alone in a fresh process.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

# (shape, dtype, kernels launched): three = the partial sums and means went through the static array
CASES = (((1, 1, 172032, 128), torch.bfloat16, 3),  # 32 sequence splits; 44 MB: too large for either cluster kernel
         ((1, 2, 50, 64), torch.float16, 3),       # one split, fewer than 64 rows
         ((2, 3, 700, 96), torch.bfloat16, 3),     # 5 splits, 96 channels
         ((2, 3, 700, 128), torch.bfloat16, 1))    # cluster kernel: no scratch at all


def _static_launches(native):
    return native.launch_stats().get("center_keys_static", 0)


def test_static_scratch_entry_point_matches_caller_scratch_on_calls_in_a_row():
    from kohakufa_cute import native

    lib = native.library()
    gen = torch.Generator().manual_seed(123)
    for round_index in range(2):  # the second round meets the first round's contents in the array
        for shape, dtype, launches in CASES:
            k = (torch.randn(shape, generator=gen) + 4).to(dtype).cuda()
            want = native.center_keys(k)
            got = torch.full_like(k, float("nan"))
            rk, ro = native.describe(k), native.describe(got)
            stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
            before = _static_launches(native)
            code = lib.kfa_center_keys_static(ctypes.byref(rk), ctypes.byref(ro), stream)
            assert code == 0, lib.kfa_last_error()
            torch.cuda.synchronize()
            assert _static_launches(native) - before == launches, (shape, round_index)
            torch.testing.assert_close(got, want, atol=0, rtol=0)
            # and against plain PyTorch arithmetic, so that a shared defect of both entry points would show
            kf = k.float()
            reference = (kf - kf.mean(dim=-2, keepdim=True)).to(dtype)
            torch.testing.assert_close(got.float(), reference.float(), atol=2.0 ** -5, rtol=2.0 ** -7)
            if shape[2] >= 8:
                # strided (projection-layout) input through the Python wrapper
                ks = k.transpose(1, 2).contiguous().transpose(1, 2)
                torch.testing.assert_close(native.center_keys_static(ks), want, atol=0, rtol=0)
    assert native.device_status(reset=True) == 0


def test_static_scratch_entry_point_rejects_sizes_beyond_its_capacity():
    from kohakufa_cute import native

    limit = native.library().kfa_center_keys_static_limit()
    assert limit == 16384
    k = torch.zeros(1, limit // 128 + 1, 8, 128, device="cuda", dtype=torch.bfloat16)
    before = native.launch_count()
    with pytest.raises(RuntimeError, match="exceeds the fixed scratch capacity"):
        native.center_keys_static(k)
    assert native.launch_count() == before
