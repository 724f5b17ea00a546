"""ctypes binding of the C-ABI CUDA library (``libkfa.so``, declared in ``include/kfa.h``).

This module plays the role of the reference's compiled host launcher
(``src/kohakufa_cute/native.cpp`` of the reference project): it allocates outputs
and scratch with the PyTorch caching allocator, describes every tensor to the
library as a plain pointer/size/stride record and launches on the current
stream.  There is no fallback: when the library is missing, loading raises.
"""

from __future__ import annotations

import ctypes
import os
import threading

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIBRARY_PATH = os.path.join(_HERE, "libkfa.so")

KFA_F16, KFA_BF16, KFA_F32, KFA_BOOL, KFA_I32 = range(5)
_DTYPES = {
    torch.float16: KFA_F16,
    torch.bfloat16: KFA_BF16,
    torch.float32: KFA_F32,
    torch.bool: KFA_BOOL,
    torch.int32: KFA_I32,
}


class KfaTensor(ctypes.Structure):
    _fields_ = [
        ("data", ctypes.c_void_p),
        ("dtype", ctypes.c_int32),
        ("ndim", ctypes.c_int32),
        ("sizes", ctypes.c_int64 * 6),
        ("strides", ctypes.c_int64 * 6),
    ]


_TP = ctypes.POINTER(KfaTensor)
_I64P = ctypes.POINTER(ctypes.c_int64)

# name -> (restype, argtypes); must list every symbol declared in include/kfa.h
SIGNATURES = {
    "kfa_version": (ctypes.c_int, []),
    "kfa_last_error": (ctypes.c_char_p, []),
    "kfa_init": (ctypes.c_int, []),
    "kfa_forward": (ctypes.c_int, [_TP, _TP, _TP, _TP, _TP, _TP, _TP, _TP, ctypes.c_float, ctypes.c_int,
                                   ctypes.c_void_p]),
    "kfa_pack_mask": (ctypes.c_int, [_TP, _TP, ctypes.c_void_p]),
    "kfa_backward_workspace_bytes": (ctypes.c_size_t, [_TP, _TP]),
    "kfa_backward": (ctypes.c_int, [_TP] * 12 + [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_float, ctypes.c_int,
                                                 ctypes.c_void_p]),
    "kfa_forward_decode_workspace_bytes": (ctypes.c_size_t, [_TP, _TP]),
    "kfa_forward_decode": (ctypes.c_int, [_TP] * 6 + [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_float, ctypes.c_void_p]),
    "kfa_forward_running": (ctypes.c_int, [_TP] * 8 + [ctypes.c_float, ctypes.c_int, ctypes.c_void_p]),
    "kfa_finish_running": (ctypes.c_int, [_TP] * 6 + [ctypes.c_void_p]),
    "kfa_backward_partial": (ctypes.c_int, [_TP] * 12 + [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_float, ctypes.c_int,
                                                         ctypes.c_int, ctypes.c_int, ctypes.c_void_p]),
    "kfa_center_keys_workspace_bytes": (ctypes.c_size_t, [_TP]),
    "kfa_center_keys": (ctypes.c_int, [_TP, _TP, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p]),
    "kfa_center_keys_static_limit": (ctypes.c_size_t, []),
    "kfa_center_keys_static": (ctypes.c_int, [_TP, _TP, ctypes.c_void_p]),
    "kfa_neighborhood_forward": (ctypes.c_int, [_TP] * 6 + [_I64P, ctypes.c_int, _I64P, ctypes.c_float,
                                                            ctypes.c_void_p]),
    "kfa_neighborhood_backward_workspace_bytes": (ctypes.c_size_t, [_TP]),
    "kfa_neighborhood_backward": (ctypes.c_int, [_TP] * 10 + [ctypes.c_void_p, ctypes.c_size_t, _I64P, ctypes.c_int,
                                                              _I64P, ctypes.c_float, ctypes.c_void_p]),
    "kfa_merge_partial": (ctypes.c_int, [_TP] * 6 + [ctypes.c_float, ctypes.c_void_p]),
    "kfa_merge_splits": (ctypes.c_int, [_TP] * 6 + [ctypes.c_float, ctypes.c_void_p]),
    "kfa_cache_size": (ctypes.c_int, []),
    "kfa_clear_cache": (None, []),
    "kfa_launch_count": (ctypes.c_uint64, []),
    "kfa_launch_stats": (ctypes.c_int, [ctypes.c_int, ctypes.c_char_p, ctypes.c_size_t,
                                        ctypes.POINTER(ctypes.c_uint64)]),
    "kfa_device_status": (ctypes.c_int, [ctypes.c_int]),
    "kfa_profile_enable": (None, [ctypes.c_int]),
    "kfa_profile_collect": (ctypes.c_int, []),
    "kfa_profile_entry": (ctypes.c_int, [ctypes.c_int, ctypes.c_char_p, ctypes.c_size_t,
                                         ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_uint64)]),
    "kfa_profile_reset": (None, []),
    "kfa_selected_family": (ctypes.c_int, [_TP, _TP, _TP, _TP, ctypes.c_int, ctypes.c_int]),
    "kfa_self_test_wait": (ctypes.c_int, [ctypes.c_longlong, ctypes.c_int, ctypes.POINTER(ctypes.c_int),
                                          ctypes.c_void_p]),
}

_lock = threading.Lock()
_library = None


def library():
    """Loads ``libkfa.so`` once; raises ``RuntimeError`` if it has not been built."""
    global _library
    if _library is None:
        with _lock:
            if _library is None:
                if not os.path.exists(LIBRARY_PATH):
                    raise RuntimeError(
                        f"{LIBRARY_PATH} is missing: build it with `python kohakufa-cute_b200/build.py` "
                        "(there is no non-CUDA fallback)."
                    )
                lib = ctypes.CDLL(LIBRARY_PATH)
                for name, (restype, argtypes) in SIGNATURES.items():
                    fn = getattr(lib, name)
                    fn.restype = restype
                    fn.argtypes = argtypes
                _library = lib
    return _library


def loaded():
    return _library is not None


def describe(tensor):
    """Non-owning ``kfa_tensor`` record for a torch tensor (None -> NULL pointer)."""
    if tensor is None:
        return None
    record = KfaTensor()
    record.data = tensor.data_ptr()
    record.dtype = _DTYPES[tensor.dtype]
    record.ndim = tensor.dim()
    for axis, (size, stride) in enumerate(zip(tensor.shape, tensor.stride())):
        record.sizes[axis] = size
        record.strides[axis] = stride
    return record


def _ref(record):
    return None if record is None else ctypes.byref(record)


def _check(code):
    if code == 0:
        return
    message = library().kfa_last_error().decode()
    if code == 1:
        raise ValueError(message)
    if code == 3:
        raise DeviceTimeoutError(message)
    raise RuntimeError(f"libkfa error {code}: {message}")


class DeviceTimeoutError(RuntimeError):
    """A bounded device-side wait ran out earlier; acknowledge with ``device_status(reset=True)``."""


def _stream(device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _plain(tensor):
    """Physical storage must equal logical values: resolve lazy conj/neg view flags."""
    return tensor.resolve_conj().resolve_neg()


def _rows_16_byte_addressable(t):
    if t.stride(-1) != 1 or t.data_ptr() % 16:
        return False
    return all(size == 1 or (stride > 0 and stride % 8 == 0) for size, stride in zip(t.shape[:-1], t.stride()[:-1]))


def _blocks_shape(q, k, mask):
    return (
        1 if mask.stride(0) == 0 else q.shape[0],
        1 if mask.stride(1) == 0 else q.shape[1],
        1 if mask.stride(2) == 0 else (q.shape[2] + 63) // 64,
        1 if mask.stride(3) == 0 else (k.shape[2] + 63) // 64,
    )


def tensor_core_head_dim(D):
    """Channels the tensor-memory kernels run a head of ``D`` channels with: multiples of 8 up to 128 as they
    are, other sizes padded with zero channels to the next multiple of 8 (up to 128) or to 256 / 384 / 512."""
    if D <= 128:
        return (D + 7) // 8 * 8
    return 256 if D <= 256 else (384 if D <= 384 else 512)


def _for_tensor_cores(tensors):
    """The operands in a form the tensor-memory kernels address (the reference serves odd head sizes and
    unaligned or channel-strided operands inside its MMA kernels with predicated loads, kernels.py:480-551;
    here the tiled loads want 16-byte rows): zero channels appended up to ``tensor_core_head_dim`` - they add
    nothing to either product, and the matching output channels are dropped again - and dense copies of operands
    whose rows are not 16-byte addressable.  Returns the tensors unchanged when nothing has to be done."""
    D = tensors[0].shape[-1]
    target = tensor_core_head_dim(D)
    if target == D and all(_rows_16_byte_addressable(t) for t in tensors):
        return tensors, D
    if target != D:
        return [torch.nn.functional.pad(t, (0, target - D)) for t in tensors], D
    return [t if _rows_16_byte_addressable(t) else t.contiguous() for t in tensors], D


def _like(original, result):
    """``result`` (possibly with extra channels) copied into a tensor laid out like ``original``, as the
    reference allocates its outputs (native.cpp:295,348)."""
    out = torch.empty_like(original)
    out.copy_(result[..., : original.shape[-1]])
    return out


def forward(q, k, v, mask, scale, causal, statistics=True):
    """(out, maximum, logsum, blocks) - mirrors the reference extension's ``forward`` (native.cpp:1034).
    With ``statistics=False`` (a forward pass nobody will differentiate) the two row statistics are neither
    allocated nor written and come back as ``None``."""
    lib = library()
    q, k, v = _plain(q), _plain(k), _plain(v)
    originals = (q, k, v)
    (q, k, v), _ = _for_tensor_cores([q, k, v])
    if any(a is not b for a, b in zip((q, k, v), originals)):
        out, maximum, logsum, blocks = forward(q, k, v, mask, scale, causal, statistics)
        return _like(originals[0], out), maximum, logsum, blocks
    with torch.cuda.device(q.device):
        out = torch.empty_like(q)
        maximum = torch.empty(q.shape[:-1], device=q.device, dtype=torch.float32) if statistics else None
        logsum = torch.empty_like(maximum) if statistics else None
        if mask is None:
            blocks = torch.empty((1, 1, 1, 1), device=q.device, dtype=torch.int32)
        else:
            blocks = torch.empty(_blocks_shape(q, k, mask), device=q.device, dtype=torch.int32)
        records = [describe(t) for t in (q, k, v, mask, out, maximum, logsum, blocks if mask is not None else None)]
        _check(lib.kfa_forward(*[_ref(r) for r in records], float(scale), int(bool(causal)), _stream(q.device)))
    return out, maximum, logsum, blocks


def decode_served(q, k, v, mask, causal):
    """Whether ``forward_decode`` serves the call: a few query rows per K/V head (positions x grouped heads <= 8)
    against at least 512 keys, 64 or 128 channels, no mask, not causal, 8-byte addressable rows."""
    if mask is not None or causal or q.shape[-1] not in (64, 128) or k.shape[2] < 512:
        return False
    if q.shape[2] * (q.shape[1] // k.shape[1]) > 8:
        return False
    return all(t.stride(-1) == 1 and t.data_ptr() % 8 == 0 and all(s % 4 == 0 for s in t.stride()[:-1]) for t in (q, k, v))


def forward_decode(q, k, v, scale, statistics=True):
    """(out, maximum, logsum, blocks) through ``kfa_forward_decode``: the decoding shapes of ``decode_served``
    on CUDA-core kernels bound by the HBM time of K and V."""
    lib = library()
    q, k, v = _plain(q), _plain(k), _plain(v)
    with torch.cuda.device(q.device):
        out = torch.empty_like(q)
        maximum = torch.empty(q.shape[:-1], device=q.device, dtype=torch.float32) if statistics else None
        logsum = torch.empty_like(maximum) if statistics else None
        rq, rk = describe(q), describe(k)
        need = lib.kfa_forward_decode_workspace_bytes(_ref(rq), _ref(rk))
        workspace = torch.empty(need, device=q.device, dtype=torch.uint8)
        records = [rq, rk, describe(v), describe(out), describe(maximum), describe(logsum)]
        _check(lib.kfa_forward_decode(*[_ref(r) for r in records], ctypes.c_void_p(workspace.data_ptr()), need,
                                      float(scale), _stream(q.device)))
        blocks = torch.empty((1, 1, 1, 1), device=q.device, dtype=torch.int32)
    return out, maximum, logsum, blocks


def split_plan(q, k, causal):
    """Number of key ranges to split a forward call into, or 0.  A short query sequence against a long key
    sequence gives the forward kernel one CTA per (batch, head) and leaves most of the GPU idle; splitting the
    keys over CTAs and merging the partial results fills it (the reference's split forward,
    split_forward.py:125-245, serves the same shapes)."""
    B, Hq, Sq, D = q.shape
    Sk = k.shape[2]
    if causal or Sq > 256 or Sk < 4096 or D > 128 or D % 8:
        return 0
    ctas = B * Hq
    if 2 * ctas > 148:
        return 0
    splits = min(148 // ctas, Sk // 1024, 32)
    return splits if splits >= 2 else 0


def forward_split(q, k, v, mask, scale, splits, statistics=True):
    """Forward pass split over the key axis (non-causal): ``kfa_forward`` on ``splits`` key ranges, folded into
    the batch axis of one launch per batch element (a remainder range gets its own), then ``kfa_merge_splits``.
    The partial outputs are normalised per range and rounded to the 16-bit type before the merge, which rounds
    the result once more.  Returns ``(out, maximum, logsum, blocks)`` like ``forward``; the statistics cover the
    whole key range, so the ordinary backward applies."""
    lib = library()
    q, k, v = _plain(q), _plain(k), _plain(v)
    B, Hq, Sq, D = q.shape
    Hkv, Sk = k.shape[1], k.shape[2]
    chunk = -(-Sk // splits)
    chunk = -(-chunk // 128) * 128
    full, tail = Sk // chunk, Sk % chunk
    parts = full + (1 if tail else 0)
    with torch.cuda.device(q.device):
        stream = _stream(q.device)
        out = torch.empty_like(q)
        maximum = torch.empty(q.shape[:-1], device=q.device, dtype=torch.float32) if statistics else None
        logsum = torch.empty_like(maximum) if statistics else None
        part_out = torch.empty((B, parts, Hq, Sq, D), device=q.device, dtype=q.dtype)
        part_max = torch.empty((B, parts, Hq, Sq), device=q.device, dtype=torch.float32)
        part_log = torch.empty_like(part_max)

        def ranges(t, b, first, count, length):
            """[count, heads, length, D] view of batch element b: range i starts at key first + i * length."""
            return torch.as_strided(t, (count, t.shape[1], length, t.shape[3]),
                                    (length * t.stride(2), t.stride(1), t.stride(2), t.stride(3)),
                                    t.storage_offset() + b * t.stride(0) + first * t.stride(2))

        def masks(b, first, count, length):
            if mask is None:
                return None
            return torch.as_strided(mask, (count, Hq, Sq, length),
                                    (length * mask.stride(3), mask.stride(1), mask.stride(2), mask.stride(3)),
                                    mask.storage_offset() + b * mask.stride(0) + first * mask.stride(3))

        for b in range(B):
            pieces = [(0, full, chunk)] if full else []
            if tail:
                pieces.append((full * chunk, 1, tail))
            done = 0
            for first, count, length in pieces:
                qs = q[b:b + 1].expand(count, Hq, Sq, D).contiguous()
                ks, vs, ms = ranges(k, b, first, count, length), ranges(v, b, first, count, length), masks(b, first, count, length)
                blocks = None if ms is None else torch.empty(_blocks_shape(qs, ks, ms), device=q.device, dtype=torch.int32)
                records = [describe(t) for t in (qs, ks, vs, ms, part_out[b, done:done + count], part_max[b, done:done + count],
                                                 part_log[b, done:done + count], blocks)]
                _check(lib.kfa_forward(*[_ref(r) for r in records], float(scale), 0, stream))
                done += count
            records = [describe(t) for t in (out[b:b + 1], None if maximum is None else maximum[b:b + 1],
                                             None if logsum is None else logsum[b:b + 1], part_out[b].unsqueeze(1),
                                             part_max[b].unsqueeze(1), part_log[b].unsqueeze(1))]
            _check(lib.kfa_merge_splits(*[_ref(r) for r in records], float(scale), stream))
        if mask is None:
            blocks = torch.empty((1, 1, 1, 1), device=q.device, dtype=torch.int32)
        else:
            blocks = pack_mask(q, k, mask) if statistics else torch.empty((1, 1, 1, 1), device=q.device, dtype=torch.int32)
    return out, maximum, logsum, blocks


def pack_mask(q, k, mask):
    """int32 tile table of an expanded [B,Hq,Sq,Sk] boolean mask (see ``kfa_pack_mask``)."""
    lib = library()
    with torch.cuda.device(q.device):
        blocks = torch.empty(_blocks_shape(q, k, mask), device=q.device, dtype=torch.int32)
        rm, rb = describe(mask), describe(blocks)
        _check(lib.kfa_pack_mask(_ref(rm), _ref(rb), _stream(q.device)))
    return blocks


def backward(q, k, v, mask, maximum, logsum, dout, blocks, out, scale, causal):
    """(dq, dk, dv) - mirrors the reference extension's ``backward`` (native.cpp:1038)."""
    lib = library()
    q, k, v, dout, out = _plain(q), _plain(k), _plain(v), _plain(dout), _plain(out)
    originals = (q, k, v)
    (q, k, v, dout, out), _ = _for_tensor_cores([q, k, v, dout, out])
    if any(a is not b for a, b in zip((q, k, v), originals)):
        grads = backward(q, k, v, mask, maximum, logsum, dout, blocks, out, scale, causal)
        return tuple(_like(o, g) for o, g in zip(originals, grads))
    with torch.cuda.device(q.device):
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        rq, rk = describe(q), describe(k)
        need = lib.kfa_backward_workspace_bytes(_ref(rq), _ref(rk))
        workspace = torch.empty(need, device=q.device, dtype=torch.uint8)
        records = [rq, rk, describe(v), describe(mask), describe(out), describe(maximum), describe(logsum),
                   describe(dout), describe(blocks if mask is not None else None), describe(dq), describe(dk),
                   describe(dv)]
        _check(lib.kfa_backward(*[_ref(r) for r in records], ctypes.c_void_p(workspace.data_ptr()), need,
                                float(scale), int(bool(causal)), _stream(q.device)))
    return dq, dk, dv


def center_keys(k):
    """round(f32(k) - mean_S f32(k)) in k's dtype (also the gradient projection of that map)."""
    lib = library()
    k = _plain(k)
    with torch.cuda.device(k.device):
        out = torch.empty_like(k)
        rk = describe(k)
        need = lib.kfa_center_keys_workspace_bytes(_ref(rk))
        workspace = torch.empty(need, device=k.device, dtype=torch.uint8)
        ro = describe(out)
        _check(lib.kfa_center_keys(_ref(rk), _ref(ro), ctypes.c_void_p(workspace.data_ptr()), need,
                                   _stream(k.device)))
    return out


def center_keys_static(k, out=None):
    """Key centring through the entry point that allocates nothing: the scratch is a fixed array
    inside the library (see ``kfa_center_keys_static``).  ``out`` is the caller's output tensor;
    when omitted one is created here, which is a convenience of this binding, not of the C call.
    Raises ``RuntimeError`` when batch*heads*channels exceeds ``kfa_center_keys_static_limit()``.
    """
    lib = library()
    k = _plain(k)
    with torch.cuda.device(k.device):
        if out is None:
            out = torch.empty_like(k)
        rk, ro = describe(k), describe(out)
        _check(lib.kfa_center_keys_static(_ref(rk), _ref(ro), _stream(k.device)))
    return out


def _int64_array(values):
    return (ctypes.c_int64 * len(values))(*[int(x) for x in values])


def neighborhood_forward(q, k, v, spatial, window, scale):
    """(out, maximum, logsum) - mirrors ``neighborhood_forward`` (native.cpp:1043)."""
    lib = library()
    q, k, v = _plain(q), _plain(k), _plain(v)
    with torch.cuda.device(q.device):
        out = torch.empty_like(q)
        maximum = torch.empty(q.shape[:-1], device=q.device, dtype=torch.float32)
        logsum = torch.empty_like(maximum)
        records = [describe(t) for t in (q, k, v, out, maximum, logsum)]
        _check(lib.kfa_neighborhood_forward(*[_ref(r) for r in records], _int64_array(spatial), len(spatial),
                                            _int64_array(window), float(scale), _stream(q.device)))
    return out, maximum, logsum


def neighborhood_backward(q, k, v, out, maximum, logsum, dout, spatial, window, scale):
    lib = library()
    q, k, v, out, dout = (_plain(t) for t in (q, k, v, out, dout))
    with torch.cuda.device(q.device):
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        rq = describe(q)
        need = lib.kfa_neighborhood_backward_workspace_bytes(_ref(rq))
        workspace = torch.empty(need, device=q.device, dtype=torch.uint8)
        records = [rq] + [describe(t) for t in (k, v, out, maximum, logsum, dout, dq, dk, dv)]
        _check(lib.kfa_neighborhood_backward(*[_ref(r) for r in records], ctypes.c_void_p(workspace.data_ptr()), need,
                                             _int64_array(spatial), len(spatial), _int64_array(window), float(scale),
                                             _stream(q.device)))
    return dq, dk, dv


def running_state(q):
    """Fresh running state ``(acc, run_maximum, run_sum)`` for ``forward_running`` on queries ``q``."""
    acc = torch.zeros(q.shape, device=q.device, dtype=torch.float32)
    run_maximum = torch.full(q.shape[:-1], float("-inf"), device=q.device, dtype=torch.float32)
    run_sum = torch.zeros(q.shape[:-1], device=q.device, dtype=torch.float32)
    return acc, run_maximum, run_sum


def forward_running(q, k, v, mask, state, scale, causal=False):
    """Attends ``q`` to one key/value block and folds the result into ``state`` in place
    (``kfa_forward_running``: unnormalised FP32 accumulator, running maximum and sum; nothing is rounded
    to the 16-bit type between blocks)."""
    lib = library()
    q, k, v = _plain(q), _plain(k), _plain(v)
    acc, run_maximum, run_sum = state
    with torch.cuda.device(q.device):
        blocks = None if mask is None else torch.empty(_blocks_shape(q, k, mask), device=q.device, dtype=torch.int32)
        records = [describe(t) for t in (q, k, v, mask, acc, run_maximum, run_sum, blocks)]
        _check(lib.kfa_forward_running(*[_ref(r) for r in records], float(scale), int(bool(causal)),
                                       _stream(q.device)))


def finish_running(state, dtype):
    """``(out, maximum, logsum)`` of a running state: one division and one rounding per element, and the
    statistics the backward expects.  The statistics reuse the state's own tensors."""
    lib = library()
    acc, run_maximum, run_sum = state
    with torch.cuda.device(acc.device):
        out = torch.empty(acc.shape, device=acc.device, dtype=dtype)
        records = [describe(t) for t in (acc, run_maximum, run_sum, out, run_maximum, run_sum)]
        _check(lib.kfa_finish_running(*[_ref(r) for r in records], _stream(acc.device)))
    return out, run_maximum, run_sum


def backward_partial(q, k, v, mask, maximum, logsum, dout, out, scale, causal, dq, dk, dv,
                     accumulate_dq=True, accumulate_dkv=False):
    """Gradient contributions of one (query block, key block) pair against the statistics of the whole
    sequence, in FP32 (``kfa_backward_partial``): ``dq`` / ``dk`` / ``dv`` are float32 tensors (views allowed,
    unit channel stride) that are overwritten or added to."""
    lib = library()
    q, k, v, dout, out = _plain(q), _plain(k), _plain(v), _plain(dout), _plain(out)
    if not _rows_16_byte_addressable(dout):
        dout = dout.contiguous()
    with torch.cuda.device(q.device):
        rq, rk = describe(q), describe(k)
        need = lib.kfa_backward_workspace_bytes(_ref(rq), _ref(rk))
        workspace = torch.empty(need, device=q.device, dtype=torch.uint8)
        blocks = None if mask is None else pack_mask(q, k, mask)
        records = [rq, rk, describe(v), describe(mask), describe(out), describe(maximum), describe(logsum),
                   describe(dout), describe(blocks), describe(dq), describe(dk), describe(dv)]
        _check(lib.kfa_backward_partial(*[_ref(r) for r in records], ctypes.c_void_p(workspace.data_ptr()), need,
                                        float(scale), int(bool(causal)), int(bool(accumulate_dq)),
                                        int(bool(accumulate_dkv)), _stream(q.device)))


def merge_partial(acc_out, acc_maximum, acc_logsum, part_out, part_maximum, part_logsum, scale):
    """In-place (max, sum) merge of one partial attention result into the running FP32 result."""
    lib = library()
    with torch.cuda.device(acc_out.device):
        records = [describe(t) for t in (acc_out, acc_maximum, acc_logsum, part_out, part_maximum, part_logsum)]
        _check(lib.kfa_merge_partial(*[_ref(r) for r in records], float(scale), _stream(acc_out.device)))


def self_test_wait(limit_cycles, ctas, device=None):
    """Runs the failure-detection self-test (``kfa_self_test_wait``); returns the number of CTAs that
    skipped their wait because an earlier one had already given up."""
    lib = library()
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    skipped = ctypes.c_int(0)
    with torch.cuda.device(device):
        _check(lib.kfa_self_test_wait(int(limit_cycles), int(ctas), ctypes.byref(skipped), _stream(device)))
    return skipped.value


def selected_family(q, k, v, mask=None, causal=False, backward=False):
    """0 = general kernels, 1 = tcgen05 tensor-memory pipeline."""
    lib = library()
    with torch.cuda.device(q.device):
        records = [describe(t) for t in (q, k, v, mask)]
        return lib.kfa_selected_family(*[_ref(r) for r in records], int(bool(causal)), int(bool(backward)))


def cache_size():
    return library().kfa_cache_size()


def clear_cache():
    library().kfa_clear_cache()


def launch_count():
    return int(library().kfa_launch_count())


def launch_stats():
    """{kernel family name: launches since load} (``kfa_launch_stats``)."""
    lib = library()
    result, index = {}, 0
    while True:
        name, launches = ctypes.create_string_buffer(64), ctypes.c_uint64()
        if lib.kfa_launch_stats(index, name, 64, ctypes.byref(launches)) != 0:
            return result
        result[name.value.decode()] = int(launches.value)
        index += 1


def init(device=None):
    """Per-device set-up (``kfa_init``); needed explicitly only when the first call on a device would
    otherwise happen inside a CUDA-graph capture."""
    with torch.cuda.device(torch.cuda.current_device() if device is None else device):
        _check(library().kfa_init())


def device_status(reset=False):
    return library().kfa_device_status(int(reset))


def profile_enable(on=True):
    """Bracket every kernel launch with CUDA events (benchmarks only; not during graph capture)."""
    library().kfa_profile_enable(int(bool(on)))


def profile_read(reset=True):
    """{kernel name: (total milliseconds, launches)} accumulated since the last reset."""
    lib = library()
    count = lib.kfa_profile_collect()
    result = {}
    for index in range(count):
        name = ctypes.create_string_buffer(64)
        total, launches = ctypes.c_double(), ctypes.c_uint64()
        _check(lib.kfa_profile_entry(index, name, 64, ctypes.byref(total), ctypes.byref(launches)))
        result[name.value.decode()] = (total.value, launches.value)
    if reset:
        lib.kfa_profile_reset()
    return result
