"""Generates the golden vectors under tests/golden/ by importing the reference project.

Run once, in a container where the reference checkout is mounted:

    python tests/golden/make_golden.py /path/to/reference

It imports only the reference's pure-PyTorch CPU oracles (``benchmarks/reference.py``,
``benchmarks/neighborhood/*reference*.py``, ``kohakufa_cute.api._center_keys``) and a few
fixture builders from its test-suite, evaluates them on small seeded inputs and stores the
inputs together with the reference's answers as compressed ``.npz`` files.  The parity tests
read only the ``.npz`` files, never the reference checkout.
"""

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def pack(tensors):
    """torch tensors -> dict of numpy arrays (16-bit floats stored as raw int16 + a dtype tag)."""
    out = {}
    for name, t in tensors.items():
        if isinstance(t, (int, float, bool)):
            out[name] = np.asarray(t)
            continue
        t = t.detach().cpu().contiguous()
        if t.dtype == torch.bfloat16:
            out[name + "::bf16"] = t.view(torch.int16).numpy()
        elif t.dtype == torch.float16:
            out[name + "::fp16"] = t.view(torch.int16).numpy()
        else:
            out[name] = t.numpy()
    return out


def save(name, tensors):
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **pack(tensors))
    print(f"{name}.npz: {os.path.getsize(path) / 1024:.1f} KiB")


def main(reference_root):
    sys.path.insert(0, reference_root)
    sys.path.insert(0, os.path.join(reference_root, "src"))
    from benchmarks.reference import fp64_reference, rounded_reference, metrics
    from benchmarks.neighborhood.reference import neighborhoods, two_term_forward_reference
    from benchmarks.neighborhood.key_precision_reference import key_precision_reference
    from benchmarks.neighborhood.precision_reference import mathematical_reference
    from kohakufa_cute.api import _center_keys
    from tests.test_key_precision import key_cancellation, key_coordinate
    from tests.test_value_precision import square_value_cancellation, value_residual_underflow

    # ---- ordinary attention: random small cases -------------------------------------------
    cases = [
        # B, Hq, Hkv, Sq, Sk, D, dtype, causal, masked, scale
        (2, 4, 2, 5, 7, 8, torch.bfloat16, False, True, None),
        (2, 4, 2, 5, 7, 8, torch.bfloat16, True, True, 0.3),
        (1, 4, 1, 33, 49, 32, torch.float16, True, False, -0.125),
        (1, 2, 2, 70, 70, 16, torch.bfloat16, True, False, None),
        (2, 2, 1, 40, 24, 32, torch.float16, False, False, 0.0),
        (1, 4, 2, 1, 150, 32, torch.bfloat16, False, False, None),
        (1, 2, 2, 65, 1, 32, torch.bfloat16, True, False, None),
        (1, 1, 1, 66, 70, 128, torch.bfloat16, False, True, None),
    ]
    for index, (B, Hq, Hkv, Sq, Sk, D, dtype, causal, masked, scale) in enumerate(cases):
        gen = torch.Generator().manual_seed(1000 + index)
        q = torch.randn(B, Hq, Sq, D, generator=gen).to(dtype)
        k = torch.randn(B, Hkv, Sk, D, generator=gen).to(dtype)
        v = torch.randn(B, Hkv, Sk, D, generator=gen).to(dtype)
        dout = torch.randn(B, Hq, Sq, D, generator=gen).to(dtype)
        mask = None
        if masked:
            mask = torch.rand(1, 1, Sq, Sk, generator=gen) > 0.3
            mask[..., 0, :] = False  # an all-hidden row
        exact = fp64_reference((q, k, v), dout, mask, causal, scale)
        rounded = rounded_reference((q, k, v), dout, mask, causal, scale)
        given = (rounded[0] * 1.001).to(dtype)  # a forward output that differs slightly from the ideal one
        conditioned = rounded_reference((q, k, v), dout, mask, causal, scale, output=given)
        record = dict(q=q, k=k, v=v, dout=dout, causal=causal, has_mask=masked,
                      scale=float("nan") if scale is None else scale, given=given)
        if masked:
            record["mask"] = mask
        for tag, result in (("exact", exact), ("rounded", rounded), ("conditioned", conditioned)):
            for name, value in zip(("out", "dq", "dk", "dv"), result):
                record[f"{tag}_{name}"] = value
        save(f"attention_case{index}", record)

    # ---- directed fixtures -----------------------------------------------------------------
    q = torch.tensor([[[[10.0]]]], dtype=torch.bfloat16)
    k = torch.tensor([[[[10.0], [5.0]]]], dtype=torch.bfloat16)
    v = torch.tensor([[[[1.0], [-1.0]]]], dtype=torch.bfloat16)
    dout = torch.ones_like(q)
    exact = fp64_reference((q.double(), k.double(), v.double()), dout.double(), scale=1.0)
    rounded = rounded_reference((q, k, v), dout, scale=1)
    record = dict(q=q, k=k, v=v, dout=dout)
    for tag, result in (("exact", exact), ("rounded", rounded)):
        for name, value in zip(("out", "dq", "dk", "dv"), result):
            record[f"{tag}_{name}"] = value
    save("saturated_pair", record)

    for dimension in (16, 128):
        (q, k, v), dout = key_cancellation(dimension, torch.bfloat16, "cpu", heads=1)
        exact = fp64_reference((q, k, v), dout)
        rounded = rounded_reference((q, k, v), dout)
        save(f"key_cancellation_d{dimension}", dict(
            q=q, k=k, v=v, dout=dout, closed_form=key_coordinate(dimension),
            exact_dk_row0=exact[2][0, 0, 0], rounded_dk_row0=rounded[2][0, 0, 0],
            exact_dq_head=exact[1][0, 0, :8], rounded_dq_head=rounded[1][0, 0, :8],
            rounded_dv_row0=rounded[3][0, 0, 0], exact_dv_row0=exact[3][0, 0, 0]))

    (q, k, v), dout, scale, target = square_value_cancellation(16, torch.bfloat16, "cpu", length=128, heads=1)
    exact = fp64_reference((q, k, v), dout, scale=scale)
    rounded = rounded_reference((q, k, v), dout, scale=scale)
    save("value_cancellation_d16", dict(q=q, k=k, v=v, dout=dout, scale=scale, target=target,
                                        exact_dv=exact[3], rounded_dv=rounded[3], rounded_out=rounded[0],
                                        rounded_dq=rounded[1], rounded_dk=rounded[2]))
    (q, k, v), dout, scale, target = value_residual_underflow(64, "cpu", length=128, heads=1)
    exact = fp64_reference((q, k, v), dout, scale=scale)
    rounded = rounded_reference((q, k, v), dout, scale=scale)
    save("value_underflow_fp16_d64", dict(q=q, k=k, v=v, dout=dout, scale=scale, target=target,
                                          exact_dv_row0=exact[3][0, 0, 0], rounded_dv_row0=rounded[3][0, 0, 0]))

    # ---- key centering ---------------------------------------------------------------------
    gen = torch.Generator().manual_seed(77)
    for dtype, tag in ((torch.bfloat16, "bf16"), (torch.float16, "fp16")):
        keys = (torch.randn(2, 3, 37, 16, generator=gen) + 32).to(dtype)
        grad = torch.randn(2, 3, 37, 16, generator=gen).to(dtype)
        leaf = keys.clone().requires_grad_(True)
        centered = _center_keys(leaf)
        (back,) = torch.autograd.grad(centered, leaf, grad)
        save(f"center_keys_{tag}", dict(k=keys, centered=centered, grad=grad, back=back))

    # ---- neighbourhood geometry + arithmetic ----------------------------------------------
    geometry = [((6, 7), (3, 4)), ((5, 5), (5, 5)), ((1, 5), (1, 3)), ((3, 5, 6), (3, 3, 4)),
                ((2, 4, 9), (2, 3, 7)), ((4, 4, 4), (1, 2, 3))]
    record = {}
    for index, (spatial, window) in enumerate(geometry):
        record[f"spatial{index}"] = torch.tensor(spatial)
        record[f"window{index}"] = torch.tensor(window)
        record[f"table{index}"] = torch.tensor(neighborhoods(spatial, window), dtype=torch.int32)
    record["count"] = len(geometry)
    save("neighborhood_geometry", record)

    arithmetic = [((6, 7), (3, 4), torch.bfloat16, 0.125), ((3, 5, 6), (3, 3, 4), torch.float16, 0.125),
                  ((2, 4, 9), (2, 3, 7), torch.bfloat16, -0.125), ((3, 4, 5), (3, 3, 3), torch.float16, 0.0)]
    for index, (spatial, window, dtype, scale) in enumerate(arithmetic):
        gen = torch.Generator().manual_seed(2000 + index)
        tokens = int(np.prod(spatial))
        q, k, v, dout = (torch.randn(1, 1, tokens, 64, generator=gen).to(dtype) for _ in range(4))
        exact = mathematical_reference((q, k, v), dout, spatial, window, scale)
        given = exact[0].to(dtype)
        policy = key_precision_reference((q, k, v), dout, spatial, window, scale, given,
                                         method="weighted_dq_reconstructed_dk")
        two_term = two_term_forward_reference((q, k, v), spatial, window, scale)
        record = dict(q=q, k=k, v=v, dout=dout, given=given, scale=scale, spatial=torch.tensor(spatial),
                      window=torch.tensor(window), two_term=two_term)
        for tag, result in (("exact", exact), ("policy", policy)):
            for name, value in zip(("out", "dq", "dk", "dv"), result):
                record[f"{tag}_{name}"] = value
        save(f"neighborhood_case{index}", record)

    # ---- metric definition ------------------------------------------------------------------
    gen = torch.Generator().manual_seed(5)
    a = torch.randn(64, generator=gen, dtype=torch.float64) * 1e-200
    b = a * 1.01
    save("metric", dict(a=a, b=b, relative_error=metrics(b, a)["relative_error"]))


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("KFA_REFERENCE_CHECKOUT", "reference"))
