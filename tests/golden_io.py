"""Reads the compressed golden vectors written by tests/golden/make_golden.py."""

import os

import numpy as np
import torch

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load(name):
    """Returns a dict of torch tensors / python scalars for ``tests/golden/<name>.npz``."""
    record = {}
    with np.load(os.path.join(GOLDEN_DIR, name + ".npz")) as data:
        for key in data.files:
            value = data[key]
            if key.endswith("::bf16"):
                record[key[:-6]] = torch.from_numpy(value.copy()).view(torch.bfloat16)
            elif key.endswith("::fp16"):
                record[key[:-6]] = torch.from_numpy(value.copy()).view(torch.float16)
            elif value.ndim == 0:
                record[key] = value.item()
            else:
                record[key] = torch.from_numpy(value.copy())
    return record


def attention_case(index):
    record = load(f"attention_case{index}")
    scale = record["scale"]
    record["scale"] = None if scale != scale else float(scale)
    record["mask"] = record.get("mask") if record["has_mask"] else None
    record["causal"] = bool(record["causal"])
    return record


ATTENTION_CASES = range(8)
NEIGHBORHOOD_CASES = range(4)
