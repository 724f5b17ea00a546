"""Closed-form window geometry: the host mirror (``kohakufa_cute.neighborhood_geometry``) against brute force
and the golden window tables, and the device functions (``na_start`` / ``na_inverse`` in ``kfa_common.cuh``,
compiled for the host) against the mirror."""

import itertools
import os
import shutil
import subprocess

import pytest
import torch

from kohakufa_cute import neighborhood_geometry as geometry
from tests.golden_io import load

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CASES = [(e, w) for e in range(1, 25) for w in range(1, e + 1)]


def _members(key, extent, window):
    return [p for p in range(extent) if geometry.window_start(p, extent, window) <= key < geometry.window_start(p, extent, window) + window]


def test_inverse_range_is_the_set_of_queries_that_see_a_key():
    for extent, window in CASES:
        for key in range(extent):
            lo, hi = geometry.inverse_range(key, extent, window)
            assert _members(key, extent, window) == list(range(lo, hi + 1)), (extent, window, key)


def test_window_start_reproduces_the_golden_tables():
    c = load("neighborhood_geometry")
    for index in range(c["count"]):
        spatial = tuple(int(x) for x in c[f"spatial{index}"])
        window = tuple(int(x) for x in c[f"window{index}"])
        pitch = [int(torch.tensor(spatial[a + 1:]).prod()) if a + 1 < len(spatial) else 1 for a in range(len(spatial))]
        table = c[f"table{index}"].tolist()
        for row, coords in enumerate(itertools.product(*(range(e) for e in spatial))):
            first = [geometry.window_start(p, e, w) for p, e, w in zip(coords, spatial, window)]
            keys = [sum((f + o) * s for f, o, s in zip(first, offs, pitch))
                    for offs in itertools.product(*(range(w) for w in window))]
            assert keys == table[row]


@pytest.mark.skipif(shutil.which("nvcc") is None and not os.path.exists("/usr/local/cuda/bin/nvcc"), reason="needs nvcc")
def test_device_functions_agree_with_the_host_mirror(tmp_path):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    source = tmp_path / "probe.cu"
    source.write_text('''
#include <cstdio>
#include "kfa_common.cuh"
int main() {
    for (int e = 1; e < 25; ++e)
        for (int w = 1; w <= e; ++w)
            for (int c = 0; c < e; ++c) {
                int lo, hi;
                kfa::na_inverse(c, e, w, lo, hi);
                std::printf("%d %d %d %d %d %d\\n", e, w, c, kfa::na_start(c, e, w), lo, hi);
            }
    return 0;
}
''')
    binary = tmp_path / "probe"
    subprocess.check_call([nvcc, "-std=c++17", "-I", os.path.join(ROOT, "kohakufa-cute_b200", "csrc"), "-o", str(binary),
                           str(source), "-Wno-deprecated-gpu-targets"])
    lines = subprocess.check_output([str(binary)], text=True).split("\n")
    seen = 0
    for line in lines:
        if not line:
            continue
        e, w, c, start, lo, hi = (int(x) for x in line.split())
        assert start == geometry.window_start(c, e, w)
        assert (lo, hi) == geometry.inverse_range(c, e, w)
        seen += 1
    assert seen == sum(e for e, _ in CASES)
