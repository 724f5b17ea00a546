"""The window masks of the neighbourhood kernels, checked on the host.

``csrc/na_tiles.cuh`` holds the geometry as ``__host__ __device__`` functions; ``host_checks/na_mask_walk_check.cu``
compiles them into a host program (nvcc, no GPU needed) that compares the cursor-based masks the kernels use
(``box_mask_walk``) with the direct ones (``box_mask``) and with the definition, over query boxes and key boxes of
ten grids, 64- and 128-token tiles, walks over all tiles and over subsets.
"""

import os
import shutil
import subprocess

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


@pytest.mark.skipif(shutil.which("nvcc") is None, reason="needs nvcc to build the host program")
def test_mask_walk_matches_direct_masks_and_definition(tmp_path):
    exe = str(tmp_path / "na_mask_walk_check")
    build = subprocess.run(
        ["nvcc", "-std=c++17", "-O2", "-gencode", "arch=compute_100a,code=sm_100a", "-I", os.path.join(ROOT, "kohakufa-cute_b200", "csrc"),
         "-o", exe, os.path.join(HERE, "host_checks", "na_mask_walk_check.cu")],
        capture_output=True, text=True, timeout=600)
    assert build.returncode == 0, build.stderr[-2000:]
    run = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stdout[-2000:]
    assert run.stdout.startswith("ok "), run.stdout[-500:]
    assert int(run.stdout.split()[1]) > 1_000_000
