"""Builds libkfa.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python kohakufa-cute_b200/build.py [--force]

The shared library is written next to the Python package as ``kohakufa_cute/libkfa.so``.
"""

import hashlib
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT_DIR = os.path.join(HERE, "kohakufa_cute")
OBJ_DIR = os.path.join(HERE, "build")
LIB = os.path.join(OUT_DIR, "libkfa.so")
SOURCES = ["kfa_api.cu", "general_kernels.cu", "neighborhood_kernels.cu", "pipeline_forward.cu",
           "pipeline_backward.cu", "wide_head.cu", "na_pipeline.cu", "tensor_map.cu", "static_scratch.cu", "wait_probe.cu", "center_keys_cluster.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "-Wno-deprecated-gpu-targets"]


if os.environ.get("KFA_TRACE"):  # tuning aid: cycle stamps from the CTA with this index
    NVCC_FLAGS = NVCC_FLAGS + ["-DKFA_TRACE=" + os.environ["KFA_TRACE"]]


if os.environ.get("KFA_DEFINES"):  # tuning aid: extra -D switches, space separated
    NVCC_FLAGS = NVCC_FLAGS + ["-D" + d for d in os.environ["KFA_DEFINES"].split()]


def _nvcc():
    return os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc" if os.path.exists("/usr/local/cuda/bin/nvcc") else "nvcc")


def _digest(paths):
    h = hashlib.sha256()
    for path in sorted(paths):
        with open(path, "rb") as f:
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def sources():
    return [s for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def build(force=False, verbose=True):
    os.makedirs(OBJ_DIR, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh", ".inl"))]
    headers.append(os.path.join(os.path.dirname(HERE), "include", "kfa.h"))
    objects, jobs = [], []
    for src in sources():
        path = os.path.join(CSRC, src)
        obj = os.path.join(OBJ_DIR, src.replace(".cu", ".o"))
        stamp = obj + ".sha"
        digest = _digest([path] + headers)
        objects.append(obj)
        fresh = os.path.exists(obj) and os.path.exists(stamp) and open(stamp).read() == digest
        if force or not fresh:
            jobs.append((path, obj, stamp, digest))

    def compile_one(job):
        path, obj, stamp, digest = job
        cmd = [_nvcc(), *NVCC_FLAGS, "-c", path, "-o", obj]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.check_call(cmd)
        with open(stamp, "w") as f:
            f.write(digest)

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        list(pool.map(compile_one, jobs))
    if jobs or force or not os.path.exists(LIB):
        cmd = [_nvcc(), "-shared", "-o", LIB, *objects, "-lcudart_static", "-ldl", "-lpthread", "-lrt",
               "-Wno-deprecated-gpu-targets"]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
