"""Builds libkfa.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python kohakufa-cute_b200/build.py [--force] [--phases]

The shared library is written next to the Python package as ``kohakufa_cute/libkfa.so``.
``--phases`` builds a second library, ``kohakufa_cute/libkfa_phases.so``, whose pipeline kernels record
how many cycles each role of one CTA spends in each phase of its loop (see ``csrc/phase_clock.cuh``;
``phase_profile.py`` runs it and prints the table).  The ordinary library carries none of that code.
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
SOURCES = ["kfa_api.cu", "general_kernels.cu", "neighborhood_kernels.cu", "pipeline_forward.cu", "decode_forward.cu",
           "pipeline_backward.cu", "wide_head.cu", "na_pipeline.cu", "tensor_map.cu", "static_scratch.cu", "wait_probe.cu", "center_keys_cluster.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "-Wno-deprecated-gpu-targets"]


def _nvcc():
    return os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc" if os.path.exists("/usr/local/cuda/bin/nvcc") else "nvcc")


def _digest(paths, flags):
    h = hashlib.sha256()
    for path in sorted(paths):
        with open(path, "rb") as f:
            h.update(f.read())
    h.update(" ".join(flags).encode())
    return h.hexdigest()


def sources():
    return [s for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def build(force=False, verbose=True, phases=False):
    flags = NVCC_FLAGS + (["-DKFA_PHASES=1"] if phases else [])
    obj_dir = OBJ_DIR + ("_phases" if phases else "")
    lib = LIB.replace("libkfa.so", "libkfa_phases.so") if phases else LIB
    os.makedirs(obj_dir, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh", ".inl"))]
    headers.append(os.path.join(os.path.dirname(HERE), "include", "kfa.h"))
    objects, jobs = [], []
    for src in sources():
        path = os.path.join(CSRC, src)
        obj = os.path.join(obj_dir, src.replace(".cu", ".o"))
        stamp = obj + ".sha"
        digest = _digest([path] + headers, flags)
        objects.append(obj)
        fresh = os.path.exists(obj) and os.path.exists(stamp) and open(stamp).read() == digest
        if force or not fresh:
            jobs.append((path, obj, stamp, digest))

    def compile_one(job):
        path, obj, stamp, digest = job
        cmd = [_nvcc(), *flags, "-c", path, "-o", obj]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.check_call(cmd)
        with open(stamp, "w") as f:
            f.write(digest)

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        list(pool.map(compile_one, jobs))
    if jobs or force or not os.path.exists(lib):
        cmd = [_nvcc(), "-shared", "-o", lib, *objects, "-lcudart_static", "-ldl", "-lpthread", "-lrt",
               "-Wno-deprecated-gpu-targets"]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.check_call(cmd)
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, phases="--phases" in sys.argv))
