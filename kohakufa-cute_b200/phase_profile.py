"""Where the cycles of one CTA of the pipeline kernels go: per role, per phase of its loop.

    python kohakufa-cute_b200/build.py --phases        # builds kohakufa_cute/libkfa_phases.so
    python kohakufa-cute_b200/phase_profile.py [--workload llm_gqa] [--cta 0] [--steps 3]

Runs forward+backward steps of a benchmark workload through the instrumented library (``csrc/phase_clock.cuh``)
and prints, for the chosen CTA index of each kernel, the cycles every instrumented role spent in each phase.
The instrumentation costs a few percent; the figures tell which role waits for which, not absolute speed.

Phases (index = position in the printed list):
  forward, softmax warpgroup of a query tile : 0 wait for the score tile, 1 tensor-memory load, 2 mask + row maximum
                                               + re-base, 3 exponentials and packing, 4 store fence + hand-over, 5 loop
  forward, MMA issuer                        : 0 wait for V, 1 wait for P, 2 issue P.V, 3 wait for K, 4 issue Q.K^T, 5 loop
  backward, consumer warpgroups              : 0 wait for the score tile, 1 tensor-memory loads, 2 P arithmetic,
                                               3 stores + hand-over, 4 set-up of the unit, 5 loop, 6 wait for dP, 7 dS arithmetic
  neighbourhood forward, softmax warps       : 0 wait for the score tile (and the last product), 1 first pass (hide,
                                               maximum), 2 re-base, 3 second pass (weights), 4 hand-over, 5 window
                                               mask of the next tile, 6 start-up (barriers, window boxes, tile
                                               bitmap), 7 epilogue
  backward, MMA issuers                      : 0 wait for the consumers, 1 issue gradient products, 2 wait for operands,
                                               3 issue score products, 4 loop, 5 further waits
"""

import argparse
import ctypes
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
sys.path.insert(0, HERE)
sys.path.insert(0, ROOT)

SLOTS = {
    "kfa_debug_phases_fwd": {0: "forward  softmax tile 0", 1: "forward  softmax tile 1", 2: "forward  MMA issuer"},
    "kfa_debug_phases_bwd": {0: "dQ       consumers wg 0", 1: "dQ       consumers wg 1", 2: "dQ       MMA issuer S",
                             3: "dQ       MMA issuer dP/dQ", 8: "dK/dV    consumers wg 0", 9: "dK/dV    consumers wg 1",
                             10: "dK/dV    MMA issuer"},
    "kfa_debug_phases_na": {0: "neighbourhood forward softmax"},
}


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--workload", default="llm_gqa")
    parser.add_argument("--cta", type=int, default=0, help="index of the CTA (block) to report, per kernel")
    parser.add_argument("--steps", type=int, default=3)
    args = parser.parse_args()
    from kohakufa_cute import native

    native.LIBRARY_PATH = os.path.join(HERE, "kohakufa_cute", "libkfa_phases.so")
    if not os.path.exists(native.LIBRARY_PATH):
        raise SystemExit("build the instrumented library first: python kohakufa-cute_b200/build.py --phases")
    import bench

    lib = native.library()
    w = dict(bench.WORKLOADS[args.workload], name=args.workload)
    (hq, hk, hv, hg), hmask = bench.make_host_inputs(w, 0, 1)
    q, k, v, g = (t.cuda().requires_grad_(i < 3) for i, t in enumerate((hq, hk, hv, hg)))
    mask = None if hmask is None else hmask.cuda()
    step = bench.build_step(w)
    table = (ctypes.c_uint * 256)()
    for name in SLOTS:
        getattr(lib, name)(None, args.cta)
    for _ in range(args.steps):
        step(q, k, v, g, mask)
    torch.cuda.synchronize()
    print(f"workload {args.workload}, CTA {args.cta}: cycles per phase (last step)")
    for name, slots in SLOTS.items():
        getattr(lib, name)(table, args.cta)
        for slot, label in slots.items():
            values = [table[slot * 8 + i] for i in range(8)]
            if sum(values):
                print(f"  {label:26s} {values}  total {sum(values)}")


if __name__ == "__main__":
    main()
