"""Where a step's time goes: per-phase cycle counters of the forward and backward kernels.

Needs a profiling build of the library (the counters are compiled out of the normal one):

    CS2D_OUT=$PWD/libcs2d_timers.so official-cross-scan_b200/csrc/build.sh -DCS2D_PHASE_TIMERS
    CS2D_LIB=$PWD/libcs2d_timers.so python -m cs2d.phase_timers [--config NAME] [--batch B]

Prints, for warp 0 of every CTA summed over the launches, the share of each phase in the wall
time of a step.  ``CS2D_BWD_WS=0`` / ``CS2D_FWD_WS=0`` select the kernels in which all warps stage
and compute in turn instead of the warp-specialised ones.
"""
from __future__ import annotations

import argparse
import ctypes

import torch

from . import _lib, ops
from .synthetic import CONFIGS, make_inputs

PHASES = ("prefetch", "bulk-copy wait", "write-out", "staging", "dB/dC flush + B/C staging", "wait for tiles",
          "recompute of h", "sweep")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="c2_vmamba_t_stage1")
    ap.add_argument("--batch", type=int, default=0)
    ap.add_argument("--iters", type=int, default=3)
    args = ap.parse_args()
    b, K, D, N, H, W, dt = CONFIGS[args.config]
    b = args.batch or b
    inp = make_inputs(b, K, D, N, H, W, dtype=dt, seed=0)
    d = {k: (v.cuda() if v is not None else None) for k, v in inp.items()}
    L = _lib.lib()
    buf = (ctypes.c_ulonglong * 16)()

    def step():
        o = ops.fwd(d["u"], d["delta"], d["A"], d["B"], d["C"], d["D"], d["delta_bias"], True, False, None)
        ops.bwd(d["u"], d["delta"], d["A"], d["B"], d["C"], d["D"], d["delta_bias"], d["dout"], o[1], o[2], True, None,
                o[3])

    step()
    torch.cuda.synchronize()
    if L.cs2d_phase_cycles(buf) != 0:
        raise SystemExit(f"cs2d: {_lib.last_error()}")
    for _ in range(args.iters):
        step()
    torch.cuda.synchronize()
    L.cs2d_phase_cycles(buf)
    print(f"{args.config} batch {b}: share of a step's wall time per phase (warp 0 of every CTA, {args.iters} runs)")
    for name, base in (("forward", 0), ("backward", 8)):
        v = [buf[base + k] for k in range(8)]
        tot = sum(v) or 1
        print(f"  {name:8s} " + "  ".join(f"{p} {x / tot * 100:.1f}%" for p, x in zip(PHASES, v) if x))


if __name__ == "__main__":
    main()
