"""TEST INFRASTRUCTURE.  Times the REFERENCE CUDA extension beside this library on every benchmark shape.

Runs ``selective_nd_scan_cuda_oflex`` built from the reference's own sources
(``make -C oracle ref`` -> ``oracle/_ref/``) and ``cs2d`` on the same seeded
inputs on one GPU, forward and backward timed separately with CUDA events, and
compares the two sets of results.  The state dimension is clamped to 12 for
both: the reference's backward kernel places its dA staging array 16 bytes past
the shared memory it requests when dstate > 12
(selective_scan_bwd_kernel_oflex.cuh:119 and :909), so it must not be run
there; this library is timed at the full dstate as well.

    python oracle/time_reference_gpu.py [--out FILE] [--iters 5] [--max-batch 32]

Prints one markdown table row per configuration.
"""
import argparse
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "official-cross-scan_b200"))
import cs2d  # noqa: E402
from cs2d.synthetic import CONFIGS, make_inputs  # noqa: E402

REF_MAX_DSTATE = 12


def _time(mod, dev, iters):
    f = lambda: mod.fwd(dev["u"], dev["delta"], dev["A"], dev["B"], dev["C"], dev["D"], dev["delta_bias"], True, False,
                        None)
    g = lambda o: mod.bwd(dev["u"], dev["delta"], dev["A"], dev["B"], dev["C"], dev["D"], dev["delta_bias"],
                          dev["dout"], o[1], o[2], True, None, o[3])
    for _ in range(3):
        o = f()
        r = g(o)
    torch.cuda.synchronize()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    tf = tb = 0.0
    for _ in range(iters):
        ev[0].record()
        o = f()
        ev[1].record()
        r = g(o)
        ev[2].record()
        torch.cuda.synchronize()
        tf += ev[0].elapsed_time(ev[1])
        tb += ev[1].elapsed_time(ev[2])
    return tf / iters, tb / iters, [o[0]] + [t for t in r[:7] if t is not None]


def _worst(ours, ref):
    """Largest |ours - ref| over all results, relative to the largest |ref| of the same tensor."""
    worst = 0.0
    for a, b in zip(ours, ref):
        a, b = a.float(), b.float()
        worst = max(worst, float((a - b).abs().max() / b.abs().max().clamp_min(1e-30)))
    return worst


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=None)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--max-batch", type=int, default=32)
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(ROOT, "oracle", "_ref"))
    import selective_nd_scan_cuda_oflex as ref
    assert ref.__file__.endswith(".so"), "expected the compiled reference extension in oracle/_ref"
    lines = ["| config | B K D N H W dtype | N timed | reference fwd / bwd (ms) | this library fwd / bwd (ms) | speed-up | "
             "this library at full N: fwd / bwd (ms), elements/s | max abs deviation from the reference / max abs value |", "|---|---|---|---|---|---|---|---|"]
    print(torch.cuda.get_device_name(0), flush=True)
    for name, (b, K, D, N, H, W, dt) in CONFIGS.items():
        b = min(b, args.max_batch)
        n = min(N, REF_MAX_DSTATE)
        assert n <= REF_MAX_DSTATE
        inp = make_inputs(b, K, D, n, H, W, dtype=dt, seed=0)
        dev = {k: (v.cuda() if v is not None else None) for k, v in inp.items()}
        rf, rb, rres = _time(ref, dev, args.iters)
        of, ob, ores = _time(cs2d, dev, args.iters)
        dev_excess = _worst(ores, rres)
        full = f"{of:.3f} / {ob:.3f}, {b * K * D * n * H * W / ((of + ob) * 1e-3):.3e}"
        if n != N:
            del dev, rres, ores
            torch.cuda.empty_cache()
            inp = make_inputs(b, K, D, N, H, W, dtype=dt, seed=0)
            dev = {k: (v.cuda() if v is not None else None) for k, v in inp.items()}
            ff, fb, _ = _time(cs2d, dev, args.iters)
            full = f"{ff:.3f} / {fb:.3f}, {b * K * D * N * H * W / ((ff + fb) * 1e-3):.3e}"
        line = (f"| {name} | {b} {K} {D} {N} {H} {W} {str(dt)[6:]} | {n} | {rf:.2f} / {rb:.2f} | {of:.3f} / {ob:.3f} | "
                f"{(rf + rb) / (of + ob):.1f}x | {full} | {dev_excess:.1e} |")
        print(line, flush=True)
        lines.append(line)
        del dev
        torch.cuda.empty_cache()
        if cs2d.device_status() != 0:
            raise RuntimeError(f"device status {cs2d.device_status()}")
    if args.out:
        with open(args.out, "w") as fh:
            fh.write("\n".join(lines) + "\n")


if __name__ == "__main__":
    main()
