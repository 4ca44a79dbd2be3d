"""TEST INFRASTRUCTURE.  How far do fp32 kernels sit from float64 on the batch-reduced
gradients at full size - the reference's own CUDA extension, and this library?

dA, dD and ddelta_bias sum over batch * H * W terms (and dA over more), every term an fp32
result with its own rounding error; the sums cancel heavily, so the absolute error of a sum is
set by the magnitude of its terms, not of its value.  This script runs the reference extension
(``make -C oracle ref`` -> ``oracle/_ref``) and the cs2d kernels on the stage-1 feature map at
the benchmark batch - B32, one direction of D192, 56x56, fp32, dstate 12 (the reference's
backward must not be run above 12, see gen_golden.py) - and prints, per tensor, the worst
|err| / (1e-5 + 1e-4 |ref|) of each against the float64 oracle.

    python oracle/ref_reduction_error.py [out.json]      # needs a CUDA device and oracle/_ref
"""
import json
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path[:0] = [os.path.join(ROOT, "official-cross-scan_b200"), ROOT]
from cs2d.synthetic import make_inputs  # noqa: E402
from oracle import cs2d_oracle as O     # noqa: E402

NAMES = ("du", "ddelta", "dA", "dB", "dC", "dD", "ddelta_bias")


def ratios(g, go):
    out = {}
    for name, t in zip(NAMES, g):
        got, ref = t.float().cpu().numpy().astype(np.float64), np.asarray(go[name], np.float64)
        out[name] = float((np.abs(got - ref) / (1e-5 + 1e-4 * np.abs(ref))).max())
    return out


def main():
    sys.path.insert(0, os.path.join(ROOT, "oracle", "_ref"))
    import selective_nd_scan_cuda_oflex as ref
    assert ref.__file__.endswith(".so"), "expected the compiled reference extension in oracle/_ref"
    import cs2d
    shape = (32, 1, 192, 12, 56, 56)
    inp = make_inputs(*shape, dtype=torch.float32, seed=0)
    d = {k: (v.cuda() if v is not None else None) for k, v in inp.items()}
    args = (d["u"], d["delta"], d["A"], d["B"], d["C"], d["D"], d["delta_bias"])
    go = O.bwd(inp["u"], inp["delta"], inp["A"], inp["B"], inp["C"], inp["D"], inp["delta_bias"], inp["dout"], True)
    res = {"shape_BKDNHW": list(shape), "tolerance": "1e-5 + 1e-4*|ref|"}
    o = ref.fwd(*args, True, False, None)
    g = ref.bwd(*args, d["dout"], o[1], o[2], True, None, o[3])
    torch.cuda.synchronize()
    res["reference_extension"] = ratios(g[:7], go)
    o = cs2d.fwd(*args, True, False, None)
    g = cs2d.bwd(*args, d["dout"], o[1], o[2], True, None, o[3])
    torch.cuda.synchronize()
    res["cs2d"] = ratios(g[:7], go)
    print(json.dumps(res, indent=1))
    if len(sys.argv) > 1:
        with open(sys.argv[1], "w") as f:
            json.dump(res, f, indent=1)


if __name__ == "__main__":
    main()
