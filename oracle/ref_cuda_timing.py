"""TEST INFRASTRUCTURE.  Times the reference's own CUDA extension (``make -C oracle ref`` ->
``oracle/_ref``) on one benchmark configuration and prints one JSON line.

    python oracle/ref_cuda_timing.py <config name> [batch]

The state dimension is capped at 12: the reference's backward kernel places its per-state dA
staging array 16 bytes past the shared memory it requests when dstate > 12
(selective_scan_bwd_kernel_oflex.cuh:119 and :909), an illegal address on this GPU, so it is
never run there.  Its cost is linear in dstate, so the figure is a fair per-state comparison.
"""
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# oracle/_ref first: the library ships a Python module of the same name as the reference extension
sys.path[:0] = [os.path.join(ROOT, "oracle", "_ref"), os.path.join(ROOT, "official-cross-scan_b200")]
from cs2d.synthetic import CONFIGS, make_inputs  # noqa: E402


def main():
    import selective_nd_scan_cuda_oflex as ref
    assert ref.__file__.endswith(".so"), "expected the compiled reference extension in oracle/_ref"
    name = sys.argv[1]
    B, K, D, N, H, W, dtype = CONFIGS[name]
    if len(sys.argv) > 2:
        B = int(sys.argv[2])
    N = min(N, 12)
    inp = make_inputs(B, K, D, N, H, W, dtype=dtype, seed=0)
    d = {k: (v.cuda() if v is not None else None) for k, v in inp.items()}
    args = (d["u"], d["delta"], d["A"], d["B"], d["C"], d["D"], d["delta_bias"])

    def timed(fn, n):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    o = ref.fwd(*args, True, False, None)
    ref.bwd(*args, d["dout"], o[1], o[2], True, None, o[3])   # warm-up (module load) outside the timing
    fwd_ms = timed(lambda: ref.fwd(*args, True, False, None), 3)
    # the reference's backward overwrites its saved tensors: every call gets a fresh forward's
    outs = [ref.fwd(*args, True, False, None) for _ in range(3)]
    it = iter(outs)
    bwd_ms = timed(lambda: (lambda s: ref.bwd(*args, d["dout"], s[1], s[2], True, None, s[3]))(next(it)), 3)
    print(json.dumps({"implementation": "reference CUDA extension (selective_nd_scan_cuda_oflex, -arch=sm_100)",
                      "workload": name, "shape_BKDNHW": [B, K, D, N, H, W], "dstate_capped_at": 12,
                      "fwd_ms": fwd_ms, "bwd_ms": bwd_ms,
                      "elements_per_s": B * K * D * N * H * W / ((fwd_ms + bwd_ms) * 1e-3)}))


if __name__ == "__main__":
    main()
