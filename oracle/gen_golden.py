"""TEST INFRASTRUCTURE.  Generates tests/golden/*.npz from the REFERENCE itself.

Runs the reference CUDA extension (``selective_nd_scan_cuda_oflex``, built from
the reference's own sources by ``make -C oracle ref`` into ``oracle/_ref/``) on
seeded inputs on a GPU and stores inputs and outputs.  The fixtures pin the CPU
restatement in ``oracle/`` (tests/test_oracle_cpu.py) and the CUDA kernels
(tests/test_parity_gpu.py).

    python oracle/gen_golden.py            # needs a CUDA device and oracle/_ref

Every case uses dstate <= 12: the reference's backward kernel writes its
per-state dA staging array 16 bytes past the shared memory it requests when
dstate > 12 (selective_scan_bwd_kernel_oflex.cuh:119 and :909), which is an
illegal address on B200 for the fp32 kernels, so it must not be run there.
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "official-cross-scan_b200"))
from cs2d.synthetic import make_inputs  # noqa: E402

# name: (shape (B,K,D,N,H,W), dtype, make_inputs kwargs, delta_softplus, out_float)
CASES = {
    "c1_fp32": ((1, 4, 8, 4, 8, 8), torch.float32, {}, True, False),
    "ragged_multichunk_fp32": ((1, 2, 4, 6, 37, 19), torch.float32, {}, True, False),
    "bf16": ((2, 4, 8, 8, 20, 24), torch.bfloat16, {}, True, False),
    "fp16_outfloat_n1": ((1, 2, 6, 1, 14, 14), torch.float16, {}, True, True),
    "delta_groups_noD": ((2, 4, 8, 4, 9, 14), torch.float32, {"delta_dim": 16, "with_D": False}, True, False),
    "decay_nobias_nosoftplus": ((1, 4, 8, 4, 7, 7), torch.float32, {"a_decay": 0.9, "with_bias": False}, False, False),
    "wide_fp32": ((1, 1, 2, 2, 5, 150), torch.float32, {}, True, False),
    "n12_56x56_fp32": ((1, 4, 2, 12, 56, 56), torch.float32, {}, True, False),
}


def main():
    sys.path.insert(0, os.path.join(ROOT, "oracle", "_ref"))
    import selective_nd_scan_cuda_oflex as ref
    assert ref.__file__.endswith(".so"), "expected the compiled reference extension in oracle/_ref"
    out_dir = os.path.join(ROOT, "tests", "golden")
    os.makedirs(out_dir, exist_ok=True)
    for name, (shape, dtype, kw, softplus, out_float) in CASES.items():
        assert shape[3] <= 12
        inp = make_inputs(*shape, dtype=dtype, seed=0, **kw)
        if not softplus:  # keep delta positive so that exp(delta*A) decays
            inp["delta"] = (inp["delta"].float().abs() * 0.1).to(dtype)
        dev = {k: (v.cuda() if v is not None else None) for k, v in inp.items()}
        dout = dev["dout"].float() if out_float else dev["dout"]
        o = ref.fwd(dev["u"], dev["delta"], dev["A"], dev["B"], dev["C"], dev["D"], dev["delta_bias"], softplus,
                    out_float, dev["A_decay"])
        g = ref.bwd(dev["u"], dev["delta"], dev["A"], dev["B"], dev["C"], dev["D"], dev["delta_bias"], dout,
                    o[1], o[2], softplus, dev["A_decay"], o[3])
        torch.cuda.synchronize()
        rec = {"shape": np.array(shape), "softplus": np.array(softplus), "out_float": np.array(out_float),
               "dtype": np.array(str(dtype))}
        for k, v in inp.items():
            if v is not None:
                rec["in_" + k] = v.float().numpy()
        rec["ref_out"] = o[0].float().cpu().numpy()
        for k, v in zip(("du", "ddelta", "dA", "dB", "dC", "dD", "ddelta_bias", "dA_decay"), g):
            if v is not None:
                rec["ref_" + k] = v.float().cpu().numpy()
        np.savez_compressed(os.path.join(out_dir, name + ".npz"), **rec)
        print("wrote", name, {k: v.shape for k, v in rec.items() if k.startswith("ref_")})


if __name__ == "__main__":
    main()
