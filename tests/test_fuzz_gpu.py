"""Seeded random shapes against the float64 oracle: every lane count (1..32 lanes per row), odd
state counts, column tiles, delta groups, missing optionals, 16-bit inputs - whichever kernel
variant the planner picks for them (warp-specialised, bulk-staged or plain)."""
import random

import numpy as np
import pytest
import torch

from conftest import TOL, check_close
import cs2d
from cs2d.synthetic import make_inputs
from oracle import cs2d_oracle as O

pytestmark = pytest.mark.gpu
NAMES = ("du", "ddelta", "dA", "dB", "dC", "dD", "ddelta_bias")


def _cases(n, seed):
    rng = random.Random(seed)
    out = []
    for i in range(n):
        K, D = rng.choice([1, 2, 4]), rng.randint(1, 12)
        N = rng.choice([1, 2, 3, 5, 8, 9, 11, 12, 13, 15, 16])
        H = rng.randint(1, 23)
        W = rng.choice([rng.randint(1, 40), rng.randint(41, 130), rng.randint(131, 300)])
        kw = {}
        if rng.random() < 0.3:
            kw["with_D"] = False
        if rng.random() < 0.3:
            kw["with_bias"] = False
        if rng.random() < 0.2 and (K * D) % 2 == 0:
            kw["delta_dim"] = K * D // 2
        out.append(((rng.randint(1, 3), K, D, N, H, W), rng.choice([torch.float32, torch.float32, torch.bfloat16]), kw, i))
    return out


@pytest.mark.parametrize("shape,dtype,kw,seed", _cases(24, 7), ids=lambda v: str(v).replace("torch.", ""))
def test_random_shape_matches_oracle(shape, dtype, kw, seed):
    inp = make_inputs(*shape, dtype=dtype, seed=seed, **kw)
    dev = {k: (v.cuda() if v is not None else None) for k, v in inp.items()}
    args = (dev["u"], dev["delta"], dev["A"], dev["B"], dev["C"], dev["D"], dev["delta_bias"])
    o = cs2d.fwd(*args, True, False, None)
    g = cs2d.bwd(*args, dev["dout"], o[1], o[2], True, None, o[3])
    assert torch.equal(cs2d.fwd_only(*args, True, False, None), o[0])
    f = {k: (v.float() if v is not None else None) for k, v in inp.items()}
    yo = O.fwd(f["u"], f["delta"], f["A"], f["B"], f["C"], f["D"], f["delta_bias"], True)
    go = O.bwd(f["u"], f["delta"], f["A"], f["B"], f["C"], f["D"], f["delta_bias"], f["dout"], True)
    rtol, atol = TOL[str(dtype)[6:]]
    check_close("out", o[0].float().cpu().numpy(), yo, rtol, atol)
    ddim = kw.get("delta_dim")
    if ddim and dtype != torch.float32:
        # delta shared by `rep` channels, 16-bit gradients: the operator (like the reference host code,
        # src/cusoflex/selective_scan_oflex.cpp:433-438) rounds every channel's ddelta to the input
        # type and then adds the `rep` rounded values.  The oracle gets the same rounding model:
        # per-channel ddelta in float64, rounded, summed in float32, rounded.
        b, K, D, _, h, w = shape
        rep = K * D // ddim
        bias = f["delta_bias"].repeat_interleave(rep) if f["delta_bias"] is not None else None
        per = O.bwd(f["u"], f["delta"].repeat_interleave(rep, 1), f["A"], f["B"], f["C"], f["D"], bias, f["dout"], True)
        dd = torch.from_numpy(per["ddelta"]).to(dtype).float().view(b, ddim, rep, h, w).sum(2).to(dtype).float()
        go["ddelta"] = dd.numpy()
    for name, t in zip(NAMES, g):
        if t is None:
            assert go[name] is None, name
            continue
        check_close(name, t.float().cpu().numpy(), go[name], rtol, atol)
    assert cs2d.device_status() == 0
