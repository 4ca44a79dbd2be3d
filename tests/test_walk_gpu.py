"""The row-walk forward (rows of at most 64 columns, more than 8 states per channel: the lanes of a row work
one image row apart, so the recurrence along the row needs no scan) against the float64 oracle, and the
backward that follows it, which reads the checkpoints this forward wrote: every lane count, strips of 7
and of 8 columns, ragged rows, channel counts that leave warps or lanes idle, 9 to 16 states, all three
input types, fp32 output, shared delta, A_decay, missing optionals, strided views."""
import numpy as np
import pytest
import torch

from conftest import TOL, check_close
import cs2d
from cs2d.synthetic import make_inputs
from oracle import cs2d_oracle as O

pytestmark = pytest.mark.gpu
NAMES = ("du", "ddelta", "dA", "dB", "dC", "dD", "ddelta_bias")

CASES = [
    ((1, 4, 6, 16, 14, 14), torch.float32, {}),        # 2 lanes per row, strips of 7
    ((2, 2, 5, 16, 9, 7), torch.float32, {}),          # 1 lane per row: 8 channels per warp, 5 used
    ((1, 1, 3, 12, 5, 30), torch.float32, {}),         # strips of 8 (4 lanes), 12 states: idle state pairs
    ((2, 4, 9, 16, 13, 56), torch.bfloat16, {}),       # 8 lanes of 7: the 56-column stage; 13 rows: a short last block
    ((1, 2, 8, 9, 28, 28), torch.bfloat16, {}),        # 9 states: a pair with one live half
    ((1, 1, 7, 16, 6, 60), torch.float32, {}),         # strips of 8, last strip ragged
    ((1, 1, 2, 10, 3, 64), torch.float16, {}),         # the widest row
    ((1, 1, 13, 16, 11, 40), torch.float32, {}),       # 13 channels: a second CTA with one channel
    ((2, 4, 8, 16, 7, 7), torch.bfloat16, {"with_D": False, "with_bias": False}),
    ((1, 1, 1, 16, 1, 1), torch.float32, {}),          # a single pixel
    ((1, 2, 30, 16, 5, 8), torch.float32, {}),
    ((1, 2, 14, 16, 56, 56), torch.float32, {}),
]


def _dev(inp):
    return {k: (v.cuda() if v is not None else None) for k, v in inp.items()}


def _oracle(inp, softplus=True):
    f = {k: (v.float() if v is not None else None) for k, v in inp.items()}
    yo = O.fwd(f["u"], f["delta"], f["A"], f["B"], f["C"], f["D"], f["delta_bias"], softplus, f.get("A_decay"))
    go = O.bwd(f["u"], f["delta"], f["A"], f["B"], f["C"], f["D"], f["delta_bias"], f["dout"], softplus, f.get("A_decay"))
    return yo, go


@pytest.mark.parametrize("shape,dtype,kw", CASES, ids=[f"{s}-{str(d)[6:]}" for s, d, _ in CASES])
def test_row_walk_forward_and_the_backward_behind_it(shape, dtype, kw):
    inp = make_inputs(*shape, dtype=dtype, seed=4, **kw)
    d = _dev(inp)
    args = (d["u"], d["delta"], d["A"], d["B"], d["C"], d["D"], d["delta_bias"])
    o = cs2d.fwd(*args, True, False, None)
    g = cs2d.bwd(*args, d["dout"], o[1], o[2], True, None, o[3])
    assert torch.equal(cs2d.fwd_only(*args, True, False, None), o[0])   # the same kernel without checkpoints
    yo, go = _oracle(inp)
    rtol, atol = TOL[str(dtype)[6:]]
    check_close("out", o[0].float().cpu().numpy(), yo, rtol, atol)
    for name, t in zip(NAMES, g):
        if t is None:
            assert go[name] is None, name
            continue
        check_close(name, t.float().cpu().numpy(), go[name], rtol, atol)
    assert cs2d.device_status() == 0


def test_state_decay_fp32_output_no_softplus_strided():
    inp = make_inputs(2, 2, 6, 16, 12, 20, dtype=torch.bfloat16, seed=5, with_bias=False, a_decay=0.9)
    inp["delta"] = (inp["delta"].float().abs() * 0.1).to(torch.bfloat16)
    d = _dev(inp)
    big = torch.zeros(2, 20, 12, 20, dtype=torch.bfloat16, device="cuda")
    big[:, 3:15] = d["u"]
    d["u"] = big[:, 3:15]                       # a channel slice of a larger tensor
    args = (d["u"], d["delta"], d["A"], d["B"], d["C"], d["D"], d["delta_bias"])
    o = cs2d.fwd(*args, False, True, d["A_decay"])
    assert o[0].dtype == torch.float32
    f = {k: (v.float() if v is not None else None) for k, v in inp.items()}
    yo = O.fwd(f["u"], f["delta"], f["A"], f["B"], f["C"], f["D"], f["delta_bias"], False, f["A_decay"])
    check_close("out", o[0].cpu().numpy(), yo, 1e-4, 1e-5)   # fp32 output: arithmetic error only
    g = cs2d.bwd(*args, d["dout"].float(), o[1], o[2], False, d["A_decay"], o[3])
    go = O.bwd(f["u"], f["delta"], f["A"], f["B"], f["C"], f["D"], f["delta_bias"], f["dout"], False, f["A_decay"])
    for name, t in zip(NAMES, g):
        if t is not None:
            check_close(name, t.float().cpu().numpy(), go[name], 2e-2, 1e-3)
    assert cs2d.device_status() == 0


def test_shared_delta():
    inp = make_inputs(1, 2, 6, 16, 8, 20, dtype=torch.float32, seed=6, delta_dim=4)
    d = _dev(inp)
    args = (d["u"], d["delta"], d["A"], d["B"], d["C"], d["D"], d["delta_bias"])
    o = cs2d.fwd(*args, True, False, None)
    yo, _ = _oracle(inp)
    check_close("out", o[0].cpu().numpy(), yo, 1e-4, 1e-5)
    assert cs2d.device_status() == 0
