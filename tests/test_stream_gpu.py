"""The streaming kernels that serve dstate == 1 (two channels packed per thread, no shared-memory
tiles, no backward scratch) against the float64 oracle: every lane count, odd channel counts per
group (a pair with one live half), ragged rows, all three input types, fp32 output / dout, shared
delta, missing optionals, strided views - and the tile kernels' deterministic backward reading
the streaming forward's checkpoints."""
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
    ((1, 4, 6, 1, 14, 14), torch.float32, {}),        # 2 lanes per row
    ((2, 2, 5, 1, 9, 7), torch.float32, {}),          # 1 lane, odd channels per group
    ((1, 1, 3, 1, 5, 30), torch.float32, {}),         # 4 lanes, ragged last strip
    ((2, 4, 9, 1, 13, 56), torch.bfloat16, {}),       # 8 lanes (7 used), 13 rows: a short last row block
    ((1, 2, 8, 1, 28, 28), torch.bfloat16, {}),       # rows of 56 bytes: 8-byte vector loads
    ((1, 1, 7, 1, 6, 100), torch.float32, {}),        # 16 lanes
    ((1, 1, 2, 1, 3, 120), torch.float16, {}),        # 16 lanes, two channel pairs per warp
    ((2, 4, 8, 1, 7, 7), torch.bfloat16, {"with_D": False, "with_bias": False}),
    ((1, 1, 1, 1, 1, 1), torch.float32, {}),          # a single pixel of a single channel
    ((1, 4, 70, 1, 12, 20), torch.float32, {}),       # more pairs than one CTA holds
    ((2, 1, 33, 1, 4, 9), torch.float16, {}),
]


def _dev(inp):
    return {k: (v.cuda() if v is not None else None) for k, v in inp.items()}


def _oracle(inp, softplus=True):
    f = {k: (v.float() if v is not None else None) for k, v in inp.items()}
    yo = O.fwd(f["u"], f["delta"], f["A"], f["B"], f["C"], f["D"], f["delta_bias"], softplus)
    go = O.bwd(f["u"], f["delta"], f["A"], f["B"], f["C"], f["D"], f["delta_bias"], f["dout"], softplus)
    return yo, go


@pytest.mark.parametrize("shape,dtype,kw", CASES, ids=[f"{s}-{str(d)[6:]}" for s, d, _ in CASES])
def test_streaming_kernels_match_oracle(shape, dtype, kw):
    inp = make_inputs(*shape, dtype=dtype, seed=4, **kw)
    d = _dev(inp)
    args = (d["u"], d["delta"], d["A"], d["B"], d["C"], d["D"], d["delta_bias"])
    o = cs2d.fwd(*args, True, False, None)
    g = cs2d.bwd(*args, d["dout"], o[1], o[2], True, None, o[3])
    assert torch.equal(cs2d.fwd_only(*args, True, False, None), o[0])
    yo, go = _oracle(inp)
    rtol, atol = TOL[str(dtype)[6:]]
    check_close("out", o[0].float().cpu().numpy(), yo, rtol, atol)
    for name, t in zip(NAMES, g):
        if t is None:
            assert go[name] is None, name
            continue
        check_close(name, t.float().cpu().numpy(), go[name], rtol, atol)
    assert cs2d.device_status() == 0


def test_fp32_output_and_gradient_of_16bit_inputs_no_softplus_strided():
    inp = make_inputs(2, 2, 6, 1, 12, 20, dtype=torch.bfloat16, seed=5, with_bias=False)
    inp["delta"] = (inp["delta"].float().abs() * 0.1).to(torch.bfloat16)
    d = _dev(inp)
    big = torch.zeros(2, 20, 12, 20, dtype=torch.bfloat16, device="cuda")
    big[:, 3:15] = d["u"]
    d["u"] = big[:, 3:15]                       # a channel slice of a larger tensor
    args = (d["u"], d["delta"], d["A"], d["B"], d["C"], d["D"], d["delta_bias"])
    o = cs2d.fwd(*args, False, True, None)
    assert o[0].dtype == torch.float32
    g = cs2d.bwd(*args, d["dout"].float(), o[1], o[2], False, None, o[3])
    yo, go = _oracle(inp, softplus=False)
    check_close("out", o[0].cpu().numpy(), yo, 1e-4, 1e-5)   # fp32 output: arithmetic error only
    for name, t in zip(NAMES, g):
        if t is not None:
            check_close(name, t.float().cpu().numpy(), go[name], 2e-2, 1e-3)


def test_shared_delta_fp32():
    inp = make_inputs(1, 2, 6, 1, 8, 20, dtype=torch.float32, seed=6, delta_dim=4)
    d = _dev(inp)
    args = (d["u"], d["delta"], d["A"], d["B"], d["C"], d["D"], d["delta_bias"])
    o = cs2d.fwd(*args, True, False, None)
    g = cs2d.bwd(*args, d["dout"], o[1], o[2], True, None, o[3])
    yo, go = _oracle(inp)
    check_close("out", o[0].cpu().numpy(), yo, 1e-4, 1e-5)
    for name, t in zip(NAMES, g):
        check_close(name, t.cpu().numpy(), go[name], 1e-4, 1e-5)


@pytest.mark.parametrize("shape,dtype", [((3, 2, 9, 1, 14, 14), torch.float32), ((2, 4, 6, 1, 9, 60), torch.bfloat16)])
def test_deterministic_backward_reads_streaming_checkpoints(shape, dtype):
    inp = make_inputs(*shape, dtype=dtype, seed=8)
    d = _dev(inp)
    args = (d["u"], d["delta"], d["A"], d["B"], d["C"], d["D"], d["delta_bias"])
    o = cs2d.fwd(*args, True, False, None)
    run = lambda det: cs2d.bwd(*args, d["dout"], o[1], o[2], True, None, o[3], deterministic=det)
    a, b2 = run(True), run(True)
    _, go = _oracle(inp)
    rtol, atol = TOL[str(dtype)[6:]]
    for name, x, y in zip(NAMES, a, b2):
        assert torch.equal(x, y), f"{name} differs between two deterministic runs"
        check_close(name, x.float().cpu().numpy(), go[name], rtol, atol)
    assert cs2d.device_status() == 0
