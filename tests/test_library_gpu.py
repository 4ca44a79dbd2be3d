"""Dispatcher operators on the GPU: same results as cs2d.ops, torch.library.opcheck, CUDA-graph replay."""
import pytest
import torch

import cs2d
import cs2d.library as L
from cs2d.synthetic import make_inputs

pytestmark = pytest.mark.gpu
NAMES = ("u", "delta", "A", "B", "C", "D", "delta_bias")


def _dev(shape, dtype=torch.float32, seed=4, grad=True):
    inp = make_inputs(*shape, dtype=dtype, seed=seed)
    return {k: (v.cuda().requires_grad_(grad and k in NAMES) if v is not None else None) for k, v in inp.items()}


def test_matches_the_autograd_function():
    a, b = _dev((2, 4, 6, 16, 20, 40)), _dev((2, 4, 6, 16, 20, 40))
    ya = cs2d.selective_scan_2d(*[a[k] for k in NAMES], True)
    yb = L.selective_scan_2d(*[b[k] for k in NAMES], True)
    assert torch.equal(ya, yb)
    ya.backward(a["dout"]); yb.backward(b["dout"])
    for k in NAMES:
        # du/ddelta are computed by one owner each (bit-identical); the rest are atomic sums
        if k in ("u", "delta"):
            assert torch.equal(a[k].grad, b[k].grad), k
        else:
            torch.testing.assert_close(a[k].grad, b[k].grad, rtol=1e-4, atol=1e-4)
    assert cs2d.device_status() == 0


def test_delta_groups_and_missing_optionals():
    inp = make_inputs(2, 4, 8, 4, 9, 14, seed=3, delta_dim=16, with_D=False)
    d = {k: (v.cuda().requires_grad_(k in NAMES) if v is not None else None) for k, v in inp.items()}
    e = {k: (v.detach().clone().requires_grad_(k in NAMES) if v is not None else None) for k, v in d.items()}
    ya = cs2d.selective_scan_2d(d["u"], d["delta"], d["A"], d["B"], d["C"], None, d["delta_bias"], True)
    yb = L.selective_scan_2d(e["u"], e["delta"], e["A"], e["B"], e["C"], None, e["delta_bias"], True)
    ya.backward(d["dout"]); yb.backward(e["dout"])
    assert torch.equal(ya, yb)
    for k in ("u", "delta", "A", "B", "C", "delta_bias"):
        torch.testing.assert_close(d[k].grad, e[k].grad, rtol=1e-4, atol=1e-4)


def test_opcheck():
    d = _dev((1, 2, 3, 4, 6, 10))
    args = (d["u"], d["delta"], d["A"], d["B"], d["C"], d["D"], d["delta_bias"], True, False, None)
    torch.library.opcheck(torch.ops.cs2d.scan_fwd.default, args,
                          test_utils=("test_schema", "test_autograd_registration", "test_faketensor"))
    out, saved = torch.ops.cs2d.scan_fwd(*[t.detach() if isinstance(t, torch.Tensor) else t for t in args])
    nd = [t.detach() for t in (d["u"], d["delta"], d["A"], d["B"], d["C"], d["D"], d["delta_bias"])]
    torch.library.opcheck(torch.ops.cs2d.scan_bwd.default, (*nd, d["dout"], saved, True, None),
                          test_utils=("test_schema", "test_faketensor"))


def test_cuda_graph_replay_matches_eager():
    shape = (2, 4, 6, 16, 20, 40)
    d = _dev(shape, grad=False)
    static = {k: d[k].clone() for k in NAMES + ("dout",)}

    def step():
        out, saved = torch.ops.cs2d.scan_fwd(*[static[k] for k in NAMES], True, False, None)
        grads = torch.ops.cs2d.scan_bwd(*[static[k] for k in NAMES], static["dout"], saved, True, None)
        return (out,) + tuple(grads)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):           # first launches set the kernels' attributes outside the capture
        for _ in range(2):
            step()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        res = step()
    other = _dev(shape, seed=11, grad=False)
    for k in static:
        static[k].copy_(other[k])
    graph.replay()
    torch.cuda.synchronize()
    got = [t.clone() for t in res]
    eager = step()
    torch.cuda.synchronize()
    assert torch.equal(got[0], eager[0]) and torch.equal(got[1], eager[1]) and torch.equal(got[2], eager[2])
    for a, b in zip(got[3:], eager[3:]):
        torch.testing.assert_close(a, b, rtol=1e-4, atol=1e-4)
    assert cs2d.device_status() == 0
