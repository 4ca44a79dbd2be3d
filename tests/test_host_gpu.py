"""The host-buffer pipeline (chunked copies overlapping the kernels) against the device operators."""
import pytest
import torch

from conftest import check_close
import cs2d
from cs2d import ops
from cs2d.synthetic import make_inputs

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("chunks", [1, 3, 8, None])
def test_host_pipeline_matches_device_operators(chunks):
    inp = make_inputs(5, 2, 6, 4, 12, 16, dtype=torch.float32, seed=4)
    host = {k: inp[k].pin_memory() for k in ("u", "delta", "B", "C", "dout")}
    params = {k: inp[k].cuda() for k in ("A", "D", "delta_bias")}
    hout = cs2d.alloc_host_outputs(host["u"], host["B"], params["A"], True, True)
    cs2d.fwd_bwd_from_host(host, params, hout, True, False, chunks=chunks)
    torch.cuda.synchronize()
    d = {k: (v.cuda() if v is not None else None) for k, v in inp.items()}
    out, x, xv, xsd = cs2d.fwd(d["u"], d["delta"], d["A"], d["B"], d["C"], d["D"], d["delta_bias"], True, False, None)
    g = cs2d.bwd(d["u"], d["delta"], d["A"], d["B"], d["C"], d["D"], d["delta_bias"], d["dout"], x, xv, True, None, xsd)
    torch.cuda.synchronize()
    assert torch.equal(hout["out"], out.cpu()) and torch.equal(hout["du"], g[0].cpu())
    assert torch.equal(hout["ddelta"], g[1].cpu())
    check_close("dB", hout["dB"].numpy(), g[3].cpu().numpy(), 1e-5, 1e-6)
    check_close("dC", hout["dC"].numpy(), g[4].cpu().numpy(), 1e-5, 1e-6)
    total, parts = ops.param_grad_layout(12, 4, True, True, False)
    flat = torch.cat([g[2].reshape(-1), g[5], g[6]]).cpu()
    check_close("param_grads", hout["param_grads"].numpy(), flat.numpy(), 1e-4, 1e-5)
    assert cs2d.device_status() == 0


def test_host_pipeline_16bit_inputs_and_reuse():
    """bf16 inputs (dB/dC leave in the input type) and a second step on the same preallocated slots."""
    inp = make_inputs(6, 4, 8, 16, 10, 24, dtype=torch.bfloat16, seed=5)
    host = {k: inp[k].pin_memory() for k in ("u", "delta", "B", "C", "dout")}
    params = {k: inp[k].cuda() for k in ("A", "D", "delta_bias")}
    hout = cs2d.alloc_host_outputs(host["u"], host["B"], params["A"], True, True)
    d = {k: (v.cuda() if v is not None else None) for k, v in inp.items()}
    out, x, xv, xsd = cs2d.fwd(d["u"], d["delta"], d["A"], d["B"], d["C"], d["D"], d["delta_bias"], True, False, None)
    g = cs2d.bwd(d["u"], d["delta"], d["A"], d["B"], d["C"], d["D"], d["delta_bias"], d["dout"], x, xv, True, None, xsd)
    for _ in range(2):
        for t in hout.values():
            t.zero_()
        cs2d.fwd_bwd_from_host(host, params, hout, True, False, chunks=4)
        torch.cuda.synchronize()
        assert torch.equal(hout["out"], out.cpu()) and torch.equal(hout["du"], g[0].cpu())
        assert hout["dB"].dtype == torch.bfloat16
        check_close("dB", hout["dB"].float().numpy(), g[3].float().cpu().numpy(), 2e-2, 1e-3)
        check_close("dC", hout["dC"].float().numpy(), g[4].float().cpu().numpy(), 2e-2, 1e-3)
    assert cs2d.device_status() == 0
