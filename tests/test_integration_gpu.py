"""The reference's own pybind module (its host file, its checks, its ``fwd`` / ``bwd`` signatures) with
this library's kernels underneath, on the reference's golden vectors.

``tests/integration/make_binding.py`` edits the reference's ``selective_scan_oflex.cpp`` as a maintainer
would (allocation of the saved state, the two dispatch blocks) and builds it against ``libcs2d.so``;
it needs a checkout of the reference, so the module is built where one is available and travels
with the other built libraries."""
import importlib.util
import os

import pytest
import torch

from conftest import ROOT, TOL, check_close

pytestmark = pytest.mark.gpu
SO = os.path.join(ROOT, "tests", "integration", "_build", "selective_nd_scan_cuda_oflex.so")
NAMES = ("du", "ddelta", "dA", "dB", "dC", "dD", "ddelta_bias", "dA_decay")


@pytest.fixture(scope="module")
def ext():
    if not os.path.exists(SO):
        pytest.skip("the reference-side binding is not built (tests/integration/make_binding.py needs the reference)")
    spec = importlib.util.spec_from_file_location("selective_nd_scan_cuda_oflex", SO)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_reference_pybind_module_on_cs2d_matches_golden_vectors(ext, golden):
    dt = {"torch.float32": torch.float32, "torch.bfloat16": torch.bfloat16, "torch.float16": torch.float16}[
        str(golden["dtype"])]
    rtol, atol = TOL[str(golden["dtype"]).replace("torch.", "")]
    d = {}
    for k in ("u", "delta", "A", "B", "C", "D", "delta_bias", "A_decay", "dout"):
        v = golden.get("in_" + k)
        d[k] = None if v is None else (torch.from_numpy(v).to(dt) if k in ("u", "delta", "B", "C", "dout")
                                       else torch.from_numpy(v)).cuda()
    softplus, out_float = bool(golden["softplus"]), bool(golden["out_float"])
    dout = d["dout"].float() if out_float else d["dout"]
    out, x, x_v, x_sd = ext.fwd(d["u"], d["delta"], d["A"], d["B"], d["C"], d["D"], d["delta_bias"], softplus, out_float,
                                d["A_decay"])
    g = ext.bwd(d["u"], d["delta"], d["A"], d["B"], d["C"], d["D"], d["delta_bias"], dout, x, x_v, softplus,
                d["A_decay"], x_sd)
    torch.cuda.synchronize()
    assert out.dtype == (torch.float32 if out_float else dt)
    check_close("out", out.float().cpu().numpy(), golden["ref_out"], rtol, atol)
    for k, t in zip(NAMES, g):
        if "ref_" + k in golden:
            assert t is not None, k
            check_close(k, t.float().cpu().numpy(), golden["ref_" + k], rtol, atol)
        else:
            assert t is None, k


def test_reference_checks_still_guard_the_module(ext):
    u = torch.zeros(1, 4, 8, 8, device="cuda")
    with pytest.raises(RuntimeError):   # the reference's own TORCH_CHECK on the state dimension
        ext.fwd(u, u, torch.zeros(4, 17, device="cuda"), torch.zeros(1, 2, 17, 8, 8, device="cuda"),
                torch.zeros(1, 2, 17, 8, 8, device="cuda"), None, None, True, False, None)
