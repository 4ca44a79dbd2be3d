"""The CPU restatement against (1) autograd of an independent forward
restatement and (2) outputs of the reference CUDA extension itself
(tests/golden, generated on a B200 by oracle/gen_golden.py)."""
import numpy as np
import pytest
import torch

from conftest import TOL, check_close
from cs2d.synthetic import make_inputs
from oracle import cs2d_oracle as O


def _oracle_inputs(rec):
    g = lambda k: rec.get("in_" + k)
    return g("u"), g("delta"), g("A"), g("B"), g("C"), g("D"), g("delta_bias"), g("A_decay"), g("dout")


def test_golden_set_present():
    from conftest import GOLDEN
    assert len(GOLDEN) >= 8


def test_oracle_matches_reference_outputs(golden):
    u, delta, A, B, C, D, bias, decay, dout = _oracle_inputs(golden)
    softplus = bool(golden["softplus"])
    rtol, atol = TOL[str(golden["dtype"]).replace("torch.", "")]
    y = O.fwd(u, delta, A, B, C, D, bias, softplus, decay)
    check_close("out", golden["ref_out"], y, rtol, atol)
    g = O.bwd(u, delta, A, B, C, D, bias, dout, softplus, decay)
    for k in ("du", "ddelta", "dA", "dB", "dC", "dD", "ddelta_bias"):
        if "ref_" + k in golden:
            check_close(k, golden["ref_" + k], g[k], rtol, atol)
    if "ref_dA_decay" in golden:  # the reference's value omits the row-scan term
        check_close("dA_decay", golden["ref_dA_decay"], g["dA_decay_ref"], rtol, atol)
        assert abs(float(g["dA_decay_ref"][0]) - float(g["dA_decay_true"][0])) > 1e-3


@pytest.mark.parametrize("kw", [dict(), dict(delta_dim=16), dict(a_decay=0.9), dict(with_D=False, with_bias=False)])
def test_adjoint_matches_autograd(kw):
    inp = make_inputs(1, 4, 8, 4, 8, 8, seed=0, **kw)
    t = {k: (v.double().requires_grad_(True) if v is not None and k != "dout" else v) for k, v in inp.items()}
    y = O.fwd_torch(t["u"], t["delta"], t["A"], t["B"], t["C"], t["D"], t["delta_bias"], True, t["A_decay"])
    yo = O.fwd(inp["u"], inp["delta"], inp["A"], inp["B"], inp["C"], inp["D"], inp["delta_bias"], True, inp["A_decay"])
    np.testing.assert_allclose(y.detach().numpy(), yo, rtol=1e-12, atol=1e-12)
    y.backward(inp["dout"].double())
    g = O.bwd(inp["u"], inp["delta"], inp["A"], inp["B"], inp["C"], inp["D"], inp["delta_bias"], inp["dout"], True,
              inp["A_decay"])
    pairs = [("du", "u"), ("ddelta", "delta"), ("dA", "A"), ("dB", "B"), ("dC", "C"), ("dD", "D"),
             ("ddelta_bias", "delta_bias"), ("dA_decay_true", "A_decay")]
    for k, tk in pairs:
        if g[k] is not None:
            np.testing.assert_allclose(g[k], t[tk].grad.numpy(), rtol=1e-10, atol=1e-10, err_msg=k)


def test_no_softplus_and_ragged_shapes():
    inp = make_inputs(2, 2, 3, 5, 5, 11, seed=3)
    inp["delta"] = inp["delta"].abs() * 0.1
    t = {k: (v.double().requires_grad_(True) if v is not None and k != "dout" else v) for k, v in inp.items()}
    y = O.fwd_torch(t["u"], t["delta"], t["A"], t["B"], t["C"], t["D"], t["delta_bias"], False, None)
    y.backward(inp["dout"].double())
    g = O.bwd(inp["u"], inp["delta"], inp["A"], inp["B"], inp["C"], inp["D"], inp["delta_bias"], inp["dout"], False)
    np.testing.assert_allclose(g["ddelta"], t["delta"].grad.numpy(), rtol=1e-10, atol=1e-10)
    np.testing.assert_allclose(g["dA"], t["A"].grad.numpy(), rtol=1e-10, atol=1e-10)


def test_float32_build_tracks_float64():
    inp = make_inputs(1, 4, 8, 16, 14, 14, seed=1)
    a = (inp["u"], inp["delta"], inp["A"], inp["B"], inp["C"], inp["D"], inp["delta_bias"])
    y64 = O.fwd(*a, True)
    y32 = O.fwd(*a, True, dtype=np.float32)
    check_close("out32", y32, y64, 1e-4, 1e-5)
    g64 = O.bwd(*a, inp["dout"], True)
    g32 = O.bwd(*a, inp["dout"], True, dtype=np.float32)
    for k in ("du", "ddelta", "dB", "dC"):
        check_close(k, g32[k], g64[k], 1e-4, 1e-5)


def test_oracle_rejects_bad_shapes():
    inp = make_inputs(1, 2, 3, 4, 4, 4)
    with pytest.raises(ValueError):
        O.fwd(inp["u"], inp["delta"], inp["A"], inp["B"][:, :, :3], inp["C"], None, None)
    with pytest.raises(ValueError):
        O.fwd(inp["u"], inp["delta"], torch.zeros(6, 17), torch.zeros(1, 2, 17, 4, 4), torch.zeros(1, 2, 17, 4, 4))
