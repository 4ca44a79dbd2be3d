"""Parameterisation of the CrossScan2D module (no GPU needed)."""
import torch

from cs2d.nn import CrossScan2D


def test_parameters_and_init():
    torch.manual_seed(0)
    m = CrossScan2D(d_inner=6, d_state=4, directions=4)
    shapes = {k: tuple(v.shape) for k, v in m.named_parameters()}
    assert shapes == {"A_log": (24, 4), "D": (24,), "dt_bias": (24,), "fusion": (4, 6)}
    A = -torch.exp(m.A_log)
    assert torch.allclose(A[0], -torch.arange(1, 5, dtype=torch.float32))
    dt = torch.nn.functional.softplus(m.dt_bias)
    assert (dt >= 1e-4).all() and (dt <= 1e-1 + 1e-6).all()
    assert torch.allclose(m.fusion.sum(0), torch.ones(6))
    assert "d_inner=6" in repr(m)
