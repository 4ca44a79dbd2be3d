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


def test_block_shapes_and_projection_layout():
    from cs2d.nn import SS2D
    torch.manual_seed(0)
    m = SS2D(d_model=8, d_state=4, expand=2, directions=4)
    assert m.d_inner == 16 and m.dt_rank == 1
    assert m.x_proj.weight.shape == (4 * (1 + 8), 16, 1, 1) and m.dt_proj.shape == (4, 16, 1)
    # what the scan receives: B / C as strided views of the projection output, innermost stride 1
    seen = {}
    m._scan = lambda u, delta, A, B, C, w, D, bias: seen.update(u=u, delta=delta, A=A, B=B, C=C) or torch.zeros_like(u)
    y = m(torch.randn(2, 6, 10, 8))
    assert y.shape == (2, 6, 10, 8)
    assert seen["u"].shape == (2, 16, 6, 10) and seen["delta"].shape == (2, 64, 6, 10)
    assert seen["B"].shape == seen["C"].shape == (2, 4, 4, 6, 10)
    assert seen["B"].stride(-1) == 1 and seen["B"].data_ptr() != seen["C"].data_ptr()
    assert seen["B"]._base is not None and seen["B"]._base is seen["C"]._base      # views of one tensor
