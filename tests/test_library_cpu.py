"""Dispatcher registration (cs2d.library): schemas and shape-only (fake) implementations, no GPU."""
import torch
from torch._subclasses.fake_tensor import FakeTensorMode

import cs2d.library as L
from cs2d import ops


def _fakes(b=2, K=4, D=8, N=16, H=56, W=56, dtype=torch.float32, ddim=None):
    dim = K * D
    ddim = dim if ddim is None else ddim
    mk = lambda *s, dt=dtype: torch.empty(*s, dtype=dt, device="cuda")
    return dict(u=mk(b, dim, H, W), delta=mk(b, ddim, H, W), A=mk(dim, N, dt=torch.float32), B=mk(b, K, N, H, W),
                C=mk(b, K, N, H, W), D=mk(dim, dt=torch.float32), bias=mk(ddim, dt=torch.float32))


def test_schemas_registered():
    f, g = torch.ops.cs2d.scan_fwd.default._schema, torch.ops.cs2d.scan_bwd.default._schema
    assert [a.name for a in f.arguments] == ["u", "delta", "A", "B", "C", "D", "delta_bias", "delta_softplus",
                                             "out_float", "A_decay"]
    assert len(f.returns) == 2 and len(g.returns) == 5
    assert not any(a.alias_info for a in list(f.arguments) + list(g.arguments))


def test_fake_forward_and_backward_shapes():
    with FakeTensorMode():
        t = _fakes(dtype=torch.bfloat16)
        out, saved = torch.ops.cs2d.scan_fwd(t["u"], t["delta"], t["A"], t["B"], t["C"], t["D"], t["bias"], True, False,
                                             None)
        assert out.shape == t["u"].shape and out.dtype == torch.bfloat16 and out.device.type == "cuda"
        assert saved.dtype == torch.float32 and saved.dim() == 1 and saved.numel() > 0
        outf, _ = torch.ops.cs2d.scan_fwd(t["u"], t["delta"], t["A"], t["B"], t["C"], None, None, True, True, None)
        assert outf.dtype == torch.float32
        du, dd, dB, dC, flat = torch.ops.cs2d.scan_bwd(t["u"], t["delta"], t["A"], t["B"], t["C"], t["D"], t["bias"],
                                                       out, saved, True, None)
        assert du.shape == t["u"].shape and dd.shape == t["delta"].shape and dB.shape == t["B"].shape
        assert dC.dtype == torch.bfloat16
        assert flat.numel() == ops.param_grad_layout(32, 16, True, True, False)[0]


def test_fake_saved_size_matches_the_planner():
    with FakeTensorMode():
        t = _fakes(b=1, K=2, D=3, N=5, H=9, W=300)   # three column tiles
        _, saved = torch.ops.cs2d.scan_fwd(t["u"], t["delta"], t["A"], t["B"], t["C"], None, None, False, False, None)
    assert saved.numel() * 4 > 1 * 6 * 3 * 300 * 4   # at least one checkpoint row per channel and state pair
