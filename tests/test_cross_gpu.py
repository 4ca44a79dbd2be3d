"""Four-corner CrossScan with direction-fusion weights against the float64
restatement (flip -> reference recurrence -> flip back -> weighted sum)."""
import numpy as np
import pytest
import torch

from conftest import check_close
import cs2d
from cs2d.synthetic import make_inputs
from oracle import cs2d_oracle as O

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape,dtype", [((2, 4, 3, 4, 6, 9), torch.float32), ((1, 4, 4, 16, 8, 8), torch.bfloat16),
                                         ((1, 4, 2, 2, 5, 13), torch.float32), ((1, 4, 1, 2, 3, 260), torch.float32),
                                         ((1, 4, 2, 16, 5, 336), torch.float32), ((2, 4, 3, 9, 6, 300), torch.bfloat16)])
@pytest.mark.parametrize("det", [False, True], ids=["atomic", "serial"])
def test_cross_scan_forward_and_gradients(shape, dtype, det):
    b, K, d, n, h, w = shape
    inp = make_inputs(b, K, d, n, h, w, dtype=dtype, seed=2)
    gen = torch.Generator().manual_seed(9)
    u0 = torch.randn(b, d, h, w, generator=gen).to(dtype)
    wt = (torch.rand(K, d, generator=gen) + 0.1)
    dy = torch.randn(b, d, h, w, generator=gen).to(dtype)
    names = ("u", "delta", "A", "B", "C", "w", "D", "delta_bias")
    host = dict(u=u0, delta=inp["delta"], A=inp["A"], B=inp["B"], C=inp["C"], w=wt, D=inp["D"],
                delta_bias=inp["delta_bias"])
    dev = {k: v.cuda().requires_grad_(True) for k, v in host.items()}
    y = cs2d.cross_scan_2d(*[dev[k] for k in names], True, deterministic=det)
    y.backward(dy.cuda())
    ref = {k: v.double().requires_grad_(True) for k, v in host.items()}
    yo = O.cross_fwd_torch(*[ref[k] for k in names], True)
    yo.backward(dy.double())
    rtol, atol = (1e-4, 1e-5) if dtype == torch.float32 else (2e-2, 1e-3)
    check_close("y", y.detach().float().cpu().numpy(), yo.detach().numpy(), rtol, atol)
    for k in names:
        check_close("d" + k, dev[k].grad.float().cpu().numpy(), ref[k].grad.numpy(), rtol, atol)
    assert cs2d.device_status() == 0


def test_module_trains_all_parameters():
    from cs2d.nn import CrossScan2D
    torch.manual_seed(1)
    m = CrossScan2D(d_inner=4, d_state=4).cuda()
    u = torch.randn(2, 4, 6, 10, device="cuda")
    delta = torch.randn(2, 16, 6, 10, device="cuda")
    Bm, Cm = torch.randn(2, 4, 4, 6, 10, device="cuda"), torch.randn(2, 4, 4, 6, 10, device="cuda")
    y = m(u, delta, Bm, Cm)
    assert y.shape == u.shape
    y.square().mean().backward()
    for name, p in m.named_parameters():
        assert p.grad is not None and torch.isfinite(p.grad).all() and p.grad.abs().sum() > 0, name


@pytest.mark.parametrize("shape", [(2, 4, 5, 16, 12, 20), (1, 4, 3, 9, 6, 300)])
def test_evaluation_path_keeps_no_state_and_matches(shape):
    b, K, d, n, h, w_ = shape
    inp = make_inputs(b, K, d, n, h, w_, seed=3)
    u0 = torch.randn(b, d, h, w_, device="cuda")
    w = torch.rand(K, d, device="cuda") + 0.1
    dev = {k: (v.cuda() if v is not None else None) for k, v in inp.items()}
    args = (u0, dev["delta"], dev["A"], dev["B"], dev["C"], w, dev["D"], dev["delta_bias"], True)
    y_train = cs2d.cross_scan_2d(*[a.clone().requires_grad_(True) if isinstance(a, torch.Tensor) else a for a in args])
    with torch.no_grad():
        y_eval = cs2d.cross_scan_2d(*args)
    # the directions add onto the image with fp32 atomics: the order, hence the last bit, may differ
    torch.testing.assert_close(y_train.detach(), y_eval, rtol=1e-5, atol=1e-5)
    # the reproducible form: one CTA writes its part of the merged image, direction after direction
    y_det = cs2d.cross_scan_2d(*[a.clone().requires_grad_(True) if isinstance(a, torch.Tensor) else a for a in args],
                               deterministic=True)
    with torch.no_grad():
        assert torch.equal(y_det.detach(), cs2d.cross_scan_2d(*args, deterministic=True))
    torch.testing.assert_close(y_det.detach(), y_eval, rtol=1e-5, atol=1e-5)
    assert cs2d.device_status() == 0


@pytest.mark.parametrize("shape,dtype", [((2, 4, 24, 16, 12, 56), torch.float32), ((1, 4, 5, 4, 6, 300), torch.bfloat16)])
def test_merged_images_are_bit_reproducible(shape, dtype):
    """deterministic=True: y and du of the four-corner operator have a single writer per element (no
    atomics): identical bits from run to run, also when the output buffers start out as garbage; and the
    values agree with the default (atomic) form."""
    b, K, d, n, h, w_ = shape
    inp = make_inputs(b, K, d, n, h, w_, dtype=dtype, seed=5)
    gen = torch.Generator().manual_seed(1)
    host = dict(u=torch.randn(b, d, h, w_, generator=gen).to(dtype), delta=inp["delta"], A=inp["A"], B=inp["B"], C=inp["C"],
                w=torch.rand(K, d, generator=gen) + 0.1, D=inp["D"], delta_bias=inp["delta_bias"])
    dy = torch.randn(b, d, h, w_, generator=gen).to(dtype).cuda()
    names = ("u", "delta", "A", "B", "C", "w", "D", "delta_bias")
    runs = []
    for _ in range(3):
        torch.empty(64 << 20, dtype=torch.uint8, device="cuda").fill_(0xFF)   # what the next buffers may reuse: NaN patterns
        dev = {k: v.cuda().requires_grad_(True) for k, v in host.items()}
        y = cs2d.cross_scan_2d(*[dev[k] for k in names], True, deterministic=True)
        y.backward(dy)
        runs.append((y.detach().clone(), dev["u"].grad.clone()))
    for y, du in runs[1:]:
        assert torch.equal(y, runs[0][0]) and torch.equal(du, runs[0][1])
    dev = {k: v.cuda().requires_grad_(True) for k, v in host.items()}
    y = cs2d.cross_scan_2d(*[dev[k] for k in names], True, deterministic=False)
    y.backward(dy)
    rtol, atol = (1e-4, 1e-5) if dtype == torch.float32 else (2e-2, 1e-3)
    check_close("y", y.detach().float().cpu().numpy(), runs[0][0].float().cpu().numpy(), rtol, atol)
    check_close("du", dev["u"].grad.float().cpu().numpy(), runs[0][1].float().cpu().numpy(), rtol, atol)
    assert torch.isfinite(runs[0][0].float()).all() and torch.isfinite(runs[0][1].float()).all()
    assert cs2d.device_status() == 0


def test_ss2d_block_training_step_matches_float64_block():
    """One training step of the SS2D block (forward, loss, gradients of every parameter and of the input)
    against the same block in float64 with the scan replaced by the oracle's restatement."""
    import copy
    from cs2d.nn import SS2D
    torch.manual_seed(3)
    m = SS2D(d_model=8, d_state=4, expand=2, directions=4).cuda()
    ref = copy.deepcopy(m).double().cpu()
    ref._scan = lambda u, delta, A, B, C, w, D, bias: O.cross_fwd_torch(u, delta, A.double(), B, C, w, D, bias, True)
    x = torch.randn(2, 6, 10, 8)
    xg, xr = x.cuda().requires_grad_(True), x.double().requires_grad_(True)
    tgt = torch.randn(2, 6, 10, 8)
    (m(xg) - tgt.cuda()).square().mean().backward()
    (ref(xr) - tgt.double()).square().mean().backward()
    # fp32 end to end through projections, convolution and LayerNorm: a block-level tolerance
    check_close("dx", xg.grad.cpu().numpy(), xr.grad.numpy(), 1e-3, 1e-5)
    got, want = dict(m.named_parameters()), dict(ref.named_parameters())
    assert set(got) == set(want)
    for name in got:
        assert got[name].grad is not None, name
        check_close("d" + name, got[name].grad.cpu().numpy(), want[name].grad.numpy(), 1e-3, 1e-5)
    assert cs2d.device_status() == 0


def test_cross_scan_with_state_decay():
    """A_decay together with the direction merge: y and every gradient against the float64 restatement;
    dA_decay against the reference's own formula (which leaves the row-scan term out), evaluated per
    direction on the flipped inputs with the direction's share w*dy of the gradient."""
    b, K, d, n, h, w_ = 2, 4, 3, 4, 6, 9
    inp = make_inputs(b, K, d, n, h, w_, seed=2, a_decay=0.9)
    gen = torch.Generator().manual_seed(9)
    u0 = torch.randn(b, d, h, w_, generator=gen)
    wt = torch.rand(K, d, generator=gen) + 0.1
    dy = torch.randn(b, d, h, w_, generator=gen)
    names = ("u", "delta", "A", "B", "C", "w", "D", "delta_bias")
    host = dict(u=u0, delta=inp["delta"], A=inp["A"], B=inp["B"], C=inp["C"], w=wt, D=inp["D"],
                delta_bias=inp["delta_bias"])
    dev = {k: v.cuda().requires_grad_(True) for k, v in host.items()}
    decay = inp["A_decay"].cuda().requires_grad_(True)
    y = cs2d.cross_scan_2d(*[dev[k] for k in names], True, decay)
    y.backward(dy.cuda())
    ref = {k: v.double().requires_grad_(True) for k, v in host.items()}
    yo = O.cross_fwd_torch(*[ref[k] for k in names], True, inp["A_decay"].double())
    yo.backward(dy.double())
    check_close("y", y.detach().cpu().numpy(), yo.detach().numpy(), 1e-4, 1e-5)
    for k in names:
        check_close("d" + k, dev[k].grad.cpu().numpy(), ref[k].grad.numpy(), 1e-4, 1e-5)
    flips = ((), (-1,), (-2,), (-2, -1))
    fl = lambda t, k: torch.flip(t, flips[k]) if flips[k] else t
    want = 0.0
    for k in range(K):
        sl = slice(k * d, (k + 1) * d)
        g = O.bwd(fl(u0, k), fl(inp["delta"][:, sl], k), inp["A"][sl], fl(inp["B"][:, k:k + 1], k),
                  fl(inp["C"][:, k:k + 1], k), inp["D"][sl], inp["delta_bias"][sl],
                  fl(dy * wt[k][None, :, None, None], k), True, inp["A_decay"])
        want = want + g["dA_decay_ref"]
    check_close("dA_decay", decay.grad.cpu().numpy(), want, 1e-4, 1e-5)
    assert cs2d.device_status() == 0


@pytest.mark.parametrize("shape,dtype,chunk", [((5, 4, 3, 4, 6, 9), torch.float32, 2), ((3, 4, 4, 16, 8, 8), torch.bfloat16, 1)])
def test_host_pipeline_of_the_four_corner_operator(shape, dtype, chunk):
    """Host buffers in, host buffers out, in batch chunks (a ragged last chunk, slots reused): the same
    values as the operator on device tensors."""
    b, K, d, n, h, w = shape
    inp = make_inputs(b, K, d, n, h, w, dtype=dtype, seed=3)
    gen = torch.Generator().manual_seed(11)
    u0 = torch.randn(b, d, h, w, generator=gen).to(dtype)
    wt = (torch.rand(K, d, generator=gen) + 0.1)
    dy = torch.randn(b, d, h, w, generator=gen).to(dtype)
    names = ("u", "delta", "A", "B", "C", "w", "D", "delta_bias")
    full = dict(u=u0, delta=inp["delta"], A=inp["A"], B=inp["B"], C=inp["C"], w=wt, D=inp["D"], delta_bias=inp["delta_bias"])
    dev = {k: v.cuda().requires_grad_(True) for k, v in full.items()}
    y = cs2d.cross_scan_2d(*[dev[k] for k in names], True)
    y.backward(dy.cuda())

    host = {"u": u0.pin_memory(), "delta": inp["delta"].pin_memory(), "B": inp["B"].pin_memory(), "C": inp["C"].pin_memory(),
            "dy": dy.pin_memory()}
    params = {"A": inp["A"].cuda(), "D": inp["D"].cuda(), "delta_bias": inp["delta_bias"].cuda(), "w": wt.cuda()}
    out = cs2d.alloc_cross_host_outputs(host["u"], host["delta"], host["B"], params["A"], True, True)
    pipe = cs2d.CrossHostPipeline(host, params, True, chunk=chunk, depth=2)
    for _ in range(2):   # the second run reuses every slot and accumulator
        pipe.run(host, out)
        torch.cuda.synchronize()
    rtol, atol = (1e-4, 1e-5) if dtype == torch.float32 else (2e-2, 1e-3)
    f = lambda t: t.detach().float().cpu().numpy()
    check_close("y", f(out["y"]), f(y), rtol, atol)
    check_close("du", f(out["du"]), f(dev["u"].grad), rtol, atol)
    check_close("ddelta", f(out["ddelta"]), f(dev["delta"].grad), rtol, atol)
    check_close("dB", f(out["dB"]), f(dev["B"].grad), rtol, atol)
    check_close("dC", f(out["dC"]), f(dev["C"].grad), rtol, atol)
    check_close("dw", f(out["dw"]), f(dev["w"].grad), rtol, atol)
    dim = K * d
    pg = out["param_grads"]
    check_close("dA", pg[:dim * n].view(dim, n).numpy(), f(dev["A"].grad), rtol, atol)
    check_close("dD", pg[dim * n:dim * n + dim].numpy(), f(dev["D"].grad), rtol, atol)
    check_close("ddelta_bias", pg[dim * n + dim:dim * n + 2 * dim].numpy(), f(dev["delta_bias"].grad), rtol, atol)
    assert cs2d.device_status() == 0
