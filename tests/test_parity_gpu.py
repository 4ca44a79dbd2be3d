"""CUDA kernels, called through the operator API and the C ABI, against the
golden vectors of the reference extension, the float64 oracle, and
size-independent properties at the full benchmark size."""
import numpy as np
import pytest
import torch

from conftest import TOL, check_close
import cs2d
from cs2d.synthetic import make_inputs
from oracle import cs2d_oracle as O

pytestmark = pytest.mark.gpu
NAMES = ("du", "ddelta", "dA", "dB", "dC", "dD", "ddelta_bias", "dA_decay")


def _dev(inp):
    return {k: (v.cuda() if v is not None else None) for k, v in inp.items()}


def _run(d, softplus=True, out_float=False, dout=None):
    out, x, xv, xsd = cs2d.fwd(d["u"], d["delta"], d["A"], d["B"], d["C"], d["D"], d["delta_bias"], softplus,
                               out_float, d["A_decay"])
    dout = d["dout"] if dout is None else dout
    g = cs2d.bwd(d["u"], d["delta"], d["A"], d["B"], d["C"], d["D"], d["delta_bias"], dout, x, xv, softplus,
                 d["A_decay"], xsd)
    torch.cuda.synchronize()
    assert cs2d.device_status() == 0
    return out, g, (x, xv, xsd)


def _np(t):
    return t.detach().float().cpu().numpy()


def test_loaded_library_is_the_cuda_build():
    assert cs2d.LIB_PATH.endswith("libcs2d.so") and torch.cuda.is_available()


def test_against_reference_golden_vectors(golden):
    dt = {"torch.float32": torch.float32, "torch.bfloat16": torch.bfloat16, "torch.float16": torch.float16}[
        str(golden["dtype"])]
    rtol, atol = TOL[str(golden["dtype"]).replace("torch.", "")]
    d = {}
    for k in ("u", "delta", "A", "B", "C", "D", "delta_bias", "A_decay", "dout"):
        v = golden.get("in_" + k)
        if v is None:
            d[k] = None
        else:
            t = torch.from_numpy(v)
            d[k] = (t.to(dt) if k in ("u", "delta", "B", "C", "dout") else t).cuda()
    softplus, out_float = bool(golden["softplus"]), bool(golden["out_float"])
    dout = d["dout"].float() if out_float else d["dout"]
    out, g, _ = _run(d, softplus, out_float, dout)
    assert out.dtype == (torch.float32 if out_float else dt)
    check_close("out", _np(out), golden["ref_out"], rtol, atol)
    for k, t in zip(NAMES, g):
        if "ref_" + k in golden:
            assert t is not None, k
            check_close(k, _np(t), golden["ref_" + k], rtol, atol)   # strict: no slack, no outliers
        else:
            assert t is None, k


CASES = [
    ((1, 4, 8, 4, 8, 8), torch.float32, {}),                      # the CPU-runnable correctness config
    ((2, 4, 8, 16, 56, 56), torch.float32, {}),                   # stage-1 map, dstate 16 (reference cannot run it)
    ((2, 2, 5, 3, 13, 21), torch.float32, {}),                    # ragged everything, odd dstate
    ((1, 4, 8, 4, 7, 7), torch.float32, {"a_decay": 0.9}),        # last-stage map, decay
    ((2, 4, 8, 16, 30, 100), torch.float32, {"with_D": False, "with_bias": False}),
    ((2, 4, 8, 4, 9, 14), torch.float32, {"delta_dim": 16}),      # delta shared by channel pairs
    ((2, 4, 16, 16, 28, 28), torch.bfloat16, {}),
    ((1, 4, 6, 1, 14, 14), torch.float16, {}),                    # dstate 1
    ((1, 2, 4, 16, 9, 200), torch.bfloat16, {}),                  # widest supported rows
    ((3, 1, 1, 2, 1, 1), torch.float32, {}),                      # a single pixel
    ((1, 4, 40, 16, 16, 128), torch.bfloat16, {}),                # segmentation-scale width
    ((1, 1, 70, 2, 5, 6), torch.float32, {}),                     # more channels than one CTA pass
    ((1, 2, 3, 16, 9, 300), torch.float32, {}),                   # two column tiles (256 + 44)
    ((1, 1, 2, 4, 6, 600), torch.float32, {"a_decay": 0.8}),      # three column tiles
    ((1, 4, 4, 16, 20, 336), torch.bfloat16, {}),                 # detection-scale width
]


@pytest.mark.parametrize("shape,dtype,kw", CASES, ids=[f"{s}-{str(d)[6:]}" for s, d, _ in CASES])
def test_against_float64_oracle(shape, dtype, kw):
    inp = make_inputs(*shape, dtype=dtype, seed=0, **kw)
    out, g, _ = _run(_dev(inp))
    rtol, atol = TOL[str(dtype).replace("torch.", "")]
    f = {k: (v.float() if v is not None else None) for k, v in inp.items()}
    yo = O.fwd(f["u"], f["delta"], f["A"], f["B"], f["C"], f["D"], f["delta_bias"], True, f["A_decay"])
    go = O.bwd(f["u"], f["delta"], f["A"], f["B"], f["C"], f["D"], f["delta_bias"], f["dout"], True, f["A_decay"])
    check_close("out", _np(out), yo, rtol, atol)
    for k, t in zip(NAMES, g):
        ref = go["dA_decay_ref" if k == "dA_decay" else k]
        if ref is None:
            assert t is None
            continue
        check_close(k, _np(t), ref, rtol, atol)


def test_no_softplus_out_float_and_strided_inputs():
    # without softplus delta must itself be positive (exp(delta*A) has to decay): no bias, |delta|
    inp = make_inputs(2, 2, 6, 4, 12, 20, dtype=torch.bfloat16, seed=5, with_bias=False)
    inp["delta"] = (inp["delta"].float().abs() * 0.1).to(torch.bfloat16)
    d = _dev(inp)
    # u as a channel slice of a larger tensor, B with a permuted batch/group layout
    big = torch.zeros(2, 20, 12, 20, dtype=torch.bfloat16, device="cuda")
    big[:, 3:15] = d["u"]
    d["u"] = big[:, 3:15]
    d["B"] = d["B"].transpose(0, 1).contiguous().transpose(0, 1)
    assert not d["u"].is_contiguous() and not d["B"].is_contiguous()
    out, g, _ = _run(d, softplus=False, out_float=True, dout=d["dout"].float())
    assert out.dtype == torch.float32
    f = {k: (v.float() if v is not None else None) for k, v in inp.items()}
    yo = O.fwd(f["u"], f["delta"], f["A"], f["B"], f["C"], f["D"], f["delta_bias"], False)
    go = O.bwd(f["u"], f["delta"], f["A"], f["B"], f["C"], f["D"], f["delta_bias"], f["dout"], False)
    check_close("out", _np(out), yo, 1e-4, 1e-5)  # fp32 output of bf16 inputs: only arithmetic error
    for k, t in zip(NAMES, g):
        if go.get(k) is not None:
            check_close(k, _np(t), go[k], 2e-2, 1e-3)


def test_autograd_function_matches_operator_pair():
    inp = make_inputs(1, 4, 8, 4, 8, 8, seed=0)
    d = _dev(inp)
    leaves = {k: d[k].clone().requires_grad_(True) for k in ("u", "delta", "A", "B", "C", "D", "delta_bias")}
    y = cs2d.selective_scan_2d(leaves["u"], leaves["delta"], leaves["A"], leaves["B"], leaves["C"], leaves["D"],
                               leaves["delta_bias"], True)
    y.backward(d["dout"])
    _, g, _ = _run(d)
    for k, t in zip(("u", "delta", "A", "B", "C", "D", "delta_bias"), g):
        # parameter gradients use fp32 atomics: equal up to summation order
        check_close(k, _np(leaves[k].grad), _np(t), 1e-5, 1e-6)


def test_errors_match_the_reference_conditions():
    d = _dev(make_inputs(1, 2, 4, 4, 8, 8))
    with pytest.raises(RuntimeError, match="state dimension"):
        cs2d.fwd(d["u"], d["delta"], torch.zeros(8, 17, device="cuda"), torch.zeros(1, 2, 17, 8, 8, device="cuda"),
                 torch.zeros(1, 2, 17, 8, 8, device="cuda"), None, None, True, False, None)
    with pytest.raises(RuntimeError, match="n_groups"):
        cs2d.fwd(d["u"], d["delta"], d["A"], torch.zeros(1, 3, 4, 8, 8, device="cuda"),
                 torch.zeros(1, 3, 4, 8, 8, device="cuda"), None, None, True, False, None)
    with pytest.raises(RuntimeError, match="last dimension"):
        cs2d.fwd(d["u"].transpose(2, 3), d["delta"], d["A"], d["B"], d["C"], None, None, True, False, None)


# ---- properties at the full size of the headline configuration ---------------------
@pytest.fixture(scope="module")
def full():
    inp = make_inputs(32, 4, 192, 16, 56, 56, dtype=torch.float32, seed=0)
    d = _dev(inp)
    out, g, saved = _run(d)
    return d, out, g, saved


def test_full_size_linearity_in_u(full):
    d, out, _, _ = full
    d2 = dict(d, u=d["u"] * 2.0)
    out2 = cs2d.fwd(d2["u"], d2["delta"], d2["A"], d2["B"], d2["C"], d2["D"], d2["delta_bias"], True, False, None)[0]
    torch.testing.assert_close(out2, out * 2.0, rtol=1e-5, atol=1e-5)


def test_full_size_batch_independence(full):
    d, out, g, _ = full
    sl = {k: (v[5:7].contiguous() if k in ("u", "delta", "B", "C", "dout") else v) for k, v in d.items()}
    o2, g2, _ = _run(sl)
    torch.testing.assert_close(o2, out[5:7], rtol=0, atol=0)
    torch.testing.assert_close(g2[0], g[0][5:7], rtol=0, atol=0)       # du
    torch.testing.assert_close(g2[1], g[1][5:7], rtol=0, atol=0)       # ddelta
    torch.testing.assert_close(g2[3], g[3][5:7], rtol=1e-5, atol=1e-5)  # dB (atomic order)


def test_full_size_reduction_identities(full):
    d, _, g, _ = full
    dD = (d["dout"].double() * d["u"].double()).sum((0, 2, 3))
    torch.testing.assert_close(g[5].double(), dD, rtol=1e-4, atol=1e-3)
    dbias = g[1].double().sum((0, 2, 3))
    torch.testing.assert_close(g[6].double(), dbias, rtol=1e-4, atol=1e-3)


def test_backward_does_not_modify_the_saved_state(full):
    d, _, g, (x, xv, xsd) = full
    before = xv.clone()
    g2 = cs2d.bwd(d["u"], d["delta"], d["A"], d["B"], d["C"], d["D"], d["delta_bias"], d["dout"], x, xv, True, None,
                  xsd)
    torch.cuda.synchronize()
    assert torch.equal(before, xv)
    torch.testing.assert_close(g2[0], g[0], rtol=0, atol=0)


def test_full_size_sample_against_oracle(full):
    d, out, g, _ = full
    f = lambda t: t.float().cpu()
    # two (batch, group) slabs of the full problem through the float64 oracle
    for b, k in ((0, 0), (31, 3)):
        ch = slice(k * 192, k * 192 + 6)
        u, dl, do = f(d["u"][b:b + 1, ch]), f(d["delta"][b:b + 1, ch]), f(d["dout"][b:b + 1, ch])
        Bm, Cm = f(d["B"][b:b + 1, k:k + 1]), f(d["C"][b:b + 1, k:k + 1])
        A, Dv, bias = f(d["A"][ch]), f(d["D"][ch]), f(d["delta_bias"][ch])
        yo = O.fwd(u, dl, A, Bm, Cm, Dv, bias, True)
        check_close("out", _np(out[b:b + 1, ch]), yo, 1e-4, 1e-5)
        go = O.bwd(u, dl, A, Bm, Cm, Dv, bias, do, True)
        check_close("du", _np(g[0][b:b + 1, ch]), go["du"], 1e-4, 1e-5)
        check_close("ddelta", _np(g[1][b:b + 1, ch]), go["ddelta"], 1e-4, 1e-5)


# At the full size both the reference extension and this library leave the strict tolerance on the
# worst of 1e6..2e7 elements and on sums over 1e5 fp32 terms, by 1.1x-1.7x (measured on a B200 against
# the float64 oracle by oracle/ref_reduction_error.py: reference up to 1.73x, this library up to 1.54x at
# B32 D192 N12 56x56).  The full-size checks therefore allow a bounded excess - and nothing else does.
FULL = dict(outlier_frac=1e-5, outlier_factor=4.0)        # element tensors
FULL_SUM = dict(outlier_frac=0.03, outlier_factor=4.0)    # per-channel sums over batch * H * W terms


def test_full_size_channel_sums_against_oracle(full):
    """dB / dC of the full problem are sums over the 192 channels of a group: one whole
    (batch, group) slab through the float64 oracle."""
    d, out, g, _ = full
    f = lambda t: t.float().cpu()
    b, k = 17, 2
    ch = slice(k * 192, (k + 1) * 192)
    go = O.bwd(f(d["u"][b:b + 1, ch]), f(d["delta"][b:b + 1, ch]), f(d["A"][ch]), f(d["B"][b:b + 1, k:k + 1]),
               f(d["C"][b:b + 1, k:k + 1]), f(d["D"][ch]), f(d["delta_bias"][ch]), f(d["dout"][b:b + 1, ch]), True)
    check_close("dB", _np(g[3][b:b + 1, k:k + 1]), go["dB"], 1e-4, 1e-5, **FULL)
    check_close("dC", _np(g[4][b:b + 1, k:k + 1]), go["dC"], 1e-4, 1e-5, **FULL)
    check_close("du", _np(g[0][b:b + 1, ch]), go["du"], 1e-4, 1e-5, **FULL)
    check_close("ddelta", _np(g[1][b:b + 1, ch]), go["ddelta"], 1e-4, 1e-5, **FULL)


def test_full_size_batch_sums_against_oracle(full):
    """dA / dD / ddelta_bias of the full problem are sums over all 32 samples and 3136 pixels: one
    whole group (192 channels, every sample) through the float64 oracle."""
    d, out, g, _ = full
    f = lambda t: t.float().cpu()
    k = 1
    ch = slice(k * 192, (k + 1) * 192)
    go = O.bwd(f(d["u"][:, ch]), f(d["delta"][:, ch]), f(d["A"][ch]), f(d["B"][:, k:k + 1]), f(d["C"][:, k:k + 1]),
               f(d["D"][ch]), f(d["delta_bias"][ch]), f(d["dout"][:, ch]), True)
    check_close("dA", _np(g[2][ch]), go["dA"], 1e-4, 1e-5, **FULL_SUM)
    check_close("dD", _np(g[5][ch]), go["dD"], 1e-4, 1e-5, **FULL_SUM)
    check_close("ddelta_bias", _np(g[6][ch]), go["ddelta_bias"], 1e-4, 1e-5, **FULL_SUM)
    check_close("dB", _np(g[3][:, k:k + 1]), go["dB"], 1e-4, 1e-5, **FULL)
    check_close("dC", _np(g[4][:, k:k + 1]), go["dC"], 1e-4, 1e-5, **FULL)


# ---- every benchmark configuration at its own feature-map shape (batch reduced to 1) --------------
from cs2d.synthetic import CONFIGS  # noqa: E402


@pytest.mark.parametrize("name", [n for n in CONFIGS if not n.startswith(("c1", "c2"))])
def test_benchmark_config_shapes_against_oracle(name):
    _, K, D, N, H, W, dtype = CONFIGS[name]
    inp = make_inputs(1, K, D, N, H, W, dtype=dtype, seed=3)
    d = _dev(inp)
    out, g, _ = _run(d)
    rtol, atol = TOL[str(dtype).replace("torch.", "")]
    f = lambda t: t.float().cpu()
    # three channels of the first and of the last direction through the float64 oracle; B/C
    # gradients are sums over all D channels of a group, so they are checked on a group that is
    # fed only those channels (a second, smaller call)
    for k in (0, K - 1):
        ch = slice(k * D, k * D + 3)
        u, dl, do = f(d["u"][:, ch]), f(d["delta"][:, ch]), f(d["dout"][:, ch])
        Bm, Cm = f(d["B"][:, k:k + 1]), f(d["C"][:, k:k + 1])
        A, Dv, bias = f(d["A"][ch]), f(d["D"][ch]), f(d["delta_bias"][ch])
        yo = O.fwd(u, dl, A, Bm, Cm, Dv, bias, True)
        go = O.bwd(u, dl, A, Bm, Cm, Dv, bias, do, True)
        check_close("out", _np(out[:, ch]), yo, rtol, atol)
        check_close("du", _np(g[0][:, ch]), go["du"], rtol, atol)
        check_close("ddelta", _np(g[1][:, ch]), go["ddelta"], rtol, atol)
        check_close("dA", _np(g[2][ch]), go["dA"], rtol, atol)
        sub = {kk: (v[:, ch].contiguous() if kk in ("u", "delta", "dout") else v) for kk, v in d.items()}
        sub.update(A=d["A"][ch].contiguous(), D=d["D"][ch].contiguous(), delta_bias=d["delta_bias"][ch].contiguous(),
                   B=d["B"][:, k:k + 1].contiguous(), C=d["C"][:, k:k + 1].contiguous())
        _, g3, _ = _run(sub)
        check_close("dB", _np(g3[3]), go["dB"], rtol, atol)
        check_close("dC", _np(g3[4]), go["dC"], rtol, atol)


@pytest.mark.parametrize("shape,dtype", [((2, 4, 6, 16, 21, 40), torch.float32), ((1, 2, 5, 3, 13, 300), torch.float32),
                                         ((2, 4, 40, 16, 14, 14), torch.bfloat16), ((2, 2, 3, 1, 9, 9), torch.float16)])
def test_forward_only_equals_forward(shape, dtype):
    """The forward that keeps no saved state (rolling row) returns bit-identical results."""
    inp = make_inputs(*shape, dtype=dtype, seed=6)
    dev = {k: (v.cuda() if v is not None else None) for k, v in inp.items()}
    args = (dev["u"], dev["delta"], dev["A"], dev["B"], dev["C"], dev["D"], dev["delta_bias"], True, False, None)
    full = cs2d.fwd(*args)[0]
    only = cs2d.fwd_only(*args)
    assert torch.equal(full, only)
    with torch.no_grad():
        assert torch.equal(cs2d.selective_scan_2d(*args), full)
    assert cs2d.device_status() == 0


@pytest.mark.parametrize("shape,dtype,kw", [((4, 4, 48, 16, 21, 40), torch.float32, {}),
                                            ((2, 4, 6, 5, 9, 60), torch.bfloat16, {"a_decay": 0.9}), ((2, 4, 5, 16, 9, 200), torch.float32, {}),
                                            ((3, 2, 40, 1, 14, 14), torch.float32, {"delta_dim": 20})])
def test_deterministic_backward_is_bit_reproducible(shape, dtype, kw):
    """cs2d_bwd_det: same bits on every run, same values as the atomic backward within tolerance."""
    inp = make_inputs(*shape, dtype=dtype, seed=8, **kw)
    dev = {k: (v.cuda() if v is not None else None) for k, v in inp.items()}
    o = cs2d.fwd(dev["u"], dev["delta"], dev["A"], dev["B"], dev["C"], dev["D"], dev["delta_bias"], True, False,
                 dev["A_decay"])
    run = lambda det: cs2d.bwd(dev["u"], dev["delta"], dev["A"], dev["B"], dev["C"], dev["D"], dev["delta_bias"],
                               dev["dout"], o[1], o[2], True, dev["A_decay"], o[3], deterministic=det)
    a, b2, c = run(True), run(True), run(False)
    rtol, atol = TOL[str(dtype)[6:]]
    for name, x, y, z in zip(("du", "ddelta", "dA", "dB", "dC", "dD", "ddelta_bias", "dA_decay"), a, b2, c):
        assert (x is None) == (z is None), name
        if x is None:
            continue
        assert torch.equal(x, y), f"{name} differs between two deterministic runs"
        # two fp32 results with different summation orders: same tolerance as against the oracle
        check_close(name, x.float().cpu().numpy(), z.float().cpu().numpy(), rtol, atol)
    with pytest.raises(RuntimeError, match="deterministic"):
        wide = make_inputs(1, 1, 2, 2, 4, 300, seed=1)
        wd = {k: (v.cuda() if v is not None else None) for k, v in wide.items()}
        ow = cs2d.fwd(wd["u"], wd["delta"], wd["A"], wd["B"], wd["C"], wd["D"], wd["delta_bias"], True, False, None)
        cs2d.bwd(wd["u"], wd["delta"], wd["A"], wd["B"], wd["C"], wd["D"], wd["delta_bias"], wd["dout"], ow[1], ow[2],
                 True, None, ow[3], deterministic=True)
    assert cs2d.device_status() == 0
