"""The allocation-free backward entry point (collected last on purpose).

``cs2d_bwd_noalloc`` is for hosts that cannot call ``cudaMalloc`` where they run
the backward - a runtime whose own pool owns all device memory, a plugin called
from an allocator callback, an FFI stub that only sees its arguments.  Its
scratch is a fixed array inside the library.  Here it is called straight through
the C ABI, twice in a row, and must reproduce what ``cs2d_bwd`` computes with a
caller-allocated scratch buffer; oversized problems must be refused with a
message rather than overrun the array.
"""
import ctypes

import pytest
import torch

from conftest import check_close
import cs2d
from cs2d import _lib, ops
from cs2d.synthetic import make_inputs


def _buffers(d, dim, n):
    z = lambda *s: torch.zeros(*s, dtype=torch.float32, device="cuda")
    return {"du": torch.empty_like(d["u"]), "ddelta": torch.empty_like(d["u"]), "dA": z(dim, n),
            "dB": z(*d["B"].shape), "dC": z(*d["C"].shape), "dD": z(dim), "dbias": z(dim)}


def _call(entry, p, d, xv, o, scratch=None):
    vp = lambda t: ctypes.c_void_p(t.data_ptr())
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    head = [ctypes.byref(p), vp(d["dout"]), d["dout"].stride(0), d["dout"].stride(1), d["dout"].stride(2), vp(xv)]
    if scratch is not None:
        head.append(vp(scratch))
    rc = entry(*head, vp(o["du"]), vp(o["ddelta"]), vp(o["dA"]), vp(o["dB"]), vp(o["dC"]), vp(o["dD"]),
               vp(o["dbias"]), None, stream)
    torch.cuda.synchronize()
    return rc


@pytest.mark.gpu
@pytest.mark.parametrize("shape,dtype", [((2, 4, 8, 16, 56, 56), torch.float32), ((3, 2, 6, 4, 9, 14), torch.bfloat16)])
def test_noalloc_matches_bwd_twice_in_a_row(shape, dtype):
    L = _lib.lib()
    inp = make_inputs(*shape, dtype=dtype, seed=11)
    d = {k: (v.cuda() if v is not None else None) for k, v in inp.items()}
    dim, n = d["A"].shape
    out, x, xv, xsd = cs2d.fwd(d["u"], d["delta"], d["A"], d["B"], d["C"], d["D"], d["delta_bias"], True, False, None)
    p = ops._problem(d["u"], d["delta"], d["A"], d["B"], d["C"], d["D"], d["delta_bias"], None, True, dtype, "test")
    need = L.cs2d_bwd_scratch_bytes(ctypes.byref(p))
    assert 0 < need <= _lib.NOALLOC_SCRATCH_BYTES
    ref = _buffers(d, dim, n)
    scratch = torch.empty(need // 4, dtype=torch.float32, device="cuda")
    assert _call(L.cs2d_bwd, p, d, xv, ref, scratch) == 0, _lib.last_error()
    rtol, atol = (1e-4, 1e-5) if dtype == torch.float32 else (2e-2, 1e-3)
    for attempt in range(2):  # the second call finds the array as the first one left it
        got = _buffers(d, dim, n)
        assert _call(L.cs2d_bwd_noalloc, p, d, xv, got) == 0, _lib.last_error()
        assert cs2d.device_status() == 0
        for k in ("du", "ddelta"):  # no atomics on this path: identical
            assert torch.equal(got[k], ref[k]), (k, attempt)
        for k in ("dA", "dB", "dC", "dD", "dbias"):  # fp32 atomics: equal up to summation order
            check_close(f"{k}[{attempt}]", got[k].cpu().numpy(), ref[k].cpu().numpy(), rtol, atol * 10)


@pytest.mark.gpu
def test_noalloc_refuses_what_does_not_fit():
    L = _lib.lib()
    # 32 x 768 channels x 8 state pairs x 64 padded columns x 8 bytes = 96 MiB of scratch
    d = {k: (v.cuda() if v is not None else None) for k, v in make_inputs(1, 4, 8, 16, 56, 56).items()}
    p = ops._problem(d["u"], d["delta"], d["A"], d["B"], d["C"], d["D"], d["delta_bias"], None, True, torch.float32,
                     "test")
    p.batch, p.dim = 32, 768
    assert L.cs2d_bwd_scratch_bytes(ctypes.byref(p)) > _lib.NOALLOC_SCRATCH_BYTES
    one = ctypes.c_void_p(d["u"].data_ptr())  # never dereferenced: the size check comes first
    rc = L.cs2d_bwd_noalloc(ctypes.byref(p), one, 1, 1, 1, one, one, one, one, one, one, None, None, None, None)
    assert rc == -2 and "built-in buffer holds" in _lib.last_error()
