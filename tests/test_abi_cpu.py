"""The C-ABI library without a GPU: it loads, exports what include/cs2d.h
declares, validates arguments before touching CUDA, and the Python operators
fail loudly instead of falling back."""
import ctypes
import os
import re

import pytest
import torch

from conftest import ROOT
import cs2d
from cs2d import _lib, ops


def _declared():
    text = open(os.path.join(ROOT, "include", "cs2d.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(cs2d_[a-z_0-9]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(_lib.LIB_PATH)
    names = _declared()
    assert {"cs2d_fwd", "cs2d_bwd", "cs2d_saved_bytes", "cs2d_bwd_scratch_bytes", "cs2d_last_error",
            "cs2d_abi_version", "cs2d_launch_count", "cs2d_device_status"} <= set(names)
    for n in names:
        assert hasattr(lib, n), n
    assert _lib.lib().cs2d_abi_version() == 2


def _problem(**over):
    p = _lib.Problem()
    p.batch, p.dim, p.nrows, p.ncols, p.dstate, p.n_groups, p.delta_dim = 2, 8, 56, 56, 16, 4, 8
    p.io_dtype, p.out_dtype, p.delta_softplus = _lib.F32, _lib.F32, 1
    for k in ("u", "delta", "A", "B", "C"):
        setattr(p, k, 16)  # never dereferenced: validation and sizing only
    for k, v in over.items():
        setattr(p, k, v)
    return p


def test_sizes_without_gpu():
    L = _lib.lib()
    p = _problem()
    # 14 row blocks x 8 pair slots x 64 padded columns x 8 bytes per (batch, channel); rows of at most 64
    # columns with more than 8 states also keep B and C regrouped in fp32 entries of four states
    # (batch x groups x rows x 4 entries x columns x 16 bytes, twice) for the row-walk forward
    bc = 2 * (2 * 4 * 56 * 4 * 56 * 16)
    assert L.cs2d_saved_bytes(ctypes.byref(p)) == 2 * 8 * 14 * 8 * 64 * 8 + bc
    assert L.cs2d_bwd_scratch_bytes(ctypes.byref(p)) == 2 * 8 * 8 * 64 * 8
    p1 = _problem(dstate=1, nrows=7, ncols=7)
    assert L.cs2d_saved_bytes(ctypes.byref(p1)) == 2 * 8 * 2 * 1 * 8 * 8
    # 336 columns = five 64-column tiles + a 16-column tile, and one edge buffer per tile boundary
    pw = _problem(ncols=336)
    per = 2 * 8 * 8 * 8  # batch x dim x pair slots x bytes per float2
    edge = 2 * 8 * 8 * 56 * 16
    assert L.cs2d_saved_bytes(ctypes.byref(pw)) == per * 14 * (5 * 64 + 16) + 5 * edge
    assert L.cs2d_bwd_scratch_bytes(ctypes.byref(pw)) == per * (5 * 64 + 16) + 5 * edge
    # deterministic backward: per-channel-tile dB/dC planes + per-batch parameter slots + one slot per CTA
    det = L.cs2d_bwd_det_scratch_bytes(ctypes.byref(p))
    nB, slots = 2 * 4 * 16 * 56 * 56, 2 * 8 * (16 + 2)
    assert det > 0 and (det // 4 - slots) % (2 * nB) in range(0, 2 * 8 * 4 + 1)
    assert L.cs2d_bwd_det_scratch_bytes(ctypes.byref(pw)) == 0   # wider than one column tile
    # a forward that no backward follows keeps one rolling row instead of 14 checkpoints
    assert L.cs2d_fwd_only_scratch_bytes(ctypes.byref(p)) == 2 * 8 * 8 * 64 * 8 + bc
    assert L.cs2d_fwd_only_scratch_bytes(ctypes.byref(pw)) == per * (5 * 64 + 16) + 5 * edge


@pytest.mark.parametrize("over,msg", [
    (dict(dstate=17), "state dimension"),
    (dict(n_groups=3), "n_groups"),
    (dict(delta_dim=3), "delta_dim"),
    (dict(io_dtype=7), "input type"),
    (dict(io_dtype=_lib.F32, out_dtype=_lib.BF16), "out/dout"),
    (dict(u=None), "must be given"),
])
def test_validation_happens_before_any_cuda_call(over, msg):
    L = _lib.lib()
    p = _problem(**over)
    assert L.cs2d_saved_bytes(ctypes.byref(p)) == 0
    assert msg in _lib.last_error()
    rc = L.cs2d_fwd(ctypes.byref(p), ctypes.c_void_p(16), 1, 1, 1, ctypes.c_void_p(16), None)
    assert rc in (-1, -2)


def test_null_outputs_rejected():
    L = _lib.lib()
    p = _problem()
    assert L.cs2d_fwd(ctypes.byref(p), None, 1, 1, 1, None, None) == -1
    assert L.cs2d_bwd(ctypes.byref(p), None, 1, 1, 1, None, None, None, None, None, None, None, None, None, None,
                      None) == -1


def test_operators_reject_cpu_tensors_and_bad_arguments():
    u = torch.zeros(1, 4, 8, 8)
    A = torch.zeros(4, 2)
    B = torch.zeros(1, 2, 2, 8, 8)
    with pytest.raises(RuntimeError, match="CUDA"):
        cs2d.fwd(u, u, A, B, B, None, None, True, False, None)
    with pytest.raises(RuntimeError, match="float32"):
        cs2d.fwd(u, u, A.double(), B, B, None, None, True, False, None)
    with pytest.raises(RuntimeError, match="dtype of u"):
        cs2d.fwd(u, u.half(), A, B, B, None, None, True, False, None)


def test_missing_library_is_an_error_not_a_fallback(monkeypatch):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/libcs2d.so")
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _lib.lib()


def test_drop_in_module_name():
    import selective_nd_scan_cuda_oflex as ext
    assert ext.fwd is ops.fwd and ext.bwd is ops.bwd


def test_abi_version_is_consistent_everywhere():
    """The header, the Python binding and the build entry point name the same ABI version."""
    header = open(os.path.join(ROOT, "include", "cs2d.h")).read()
    version = int(re.search(r"#define CS2D_ABI_VERSION (\d+)", header).group(1))
    assert _lib.lib().cs2d_abi_version() == version
    binding = open(os.path.join(ROOT, "official-cross-scan_b200", "cs2d", "_lib.py")).read()
    assert f"cs2d_abi_version() != {version}" in binding
    entry = open(os.path.join(ROOT, "__graft_entry__.py")).read()
    assert f"cs2d_abi_version() == {version}" in entry
