"""TEST INFRASTRUCTURE - NOT PRODUCT CODE.

Python face of the CPU restatement of the reference's 2D-CrossScan selective
scan (``kernels/selective_nd_scan`` of longlong-yu/official-cross-scan).

* ``fwd`` / ``bwd`` call the C restatement (``cs2d_oracle.c``; float64 is the
  arbiter, float32 is the timed CPU baseline).  They take the same arguments,
  in the same order and with the same meaning, as the reference's pybind
  functions ``fwd`` / ``bwd`` (``src/cusoflex/selective_scan_oflex.cpp:179-187``
  and ``:286-297``) minus the saved-state tensors.
* ``fwd_torch`` is a second, independent float64 restatement of the *forward*
  device code (``include/cusoflex/selective_scan_fwd_kernel_oflex.cuh:159-337``)
  written with differentiable torch ops; ``torch.autograd`` of it checks the
  hand-derived adjoint in the C file.

Pinning: the reference has no tests, fixtures or CPU path.  The restatement is
pinned against outputs of the reference CUDA extension itself, produced on a
B200 by ``oracle/gen_golden.py`` and stored under ``tests/golden/``.

Only tests/, the smoke check and the benchmark's CPU-baseline leg may import
this module; the product must never route through it.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "libcs2d_oracle.so")
_lib = None


class _Shape(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int) for n in (
        "batch", "dim", "nrows", "ncols", "dstate", "n_groups", "delta_dim", "delta_softplus")]


def build(force: bool = False) -> str:
    """Compile the C restatement (gcc, seconds).  Returns the library path."""
    if force or not os.path.exists(_LIB_PATH) or any(
            os.path.getmtime(os.path.join(_HERE, f)) > os.path.getmtime(_LIB_PATH)
            for f in ("cs2d_oracle.c", "cs2d_oracle_impl.h")):
        subprocess.run(["make", "-C", _HERE, "-s"], check=True)
    return _LIB_PATH


def _load():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
    return _lib


def max_threads() -> int:
    return int(_load().cs2d_oracle_max_threads())


def _np(x, dt):
    if x is None:
        return None
    if hasattr(x, "detach"):  # torch tensor
        x = x.detach().to("cpu").double().numpy() if dt == np.float64 else x.detach().to("cpu").float().numpy()
    return np.ascontiguousarray(np.asarray(x, dtype=dt))


def _ptr(a):
    return a.ctypes.data_as(ctypes.c_void_p) if a is not None else None


def _shape(u, delta, A, B, delta_softplus):
    b, dim, h, w = u.shape
    return _Shape(b, dim, h, w, A.shape[1], B.shape[1], delta.shape[1], int(bool(delta_softplus)))


def _check(u, delta, A, B, C):
    b, dim, h, w = u.shape
    n = A.shape[1]
    g = B.shape[1]
    if delta.shape != (b, delta.shape[1], h, w) or A.shape != (dim, n):
        raise ValueError("shape mismatch")
    if B.shape != (b, g, n, h, w) or C.shape != B.shape:
        raise ValueError("B/C must have shape (batch, n_groups, dstate, nrows, ncols)")
    if dim % g or dim % delta.shape[1]:
        raise ValueError("dims should be dividable by n_groups / delta_dim")
    if n > 16:
        raise ValueError("state dimension must be <= 16")


def fwd(u, delta, A, B, C, D=None, delta_bias=None, delta_softplus=False, A_decay=None,
        dtype=np.float64):
    """Forward of the restatement.  Returns ``out`` with shape of ``u``."""
    u, delta, A, B, C, D, delta_bias, A_decay = (_np(t, dtype) for t in (u, delta, A, B, C, D, delta_bias, A_decay))
    _check(u, delta, A, B, C)
    out = np.empty_like(u)
    fn = getattr(_load(), "cs2d_oracle_fwd_f64" if dtype == np.float64 else "cs2d_oracle_fwd_f32")
    sh = _shape(u, delta, A, B, delta_softplus)
    rc = fn(ctypes.byref(sh), _ptr(u), _ptr(delta), _ptr(A), _ptr(B), _ptr(C), _ptr(D), _ptr(delta_bias),
            _ptr(A_decay), _ptr(out))
    if rc != 0:
        raise RuntimeError(f"cs2d_oracle_fwd failed ({rc})")
    return out


def bwd(u, delta, A, B, C, D, delta_bias, dout, delta_softplus=False, A_decay=None,
        dtype=np.float64):
    """Backward of the restatement.

    Returns a dict with ``du, ddelta, dA, dB, dC, dD, ddelta_bias`` shaped like
    the reference's ``bwd`` results (``ddelta``/``ddelta_bias`` already reduced
    to ``delta_dim`` as ``selective_scan_oflex.cpp:433-438`` does) plus
    ``dA_decay_ref`` (the reference's value, which omits the row-scan term) and
    ``dA_decay_true`` (the analytic gradient).
    """
    u, delta, A, B, C, D, delta_bias, A_decay, dout = (
        _np(t, dtype) for t in (u, delta, A, B, C, D, delta_bias, A_decay, dout))
    _check(u, delta, A, B, C)
    b, dim, h, w = u.shape
    ddim = delta.shape[1]
    du = np.empty_like(u)
    ddelta = np.empty_like(u)
    dA = np.empty_like(A)
    dB = np.empty_like(B)
    dC = np.empty_like(C)
    dD = np.empty(dim, dtype)
    dbias = np.empty(dim, dtype)
    dr = np.zeros(1, dtype)
    dt = np.zeros(1, dtype)
    fn = getattr(_load(), "cs2d_oracle_bwd_f64" if dtype == np.float64 else "cs2d_oracle_bwd_f32")
    sh = _shape(u, delta, A, B, delta_softplus)
    rc = fn(ctypes.byref(sh), _ptr(u), _ptr(delta), _ptr(A), _ptr(B), _ptr(C), _ptr(D), _ptr(delta_bias),
            _ptr(A_decay), _ptr(dout), _ptr(du), _ptr(ddelta), _ptr(dA), _ptr(dB), _ptr(dC), _ptr(dD),
            _ptr(dbias), _ptr(dr), _ptr(dt))
    if rc != 0:
        raise RuntimeError(f"cs2d_oracle_bwd failed ({rc})")
    if ddim != dim:
        rep = dim // ddim
        ddelta = ddelta.reshape(b, ddim, rep, h, w).sum(2)
        dbias = dbias.reshape(ddim, rep).sum(1)
    return {
        "du": du, "ddelta": ddelta, "dA": dA, "dB": dB, "dC": dC,
        "dD": dD if D is not None else None,
        "ddelta_bias": dbias if delta_bias is not None else None,
        "dA_decay_ref": dr if A_decay is not None else None,
        "dA_decay_true": dt if A_decay is not None else None,
    }


def fwd_torch(u, delta, A, B, C, D=None, delta_bias=None, delta_softplus=False, A_decay=None):
    """Differentiable float64 restatement of the forward device code (small cases only).

    Follows ``selective_scan_fwd_kernel_oflex.cuh``: softplus with threshold 20
    (:221-224), ``a = exp2(dl*A*log2e)*A_decay`` (:245), the 2-D coupling
    (:263-271), the row scan ``s`` (:306-327) and the output (:227,:301,:334).
    """
    import torch
    b, dim, h, w = u.shape
    n = A.shape[1]
    g = B.shape[1]
    ddim = delta.shape[1]
    x = delta.repeat_interleave(dim // ddim, dim=1)
    if delta_bias is not None:
        x = x + delta_bias.repeat_interleave(dim // ddim)[None, :, None, None]
    dl = torch.where(x <= 20, torch.log1p(torch.exp(x)), x) if delta_softplus else x
    decay = A_decay if A_decay is not None else torch.ones(1, dtype=u.dtype)
    a = torch.exp(dl[:, :, None] * A[None, :, :, None, None]) * decay          # (b,dim,n,h,w)
    Bx = B.repeat_interleave(dim // g, dim=1)                                    # (b,dim,n,h,w)
    Cx = C.repeat_interleave(dim // g, dim=1)
    p = Bx * (dl * u)[:, :, None]
    zero = torch.zeros(b, dim, n, dtype=u.dtype)
    hs = [[None] * w for _ in range(h)]
    ss = [[None] * w for _ in range(h)]
    for r in range(h):
        for c in range(w):
            hl = hs[r][c - 1] if c > 0 else zero
            hu = hs[r - 1][c] if r > 0 else zero
            hd = hs[r - 1][c - 1] if (r > 0 and c > 0) else zero
            au = a[..., r - 1, c] if r > 0 else decay
            al = a[..., r, c - 1] if c > 0 else decay
            hs[r][c] = a[..., r, c] * (hl + hu - 0.5 * (au + al) * hd) + p[..., r, c]
            ss[r][c] = a[..., r, c] * (ss[r][c - 1] if c > 0 else zero) + p[..., r, c]
    hh = torch.stack([torch.stack(row, -1) for row in hs], -2)
    sv = torch.stack([torch.stack(row, -1) for row in ss], -2)
    y = (Cx * (hh - sv + 0.25 * p)).sum(2)
    if D is not None:
        y = y + D[None, :, None, None] * u
    return y


def cross_fwd_torch(u, delta, A, B, C, w, D=None, delta_bias=None, delta_softplus=True, A_decay=None):
    """Differentiable float64 restatement of the four-corner CrossScan with fusion weights.

    The reference has no code for the merge; the definition is: flip the inputs of
    direction k into the kernel's scan order, run the reference recurrence
    (``fwd_torch``), flip the result back, and sum the directions with ``w[k, d]``.
    Inputs are in image coordinates: u (b, D, h, w), delta (b, K*D, h, w), A (K*D, n),
    B, C (b, K, n, h, w), w (K, D).  Small cases only.
    """
    import torch
    flips = ((), (-1,), (-2,), (-2, -1))  # k: 0 none, 1 columns, 2 rows, 3 both
    fl = lambda t, k: torch.flip(t, flips[k % 4]) if flips[k % 4] else t
    b, d, h, wd = u.shape
    K = B.shape[1]
    y = 0
    for k in range(K):
        sl = slice(k * d, (k + 1) * d)
        yk = fwd_torch(fl(u, k), fl(delta[:, sl], k), A[sl], fl(B[:, k:k + 1], k), fl(C[:, k:k + 1], k),
                       None if D is None else D[sl], None if delta_bias is None else delta_bias[sl], delta_softplus,
                       A_decay)
        y = y + w[k][None, :, None, None] * fl(yk, k)
    return y
