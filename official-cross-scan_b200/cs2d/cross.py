"""Four-corner CrossScan with trainable direction-fusion weights.

The reference extension scans one orientation only (top-left origin, rows
down, columns right; an in-source TODO notes that per-group scan orders are
not implemented, ``selective_scan_fwd_kernel_oflex.cuh:140``) and expects its
caller to fold the K = 4 corner directions into the channel dimension as
``n_groups = K`` groups of flipped copies.  That caller is not part of the
reference.  This module is that caller:

    y[b, d, r, c] = sum_k w[k, d] * y_k[b, d, r, c]

where ``y_k`` is the scan of direction k (0: rows down / columns right, 1: rows
down / columns left, 2: rows up / columns right, 3: rows up / columns left)
over ``u[b, d]`` with the direction's own ``delta[b, k*D+d]``, ``A[k*D+d]``,
``B[b, k]``, ``C[b, k]``, ``D[k*D+d]``, ``delta_bias[k*D+d]``; every tensor is in
image coordinates.

All four directions run in ONE kernel launch each way.  The kernels apply the
flips as index maps while they stage tiles and write results, the K directions
read the same ``u`` (and, in the backward, the same ``dy``), and the weighted sum
over the directions happens inside the kernels as well (``cs2d_dirs.merge_w``):
the directions' CTAs add ``w*y_k`` (forward) and ``w*du_k`` (backward) onto one
fp32 image each, the other gradients are scaled by ``w`` and ``dw`` is
accumulated.  Nothing is flipped, replicated or kept per direction in memory;
rows wider than 256 columns run as column tiles like the plain operator.

Two forms of the merge.  By default the four directions of a channel tile are four
CTAs that add with fp32 atomics (the last bit of ``y`` / ``du`` depends on their
order).  With ``deterministic=True`` one CTA owns the channel tile for all K
directions and walks them one after the other, so it alone writes its part of the
merged images - stored by the first direction, read-modify-written by the others
in a fixed order: no atomics, no zero fills, bit-identical ``y`` and ``du`` from run
to run, at a quarter of the CTAs (measured 17-24 % slower on 56x56 and 128x128
maps, much slower when batch x channel tiles cannot fill the GPU).
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib, ops


def _masks(K):
    rows = sum(1 << k for k in range(K) if k % 4 in (2, 3))
    cols = sum(1 << k for k in range(K) if k % 4 in (1, 3))
    return rows, cols


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _dir_forward(u, delta, A, B, C, w, D, delta_bias, delta_softplus, keep_state=True, A_decay=None,
                 deterministic=False):
    """One launch for all directions, merged in the kernel: returns y (b, d, h, w) fp32 and the saved state
    (``None`` when ``keep_state`` is false: the forward then only holds one rolling row of state)."""
    L = _lib.lib()
    K, dim = B.size(1), A.size(0)
    p = ops._problem(u, delta, A, B, C, D, delta_bias, A_decay, delta_softplus, torch.float32, "cross_scan_fwd",
                     shared_u_dim=dim)
    rows, cols = _masks(K)
    wf = w.detach().float().contiguous()
    dirs = _lib.Dirs(rows, cols, 1, _lib.DIRS_SERIAL if deterministic else 0, wf.data_ptr(), None)
    nbytes = (L.cs2d_saved_bytes if keep_state else L.cs2d_fwd_only_scratch_bytes)(ctypes.byref(p))
    if nbytes == 0:
        raise RuntimeError(f"cs2d forward: {_lib.last_error()}")
    with torch.cuda.device(u.device):
        # reproducible form, rows of at most 256 columns: the kernel writes the merged image; otherwise it adds onto it
        alloc = torch.empty if deterministic and u.size(-1) <= 256 else torch.zeros
        out = alloc(tuple(u.shape), dtype=torch.float32, device=u.device)
        saved = torch.empty(nbytes // 4, dtype=torch.float32, device=u.device)
        rc = (L.cs2d_fwd_dir if keep_state else L.cs2d_fwd_only)(
            ctypes.byref(p), ctypes.byref(dirs), _ptr(out), out.stride(0), out.stride(1), out.stride(2), _ptr(saved),
            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    ops._raise_on(rc, "forward")
    return out, (saved if keep_state else None)


def _dir_backward(u, delta, A, B, C, w, D, delta_bias, dy, saved, delta_softplus, A_decay=None, deterministic=False):
    """dy: gradient of the merged image (b, d, h, w), input dtype or fp32, shared by the directions."""
    L = _lib.lib()
    K, dim, n = B.size(1), A.size(0), A.size(1)
    dev = u.device
    p = ops._problem(u, delta, A, B, C, D, delta_bias, A_decay, delta_softplus, dy.dtype, "cross_scan_bwd",
                     shared_u_dim=dim)
    rows, cols = _masks(K)
    wf = w.detach().float().contiguous()
    with torch.cuda.device(dev):
        alloc = torch.empty if deterministic and u.size(-1) <= 256 else torch.zeros
        du = alloc(tuple(u.shape), dtype=torch.float32, device=dev)
        dw = torch.zeros(dim, dtype=torch.float32, device=dev)
        ddelta = torch.empty(tuple(delta.shape), dtype=u.dtype, device=dev)
        total, parts = ops.param_grad_layout(dim, n, D is not None, delta_bias is not None, A_decay is not None)
        flat = torch.zeros(total, dtype=torch.float32, device=dev)
        part = lambda name: flat[parts[name][0]:parts[name][0] + parts[name][1]] if name in parts else None
        dB = torch.zeros(tuple(B.shape), dtype=torch.float32, device=dev)
        dC = torch.zeros(tuple(C.shape), dtype=torch.float32, device=dev)
        scratch = torch.empty(L.cs2d_bwd_scratch_bytes(ctypes.byref(p)) // 4, dtype=torch.float32, device=dev)
        dirs = _lib.Dirs(rows, cols, 3, _lib.DIRS_SERIAL if deterministic else 0, wf.data_ptr(), dw.data_ptr())  # u, dy shared
        rc = L.cs2d_bwd_dir(ctypes.byref(p), ctypes.byref(dirs), _ptr(dy), dy.stride(0), dy.stride(1), dy.stride(2),
                            _ptr(saved), _ptr(scratch), _ptr(du), _ptr(ddelta), _ptr(part("dA")), _ptr(dB), _ptr(dC),
                            _ptr(part("dD")), _ptr(part("ddelta_bias")), _ptr(part("dA_decay")),
                            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    ops._raise_on(rc, "backward")
    return (du.to(u.dtype), ddelta, part("dA").view(dim, n), dB.to(B.dtype), dC.to(C.dtype), dw.view(K, dim // K),
            part("dD"), part("ddelta_bias"), part("dA_decay"))


class CrossScan2D(torch.autograd.Function):
    @staticmethod
    def forward(ctx, u, delta, A, B, C, w, D=None, delta_bias=None, delta_softplus=True, A_decay=None,
                deterministic=False):
        _check_shapes(u, delta, A, B, w)
        ctx.delta_softplus, ctx.deterministic = delta_softplus, bool(deterministic)
        u, delta = u.contiguous(), delta.contiguous()   # B, C may be strided views (innermost stride 1)
        y, saved = _dir_forward(u, delta, A, B, C, w, D, delta_bias, delta_softplus, A_decay=A_decay,
                                deterministic=ctx.deterministic)
        ctx.save_for_backward(u, delta, A, B, C, D, delta_bias, w, saved, A_decay)
        return y.to(u.dtype)

    @staticmethod
    def backward(ctx, dy):
        u, delta, A, B, C, D, delta_bias, w, saved, A_decay = ctx.saved_tensors
        if dy.stride(-1) != 1:
            dy = dy.contiguous()
        du, ddelta, dA, dB, dC, dw, dD, dbias, ddecay = _dir_backward(u, delta, A, B, C, w, D, delta_bias, dy, saved,
                                                                      ctx.delta_softplus, A_decay, ctx.deterministic)
        return du, ddelta, dA, dB, dC, dw.to(w.dtype), dD, dbias, None, ddecay, None


def _check_shapes(u, delta, A, B, w):
    d, K = u.size(1), B.size(1)
    if delta.size(1) != K * d or A.size(0) != K * d or tuple(w.shape) != (K, d):
        raise RuntimeError("expected delta (b, K*D, h, w), A (K*D, n), w (K, D)")


def cross_scan_2d(u, delta, A, B, C, w, D=None, delta_bias=None, delta_softplus=True, A_decay=None,
                  deterministic=None):
    """Differentiable four-corner CrossScan; see the module docstring for shapes.  ``A_decay`` (a positive
    float32 tensor of one element) scales every state transition, as in the plain operator; its gradient
    follows the reference's formula (the row-scan term is left out there).  ``deterministic`` (default:
    ``torch.are_deterministic_algorithms_enabled()``) selects the form of the merge whose ``y`` and ``du``
    come out with the same bits on every run (one CTA walks all directions); it is slower."""
    if deterministic is None:
        deterministic = torch.are_deterministic_algorithms_enabled()
    needs_grad = torch.is_grad_enabled() and any(t is not None and t.requires_grad
                                                 for t in (u, delta, A, B, C, w, D, delta_bias, A_decay))
    if not needs_grad:  # evaluation: no saved state
        _check_shapes(u, delta, A, B, w)
        y, _ = _dir_forward(u.contiguous(), delta.contiguous(), A, B, C, w, D, delta_bias, delta_softplus,
                            keep_state=False, A_decay=A_decay, deterministic=deterministic)
        return y.to(u.dtype)
    return CrossScan2D.apply(u, delta, A, B, C, w, D, delta_bias, delta_softplus, A_decay, bool(deterministic))
