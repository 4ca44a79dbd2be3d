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
image coordinates.  The scan itself runs in the CUDA kernels (``ops.fwd`` /
``ops.bwd``, one launch for all four directions); flips and the weighted merge
are done here with torch ops for now.
"""
from __future__ import annotations

import torch

from . import ops

_FLIPS = ((), (-1,), (-2,), (-2, -1))  # k: 0 none, 1 columns, 2 rows, 3 both


def _flip(t, k):
    return torch.flip(t, _FLIPS[k % 4]) if _FLIPS[k % 4] else t


def _to_scan(t, K, per_dir):
    """(b, K*per_dir, h, w) in image coordinates -> every direction in its scan order."""
    b, _, h, w = t.shape
    v = t.view(b, K, per_dir, h, w)
    return torch.stack([_flip(v[:, k], k) for k in range(K)], 1).reshape(b, K * per_dir, h, w)


def _to_scan5(t):
    """(b, K, n, h, w) -> every direction in its scan order."""
    return torch.stack([_flip(t[:, k], k) for k in range(t.size(1))], 1)


class CrossScan2D(torch.autograd.Function):
    @staticmethod
    def forward(ctx, u, delta, A, B, C, w, D=None, delta_bias=None, delta_softplus=True):
        b, d, h, wd = u.shape
        K = B.size(1)
        if delta.size(1) != K * d or A.size(0) != K * d or tuple(w.shape) != (K, d):
            raise RuntimeError("expected delta (b, K*D, h, w), A (K*D, n), w (K, D)")
        us = torch.cat([_flip(u, k) for k in range(K)], 1).contiguous()
        ds = _to_scan(delta, K, d).contiguous()
        Bs, Cs = _to_scan5(B).contiguous(), _to_scan5(C).contiguous()
        out, x, x_v, x_sd = ops.fwd(us, ds, A, Bs, Cs, D, delta_bias, delta_softplus, True, None)
        yk = torch.stack([_flip(out[:, k * d:(k + 1) * d], k) for k in range(K)], 1)   # (b, K, d, h, w) fp32
        y = (yk * w.float()[None, :, :, None, None]).sum(1)
        ctx.save_for_backward(us, ds, A, Bs, Cs, D, delta_bias, w, yk, x, x_v, x_sd)
        ctx.delta_softplus = delta_softplus
        return y.to(u.dtype)

    @staticmethod
    def backward(ctx, dy):
        us, ds, A, Bs, Cs, D, delta_bias, w, yk, x, x_v, x_sd = ctx.saved_tensors
        b, K, d, h, wd = yk.shape
        dyf = dy.float()
        dw = (dyf[:, None] * yk).sum((0, 3, 4)).to(w.dtype)
        g = torch.cat([_flip(dyf * w.float()[k][None, :, None, None], k) for k in range(K)], 1).contiguous()
        du_s, dd_s, dA, dB_s, dC_s, dD, dbias, _ = ops.bwd(us, ds, A, Bs, Cs, D, delta_bias, g, x, x_v,
                                                           ctx.delta_softplus, None, x_sd)
        du = sum(_flip(du_s[:, k * d:(k + 1) * d].float(), k) for k in range(K)).to(us.dtype)
        ddelta = _to_scan(dd_s, K, d)          # flips are involutions: the same map goes back
        dB, dC = _to_scan5(dB_s), _to_scan5(dC_s)
        return du, ddelta, dA, dB, dC, dw, dD, dbias, None


def cross_scan_2d(u, delta, A, B, C, w, D=None, delta_bias=None, delta_softplus=True):
    """Differentiable four-corner CrossScan; see the module docstring for shapes."""
    return CrossScan2D.apply(u, delta, A, B, C, w, D, delta_bias, delta_softplus)
