"""``torch.library`` registration of the 2D-CrossScan selective scan.

The reference extension is a bare pybind module (``selective_scan_oflex.cpp:442-445``):
it has no dispatcher entry, no autograd formula and no shape function, so it
cannot sit inside ``torch.compile``, ``torch.export`` or fake-tensor tracing.
This module registers two dispatcher operators over ``cs2d.ops``

    cs2d::scan_fwd(u, delta, A, B, C, D?, delta_bias?, delta_softplus, out_float, A_decay?) -> (out, saved)
    cs2d::scan_bwd(u, delta, A, B, C, D?, delta_bias?, dout, saved, delta_softplus, A_decay?)
        -> (du, ddelta, dB, dC, param_grads)

with fake (shape-only) implementations and an autograd formula, and
``selective_scan_2d`` as the differentiable entry point built on them.
``saved`` is the row-checkpoint buffer (``x_v`` of ``ops.fwd``); ``param_grads``
is the flat fp32 buffer ``dA | dD | ddelta_bias | dA_decay`` described by
``ops.param_grad_layout``.  The kernels neither allocate nor synchronise, and
torch's caching allocator serves the outputs, so both operators can be recorded
into a CUDA graph once every kernel variant they use has been launched once
(the first launch of a variant sets its shared-memory attribute).
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch
from torch import Tensor

from . import _lib, ops

_DT = ops._DT


def _saved_numel(u, A, B, delta, out_float):
    """Size of the saved-state buffer from shapes alone (no device pointers needed)."""
    p = _lib.Problem()
    p.batch, p.dim, p.nrows, p.ncols = (int(s) for s in u.shape)
    p.dstate, p.n_groups, p.delta_dim = int(A.shape[1]), int(B.shape[1]), int(delta.shape[1])
    p.io_dtype = _DT[u.dtype]
    p.out_dtype = _DT[torch.float32 if out_float else u.dtype]
    # the size query validates that the tensors are present but never dereferences them:
    # fake tensors have no storage, so it gets placeholder addresses
    p.u = p.delta = p.A = p.B = p.C = 256
    nbytes = _lib.lib().cs2d_saved_bytes(ctypes.byref(p))
    if nbytes == 0:
        raise RuntimeError(f"cs2d forward: {_lib.last_error()}")
    return nbytes // 4


@torch.library.custom_op("cs2d::scan_fwd", mutates_args=(), device_types="cuda")
def scan_fwd(u: Tensor, delta: Tensor, A: Tensor, B: Tensor, C: Tensor, D: Optional[Tensor],
             delta_bias: Optional[Tensor], delta_softplus: bool, out_float: bool,
             A_decay: Optional[Tensor]) -> Tuple[Tensor, Tensor]:
    out, _, x_v, _ = ops.fwd(u, delta, A, B, C, D, delta_bias, delta_softplus, out_float, A_decay)
    return out, x_v


@scan_fwd.register_fake
def _scan_fwd_fake(u, delta, A, B, C, D, delta_bias, delta_softplus, out_float, A_decay):
    out = u.new_empty(tuple(u.shape), dtype=torch.float32 if out_float else u.dtype)
    return out, u.new_empty((_saved_numel(u, A, B, delta, out_float),), dtype=torch.float32)


@torch.library.custom_op("cs2d::scan_bwd", mutates_args=(), device_types="cuda")
def scan_bwd(u: Tensor, delta: Tensor, A: Tensor, B: Tensor, C: Tensor, D: Optional[Tensor],
             delta_bias: Optional[Tensor], dout: Tensor, saved: Tensor, delta_softplus: bool,
             A_decay: Optional[Tensor]) -> Tuple[Tensor, Tensor, Tensor, Tensor, Tensor]:
    dim, n = A.shape
    total, _ = ops.param_grad_layout(dim, n, D is not None, delta_bias is not None, A_decay is not None)
    flat = torch.zeros(total, dtype=torch.float32, device=u.device)
    du, ddelta, _, dB, dC, _, _, _ = ops.bwd(u, delta, A, B, C, D, delta_bias, dout, None, saved, delta_softplus,
                                             A_decay, None, param_grads=flat)
    return du, ddelta, dB, dC, flat


@scan_bwd.register_fake
def _scan_bwd_fake(u, delta, A, B, C, D, delta_bias, dout, saved, delta_softplus, A_decay):
    dim, n = A.shape
    total, _ = ops.param_grad_layout(dim, n, D is not None, delta_bias is not None, A_decay is not None)
    return (torch.empty_like(u, memory_format=torch.contiguous_format),
            delta.new_empty(tuple(delta.shape)), B.new_empty(tuple(B.shape)), C.new_empty(tuple(C.shape)),
            u.new_empty((total,), dtype=torch.float32))


def _setup(ctx, inputs, output):
    u, delta, A, B, C, D, delta_bias, delta_softplus, out_float, A_decay = inputs
    ctx.delta_softplus = delta_softplus
    ctx.save_for_backward(u, delta, A, B, C, D, delta_bias, A_decay, output[1])
    ctx.set_materialize_grads(False)


def _backward(ctx, dout, _dsaved):
    u, delta, A, B, C, D, delta_bias, A_decay, saved = ctx.saved_tensors
    if dout is None:
        return (None,) * 10
    if dout.stride(-1) != 1:
        dout = dout.contiguous()
    du, ddelta, dB, dC, flat = torch.ops.cs2d.scan_bwd(u, delta, A, B, C, D, delta_bias, dout, saved,
                                                       ctx.delta_softplus, A_decay)
    dim, n = A.shape
    _, parts = ops.param_grad_layout(dim, n, D is not None, delta_bias is not None, A_decay is not None)
    part = lambda name: flat[parts[name][0]:parts[name][0] + parts[name][1]] if name in parts else None
    dbias = part("ddelta_bias")
    if dbias is not None and delta.size(1) != dim:
        dbias = dbias.view(delta.size(1), dim // delta.size(1)).sum(1)
    return du, ddelta, part("dA").view(dim, n), dB, dC, part("dD"), dbias, None, None, part("dA_decay")


scan_fwd.register_autograd(_backward, setup_context=_setup)


def selective_scan_2d(u, delta, A, B, C, D=None, delta_bias=None, delta_softplus=False, out_float=False,
                      A_decay=None):
    """Differentiable scan through the dispatcher operators (traceable; same results as ``ops.selective_scan_2d``)."""
    return torch.ops.cs2d.scan_fwd(u, delta, A, B, C, D, delta_bias, delta_softplus, out_float, A_decay)[0]
