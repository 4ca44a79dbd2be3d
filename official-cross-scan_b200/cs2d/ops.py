"""Host side of the 2D-CrossScan selective scan: the reference's operator API.

``fwd`` and ``bwd`` take the same positional arguments, apply the same checks
and return the same lists as the two pybind functions of the reference
extension ``selective_nd_scan_cuda_oflex``
(``kernels/selective_nd_scan/src/cusoflex/selective_scan_oflex.cpp:179-284``
and ``:286-440``).  They allocate the outputs with torch and call the C-ABI
library on the current CUDA stream; all arithmetic happens in the CUDA
kernels, there is no PyTorch or CPU fallback.

Differences a caller can observe:
* the three saved tensors ``x, x_v, x_sd`` returned by ``fwd`` are opaque in
  the reference too; here ``x_v`` carries the row checkpoints and ``x`` /
  ``x_sd`` are empty.  ``bwd`` does not modify them (the reference overwrites
  them, so there a second ``bwd`` on the same tensors is invalid);
* ``A_decay`` must be positive.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib

_DT = {torch.float32: _lib.F32, torch.float16: _lib.F16, torch.bfloat16: _lib.BF16}
MAX_DSTATE = 16


def _check(cond, msg="check failed"):
    if not cond:
        raise RuntimeError(msg)


def _inner_ok(t):
    return t.stride(-1) == 1 or t.size(-1) == 1


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _problem(u, delta, A, B, C, D, delta_bias, A_decay, delta_softplus, out_dtype, who, shared_u_dim=None):
    input_type = u.dtype
    _check(input_type in _DT, f"{who} not implemented for input type '{input_type}'")
    _check(A.dtype == torch.float32, "A must be float32")
    _check(delta.dtype == input_type and B.dtype == input_type and C.dtype == input_type,
           "delta, B, C must have the dtype of u")
    for name, t in (("u", u), ("delta", delta), ("A", A), ("B", B), ("C", C)):
        _check(t.is_cuda, f"{name} must be a CUDA tensor")
    _check(u.dim() == 4, "u must have shape (batch_size, dim, nrows, ncols)")
    _check(_inner_ok(u) and _inner_ok(delta), "u and delta must be contiguous in the last dimension")
    batch, dim, nrows, ncols = u.shape
    if shared_u_dim is not None:  # u holds the channels of ONE group, read by all groups (cs2d_dirs)
        _check(B.dim() == 5 and dim * B.size(1) == shared_u_dim, "u must have dim / n_groups channels")
        dim = shared_u_dim
    _check(A.dim() == 2 and B.dim() == 5 and delta.dim() == 4, "A, B, delta have the wrong rank")
    dstate, n_groups, delta_dim = A.size(1), B.size(1), delta.size(1)
    _check(dim % n_groups == 0, "dims should be dividable by n_groups")
    _check(dim % delta_dim == 0, "dims should be dividable by delta_dim")
    _check(dstate <= MAX_DSTATE, f"selective_scan only supports state dimension <= {MAX_DSTATE}")
    _check(tuple(delta.shape) == (batch, delta_dim, nrows, ncols),
           "delta must have shape (batch_size, delta_dim, nrows, ncols)")
    _check(tuple(A.shape) == (dim, dstate), "A must have shape (dim, dstate)")
    if A_decay is not None:
        _check(tuple(A_decay.shape) == (1,), "A_decay must have shape (1)")
        _check(A_decay.dtype == torch.float32 and A_decay.is_cuda, "A_decay must be a float32 CUDA tensor")
    _check(tuple(B.shape) == (batch, n_groups, dstate, nrows, ncols),
           "B must have shape (batch_size, n_groups, dstate, nrows, ncols)")
    _check(_inner_ok(B), "B must be contiguous in the last dimension")
    _check(tuple(C.shape) == (batch, n_groups, dstate, nrows, ncols),
           "C must have shape (batch_size, n_groups, dstate, nrows, ncols)")
    _check(_inner_ok(C), "C must be contiguous in the last dimension")
    if D is not None:
        _check(D.dtype == torch.float32 and D.is_cuda and _inner_ok(D), "D must be a contiguous float32 CUDA tensor")
        _check(tuple(D.shape) == (dim,), "D must have shape (dim)")
    if delta_bias is not None:
        _check(delta_bias.dtype == torch.float32 and delta_bias.is_cuda and _inner_ok(delta_bias),
               "delta_bias must be a contiguous float32 CUDA tensor")
        _check(tuple(delta_bias.shape) == (delta_dim,), "delta_bias must have shape (delta_dim)")
    p = _lib.Problem()
    p.batch, p.dim, p.nrows, p.ncols = batch, dim, nrows, ncols
    p.dstate, p.n_groups, p.delta_dim = dstate, n_groups, delta_dim
    p.io_dtype, p.out_dtype, p.delta_softplus = _DT[input_type], _DT[out_dtype], int(bool(delta_softplus))
    p.u, p.u_bs, p.u_ds, p.u_hs = u.data_ptr(), u.stride(0), u.stride(1), u.stride(2)
    p.delta, p.delta_bs, p.delta_ds, p.delta_hs = delta.data_ptr(), delta.stride(0), delta.stride(1), delta.stride(2)
    p.A, p.A_ds, p.A_ns = A.data_ptr(), A.stride(0), A.stride(1)
    p.B, p.B_bs, p.B_gs, p.B_ns, p.B_hs = B.data_ptr(), B.stride(0), B.stride(1), B.stride(2), B.stride(3)
    p.C, p.C_bs, p.C_gs, p.C_ns, p.C_hs = C.data_ptr(), C.stride(0), C.stride(1), C.stride(2), C.stride(3)
    p.D = D.data_ptr() if D is not None else None
    p.delta_bias = delta_bias.data_ptr() if delta_bias is not None else None
    p.A_decay = A_decay.data_ptr() if A_decay is not None else None
    return p


def _raise_on(rc, what):
    if rc != 0:
        raise RuntimeError(f"cs2d {what} failed ({rc}): {_lib.last_error()}")


def fwd(u, delta, A, B, C, D_=None, delta_bias_=None, delta_softplus=False, out_float=False, A_decay_=None):
    """Selective nd scan forward.  Returns ``[out, x, x_v, x_sd]``."""
    L = _lib.lib()
    out_dtype = torch.float32 if out_float else u.dtype
    p = _problem(u, delta, A, B, C, D_, delta_bias_, A_decay_, delta_softplus, out_dtype, "selective_scan_fwd")
    nbytes = L.cs2d_saved_bytes(ctypes.byref(p))
    if nbytes == 0:
        raise RuntimeError(f"cs2d forward: {_lib.last_error()}")
    with torch.cuda.device(u.device):
        out = torch.empty(tuple(u.shape), dtype=out_dtype, device=u.device)
        x_v = torch.empty(nbytes // 4, dtype=torch.float32, device=u.device)
        x = torch.empty(0, dtype=torch.float32, device=u.device)
        x_sd = torch.empty(0, dtype=torch.float32, device=u.device)
        stream = torch.cuda.current_stream(u.device).cuda_stream
        rc = L.cs2d_fwd(ctypes.byref(p), _ptr(out), out.stride(0), out.stride(1), out.stride(2), _ptr(x_v),
                        ctypes.c_void_p(stream))
    _raise_on(rc, "forward")
    return [out, x, x_v, x_sd]


def fwd_only(u, delta, A, B, C, D_=None, delta_bias_=None, delta_softplus=False, out_float=False, A_decay_=None):
    """Forward that no backward will follow: returns ``out`` alone.

    Same kernels and results as ``fwd``; the state between row blocks lives in one
    rolling row per channel and state pair instead of the checkpoint buffer (a
    quarter of all h values), so evaluation needs a fraction of the memory.
    """
    L = _lib.lib()
    out_dtype = torch.float32 if out_float else u.dtype
    p = _problem(u, delta, A, B, C, D_, delta_bias_, A_decay_, delta_softplus, out_dtype, "selective_scan_fwd")
    nbytes = L.cs2d_fwd_only_scratch_bytes(ctypes.byref(p))
    if nbytes == 0:
        raise RuntimeError(f"cs2d forward: {_lib.last_error()}")
    with torch.cuda.device(u.device):
        out = torch.empty(tuple(u.shape), dtype=out_dtype, device=u.device)
        scratch = torch.empty(nbytes // 4, dtype=torch.float32, device=u.device)
        stream = torch.cuda.current_stream(u.device).cuda_stream
        rc = L.cs2d_fwd_only(ctypes.byref(p), None, _ptr(out), out.stride(0), out.stride(1), out.stride(2),
                             _ptr(scratch), ctypes.c_void_p(stream))
    _raise_on(rc, "forward")
    return out


def param_grad_layout(dim, dstate, has_D, has_bias, has_decay):
    """Offsets of the per-channel parameter gradients inside one flat fp32 buffer.

    ``[dA (dim*dstate) | dD (dim) | ddelta_bias (dim) | dA_decay (1)]`` with absent
    parts omitted.  These are the only outputs that sum over the batch, so a
    batch-sharded job all-reduces exactly this buffer (see ``cs2d.parallel``).
    Returns ``(total, {name: (offset, numel)})``.
    """
    parts, off = {}, 0
    for name, n, on in (("dA", dim * dstate, True), ("dD", dim, has_D), ("ddelta_bias", dim, has_bias),
                        ("dA_decay", 1, has_decay)):
        if on:
            parts[name] = (off, n)
            off += n
    return off, parts


def bwd(u, delta, A, B, C, D_, delta_bias_, dout, x_, x_v_, delta_softplus, A_decay_=None, x_sd_=None,
        param_grads=None, deterministic=None):
    """Selective nd scan backward.

    Returns ``[du, ddelta, dA, dB, dC, dD, ddelta_bias, dA_decay]`` with ``None``
    for the gradients of absent optional inputs.

    ``param_grads`` (not part of the reference signature) may be a zero-filled
    flat fp32 CUDA tensor of ``param_grad_layout(...)[0]`` elements; dA, dD,
    ddelta_bias and dA_decay are then views into it, so that one collective can
    reduce them across ranks without packing copies.

    ``deterministic`` (default: ``torch.are_deterministic_algorithms_enabled()``)
    selects the backward without floating-point atomics (``cs2d_bwd_det``):
    bit-identical gradients from run to run, for rows of at most 256 columns.
    """
    L = _lib.lib()
    if deterministic is None:
        deterministic = torch.are_deterministic_algorithms_enabled()
    _check(dout.is_cuda, "dout must be a CUDA tensor")
    _check(dout.dtype == u.dtype or dout.dtype == torch.float32, "dout must have the input dtype or float32")
    _check(_inner_ok(dout), "dout must be contiguous in the last dimension")
    _check(tuple(dout.shape) == tuple(u.shape), "dout must have shape (batch_size, dim, nrows, ncols)")
    p = _problem(u, delta, A, B, C, D_, delta_bias_, A_decay_, delta_softplus, dout.dtype, "selective_scan_bwd")
    _check(x_v_ is not None, "the saved state x_v returned by fwd is required")
    nbytes = L.cs2d_saved_bytes(ctypes.byref(p))
    if nbytes == 0:
        raise RuntimeError(f"cs2d backward: {_lib.last_error()}")
    _check(x_v_.is_cuda and x_v_.dtype == torch.float32 and x_v_.is_contiguous() and x_v_.numel() * 4 == nbytes,
           "x_v is not the saved state fwd returned for these inputs")
    batch, dim, nrows, ncols = u.shape
    delta_dim = delta.size(1)
    dev = u.device
    with torch.cuda.device(dev):
        du = torch.empty(tuple(u.shape), dtype=u.dtype, device=dev)
        ddelta = torch.empty(tuple(u.shape), dtype=u.dtype, device=dev)
        total, parts = param_grad_layout(dim, A.size(1), D_ is not None, delta_bias_ is not None,
                                         A_decay_ is not None)
        if param_grads is None:
            param_grads = torch.zeros(total, dtype=torch.float32, device=dev)
        _check(param_grads.is_cuda and param_grads.dtype == torch.float32 and param_grads.is_contiguous()
               and param_grads.numel() == total, "param_grads must be a flat float32 CUDA tensor of the layout size")

        def part(name):
            if name not in parts:
                return None
            off, n = parts[name]
            return param_grads[off:off + n]

        dA = part("dA").view(dim, A.size(1))
        dD, ddelta_bias, dA_decay = part("dD"), part("ddelta_bias"), part("dA_decay")
        dB = torch.zeros(tuple(B.shape), dtype=torch.float32, device=dev)
        dC = torch.zeros(tuple(C.shape), dtype=torch.float32, device=dev)
        scratch = torch.empty(L.cs2d_bwd_scratch_bytes(ctypes.byref(p)) // 4, dtype=torch.float32, device=dev)
        stream = torch.cuda.current_stream(dev).cuda_stream
        if deterministic:
            nbytes_det = L.cs2d_bwd_det_scratch_bytes(ctypes.byref(p))
            if nbytes_det == 0:
                raise RuntimeError(f"cs2d backward has no deterministic implementation for this shape: {_lib.last_error()}")
            det = torch.empty(nbytes_det // 4, dtype=torch.float32, device=dev)
            rc = L.cs2d_bwd_det(ctypes.byref(p), None, _ptr(dout), dout.stride(0), dout.stride(1), dout.stride(2),
                                _ptr(x_v_), _ptr(scratch), _ptr(det), _ptr(du), _ptr(ddelta), _ptr(dA), _ptr(dB), _ptr(dC),
                                _ptr(dD), _ptr(ddelta_bias), _ptr(dA_decay), ctypes.c_void_p(stream))
        else:
            rc = L.cs2d_bwd(ctypes.byref(p), _ptr(dout), dout.stride(0), dout.stride(1), dout.stride(2), _ptr(x_v_),
                            _ptr(scratch), _ptr(du), _ptr(ddelta), _ptr(dA), _ptr(dB), _ptr(dC), _ptr(dD),
                            _ptr(ddelta_bias), _ptr(dA_decay), ctypes.c_void_p(stream))
    _raise_on(rc, "backward")
    if dim != delta_dim:
        rep = dim // delta_dim
        ddelta = ddelta.view(batch, delta_dim, rep, nrows, ncols).sum(2)
        if ddelta_bias is not None:
            ddelta_bias = ddelta_bias.view(delta_dim, rep).sum(1)
    return [du, ddelta, dA, dB.to(B.dtype), dC.to(C.dtype), dD, ddelta_bias, dA_decay]


class SelectiveScan2D(torch.autograd.Function):
    """Autograd wrapper over ``fwd`` / ``bwd`` (the reference ships none)."""

    @staticmethod
    def forward(ctx, u, delta, A, B, C, D=None, delta_bias=None, delta_softplus=False, out_float=False,
                A_decay=None):
        out, x, x_v, x_sd = fwd(u, delta, A, B, C, D, delta_bias, delta_softplus, out_float, A_decay)
        ctx.delta_softplus = delta_softplus
        ctx.has = (D is not None, delta_bias is not None, A_decay is not None)
        ctx.save_for_backward(u, delta, A, B, C, D, delta_bias, A_decay, x, x_v, x_sd)
        return out

    @staticmethod
    def backward(ctx, dout):
        u, delta, A, B, C, D, delta_bias, A_decay, x, x_v, x_sd = ctx.saved_tensors
        if dout.stride(-1) != 1:
            dout = dout.contiguous()
        du, ddelta, dA, dB, dC, dD, dbias, ddecay = bwd(u, delta, A, B, C, D, delta_bias, dout, x, x_v,
                                                        ctx.delta_softplus, A_decay, x_sd)
        return du, ddelta, dA, dB, dC, dD, dbias, None, None, ddecay


def selective_scan_2d(u, delta, A, B, C, D=None, delta_bias=None, delta_softplus=False, out_float=False,
                      A_decay=None):
    """Differentiable 2D-CrossScan selective scan (one scan orientation; see ``fwd``).

    When nothing can ask for a gradient (``torch.no_grad()`` or no input requires one) the
    forward keeps no saved state (``fwd_only``).
    """
    if not (torch.is_grad_enabled() and any(t is not None and t.requires_grad
                                            for t in (u, delta, A, B, C, D, delta_bias, A_decay))):
        return fwd_only(u, delta, A, B, C, D, delta_bias, delta_softplus, out_float, A_decay)
    return SelectiveScan2D.apply(u, delta, A, B, C, D, delta_bias, delta_softplus, out_float, A_decay)
