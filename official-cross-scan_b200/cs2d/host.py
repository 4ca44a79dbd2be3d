"""Forward + backward for callers whose tensors live in HOST memory.

The operators in ``cs2d.ops`` take device tensors, like the reference extension
(``selective_scan_oflex.cpp:197-201`` rejects anything else).  A caller that
holds its activations in (pinned) host memory would pay three serial phases
per step: copy in, compute, copy out.  Every (batch, channel) recurrence is
independent, so ``fwd_bwd_from_host`` cuts the batch into chunks and runs them
through three streams - host-to-device copies, kernels, device-to-host copies -
so that both copy directions overlap the kernels.  The per-channel parameter
gradients, the only outputs that sum over the batch, accumulate across chunks
in one flat device buffer (``ops.param_grad_layout``) and are copied out once.
"""
from __future__ import annotations

import torch

from . import ops

_BIG = ("u", "delta", "B", "C", "dout")


def alloc_host_outputs(u, B, A, has_D, has_bias, out_float=False):
    """Pinned host buffers for every output of one forward + backward step."""
    dim, n = A.shape
    odt = torch.float32 if out_float else u.dtype
    total, _ = ops.param_grad_layout(dim, n, has_D, has_bias, False)
    pin = lambda shape, dt: torch.empty(shape, dtype=dt, pin_memory=True)
    return {"out": pin(tuple(u.shape), odt), "du": pin(tuple(u.shape), u.dtype), "ddelta": pin(tuple(u.shape), u.dtype),
            "dB": pin(tuple(B.shape), B.dtype), "dC": pin(tuple(B.shape), B.dtype), "param_grads": pin((total,), torch.float32)}


def fwd_bwd_from_host(host, params, out_host, delta_softplus=True, out_float=False, chunks=4, device=None,
                      allreduce=False):
    """One forward + backward step on host-resident data.

    host      dict of pinned CPU tensors ``u, delta, B, C, dout`` (batch first)
    params    dict of device tensors ``A`` and optionally ``D``, ``delta_bias``
    out_host  dict from ``alloc_host_outputs``; filled in place
    With ``allreduce`` the parameter gradients are summed over the ranks of the default
    process group before they are copied out (batch-sharded jobs).
    Returns ``out_host`` once every copy has been queued behind the current stream (synchronise it
    or the device before reading).  ``param_grads`` holds
    ``dA | dD | ddelta_bias`` laid out by ``ops.param_grad_layout``.
    """
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    A, D, bias = params["A"], params.get("D"), params.get("delta_bias")
    batch = host["u"].size(0)
    if host["delta"].size(1) != host["u"].size(1):
        raise RuntimeError("fwd_bwd_from_host needs delta with one channel per u channel")
    chunks = max(1, min(chunks, batch))
    dim, n = A.shape
    total, _ = ops.param_grad_layout(dim, n, D is not None, bias is not None, False)
    with torch.cuda.device(dev):
        main = torch.cuda.current_stream()
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
        flat = torch.zeros(total, dtype=torch.float32, device=dev)
        s_in.wait_stream(main)
        bounds = [(batch * i // chunks, batch * (i + 1) // chunks) for i in range(chunks)]
        staged = []
        for lo, hi in bounds:  # all copies in are queued up front; the copy engine runs ahead of the kernels
            with torch.cuda.stream(s_in):
                t = {k: host[k][lo:hi].to(dev, non_blocking=True) for k in _BIG}
                ev = torch.cuda.Event()
                ev.record(s_in)
            staged.append((t, ev))
        for (lo, hi), (t, ev) in zip(bounds, staged):
            main.wait_event(ev)
            out, x, x_v, x_sd = ops.fwd(t["u"], t["delta"], A, t["B"], t["C"], D, bias, delta_softplus, out_float, None)
            g = ops.bwd(t["u"], t["delta"], A, t["B"], t["C"], D, bias, t["dout"], x, x_v, delta_softplus, None, x_sd,
                        param_grads=flat)
            done = torch.cuda.Event()
            done.record(main)
            s_out.wait_event(done)
            with torch.cuda.stream(s_out):
                for name, src in (("out", out), ("du", g[0]), ("ddelta", g[1]), ("dB", g[3]), ("dC", g[4])):
                    out_host[name][lo:hi].copy_(src, non_blocking=True)
                    src.record_stream(s_out)
            for v in t.values():
                v.record_stream(main)
        if allreduce:
            from . import parallel
            parallel.allreduce_param_grads(flat)
        s_out.wait_stream(main)
        with torch.cuda.stream(s_out):
            out_host["param_grads"].copy_(flat, non_blocking=True)
            flat.record_stream(s_out)
        main.wait_stream(s_out)
    return out_host
