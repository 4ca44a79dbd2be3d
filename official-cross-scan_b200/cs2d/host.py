"""Forward + backward for callers whose tensors live in HOST memory.

The operators in ``cs2d.ops`` take device tensors, like the reference extension
(``selective_scan_oflex.cpp:197-201`` rejects anything else).  A caller that
holds its activations in (pinned) host memory would pay three serial phases
per step: copy in, compute, copy out.  Every (batch, channel) recurrence is
independent, so ``HostPipeline`` cuts the batch into chunks and runs them
through three streams - host-to-device copies, kernels, device-to-host copies -
so that both copy directions overlap the kernels.  The per-channel parameter
gradients, the only outputs that sum over the batch, accumulate across chunks
in one flat device buffer (``ops.param_grad_layout``) and are copied out once.

All device buffers are allocated once, as a ring of ``depth`` chunk slots, and
the kernels are called through the C ABI on them: a step allocates nothing, so
its timing does not depend on the state of torch's caching allocator.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib, ops

_BIG = ("u", "delta", "B", "C", "dout")


def alloc_host_outputs(u, B, A, has_D, has_bias, out_float=False):
    """Pinned host buffers for every output of one forward + backward step."""
    dim, n = A.shape
    odt = torch.float32 if out_float else u.dtype
    total, _ = ops.param_grad_layout(dim, n, has_D, has_bias, False)
    pin = lambda shape, dt: torch.empty(shape, dtype=dt, pin_memory=True)
    return {"out": pin(tuple(u.shape), odt), "du": pin(tuple(u.shape), u.dtype), "ddelta": pin(tuple(u.shape), u.dtype),
            "dB": pin(tuple(B.shape), B.dtype), "dC": pin(tuple(B.shape), B.dtype), "param_grads": pin((total,), torch.float32)}


def _auto_chunk(host, batch):
    """Samples per chunk: about 32 MB of input, at most 64 chunks.

    The last chunk's kernels and copy-out are overlapped by nothing, so short chunks win as long as
    the per-chunk launch work stays hidden: on B32 K4 D192 N16 56x56 fp32 (0.98 GB each way; the two
    copies alone take 19.6-21 ms on a PCIe 5 x16 link) 32 chunks took 23.4 ms, 16 chunks 25.1 ms,
    4 chunks 28.1 ms.
    """
    per_sample = sum(host[k][0].numel() * host[k].element_size() for k in _BIG)
    chunks = min(64, max(1, round(batch * per_sample / 32e6)))
    return -(-batch // chunks)


class HostPipeline:
    """Preallocated three-stream pipeline for one problem shape; see the module docstring."""

    def __init__(self, host, params, delta_softplus=True, out_float=False, chunk=None, depth=3, device=None):
        self.dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.A, self.D, self.bias = params["A"], params.get("D"), params.get("delta_bias")
        self.softplus, self.out_float = delta_softplus, out_float
        u, B = host["u"], host["B"]
        if host["delta"].size(1) != u.size(1):
            raise RuntimeError("the host pipeline needs delta with one channel per u channel")
        self.batch = u.size(0)
        self.chunk = max(1, min(chunk or _auto_chunk(host, self.batch), self.batch))
        self.key = _key(host, self.chunk, delta_softplus, out_float, params)
        dim, n = self.A.shape
        self.total, self.parts = ops.param_grad_layout(dim, n, self.D is not None, self.bias is not None, False)
        c, dev = self.chunk, self.dev
        odt = torch.float32 if out_float else u.dtype
        with torch.cuda.device(dev):
            self.flat = torch.zeros(self.total, dtype=torch.float32, device=dev)
            self.s_in, self.s_out = torch.cuda.Stream(), torch.cuda.Stream()
            mk = lambda ref, dt=None: torch.empty((c,) + tuple(ref.shape[1:]), dtype=dt or ref.dtype, device=dev)
            self.slots = []
            for _ in range(max(2, depth)):
                s = {k: mk(host[k]) for k in _BIG}
                s.update(out=mk(u, odt), du=mk(u), ddelta=mk(u), dB32=mk(B, torch.float32), dC32=mk(B, torch.float32))
                if B.dtype != torch.float32:
                    s.update(dB=mk(B), dC=mk(B))
                s["free"], s["loaded"], s["done"] = torch.cuda.Event(), torch.cuda.Event(), torch.cuda.Event()
                self.slots.append(s)
            # saved state and backward scratch are sized for a full chunk
            s0 = self.slots[0]
            p = ops._problem(s0["u"], s0["delta"], self.A, s0["B"], s0["C"], self.D, self.bias, None, delta_softplus, odt,
                             "host pipeline")
            L = _lib.lib()
            nsaved, nscr = L.cs2d_saved_bytes(ctypes.byref(p)), L.cs2d_bwd_scratch_bytes(ctypes.byref(p))
            if nsaved == 0 or nscr == 0:
                raise RuntimeError(f"cs2d host pipeline: {_lib.last_error()}")
            for s in self.slots:
                s["saved"] = torch.empty(nsaved // 4, dtype=torch.float32, device=dev)
                s["scratch"] = torch.empty(nscr // 4, dtype=torch.float32, device=dev)

    def _part(self, name):
        if name not in self.parts:
            return None
        off, n = self.parts[name]
        return self.flat[off:off + n]

    def run(self, host, out_host, allreduce=False):
        """One forward + backward step; returns ``out_host`` with every copy queued behind the current stream."""
        L = _lib.lib()
        vp = lambda t: ctypes.c_void_p(t.data_ptr()) if t is not None else None
        odt = torch.float32 if self.out_float else host["u"].dtype
        with torch.cuda.device(self.dev):
            main = torch.cuda.current_stream()
            stream = ctypes.c_void_p(main.cuda_stream)
            self.flat.zero_()
            self.s_in.wait_stream(main)
            nslots = len(self.slots)
            bounds = [(lo, min(lo + self.chunk, self.batch)) for lo in range(0, self.batch, self.chunk)]
            for i, (lo, hi) in enumerate(bounds):
                s, n = self.slots[i % nslots], hi - lo
                with torch.cuda.stream(self.s_in):
                    if i >= nslots:
                        self.s_in.wait_event(s["free"])     # the slot's previous results have left the device
                    for k in _BIG:
                        s[k][:n].copy_(host[k][lo:hi], non_blocking=True)
                    s["loaded"].record(self.s_in)
                main.wait_event(s["loaded"])
                if i >= nslots:
                    main.wait_event(s["free"])
                t = {k: s[k][:n] for k in _BIG + ("out", "du", "ddelta", "dB32", "dC32")}
                p = ops._problem(t["u"], t["delta"], self.A, t["B"], t["C"], self.D, self.bias, None, self.softplus, odt,
                                 "host pipeline")
                rc = L.cs2d_fwd(ctypes.byref(p), vp(t["out"]), t["out"].stride(0), t["out"].stride(1), t["out"].stride(2),
                                vp(s["saved"]), stream)
                ops._raise_on(rc, "forward")
                t["dB32"].zero_()
                t["dC32"].zero_()
                p.out_dtype = ops._DT[t["dout"].dtype]
                rc = L.cs2d_bwd(ctypes.byref(p), vp(t["dout"]), t["dout"].stride(0), t["dout"].stride(1),
                                t["dout"].stride(2), vp(s["saved"]), vp(s["scratch"]), vp(t["du"]), vp(t["ddelta"]),
                                vp(self._part("dA")), vp(t["dB32"]), vp(t["dC32"]), vp(self._part("dD")),
                                vp(self._part("ddelta_bias")), None, stream)
                ops._raise_on(rc, "backward")
                dB, dC = t["dB32"], t["dC32"]
                if "dB" in s:   # 16-bit inputs: dB, dC leave in the input type, like the reference's cast
                    dB, dC = s["dB"][:n], s["dC"][:n]
                    dB.copy_(t["dB32"])
                    dC.copy_(t["dC32"])
                s["done"].record(main)
                with torch.cuda.stream(self.s_out):
                    self.s_out.wait_event(s["done"])
                    for name, src in (("out", t["out"]), ("du", t["du"]), ("ddelta", t["ddelta"]), ("dB", dB), ("dC", dC)):
                        out_host[name][lo:hi].copy_(src, non_blocking=True)
                    s["free"].record(self.s_out)
            if allreduce:
                from . import parallel
                parallel.allreduce_param_grads(self.flat)
            out_host["param_grads"].copy_(self.flat, non_blocking=True)
            main.wait_stream(self.s_out)
        return out_host


def _key(host, chunk, delta_softplus, out_float, params):
    return (tuple(host["u"].shape), tuple(host["B"].shape), host["u"].dtype, host["dout"].dtype, chunk,
            bool(delta_softplus), bool(out_float), params.get("D") is not None, params.get("delta_bias") is not None)


_cache = {}


def fwd_bwd_from_host(host, params, out_host, delta_softplus=True, out_float=False, chunks=None, device=None,
                      allreduce=False):
    """One forward + backward step on host-resident data.

    host      dict of pinned CPU tensors ``u, delta, B, C, dout`` (batch first)
    chunks    number of batch chunks, or None: chunks of about 32 MB of input (at most 64)
    params    dict of device tensors ``A`` and optionally ``D``, ``delta_bias``
    out_host  dict from ``alloc_host_outputs``; filled in place
    With ``allreduce`` the parameter gradients are summed over the ranks of the default
    process group before they are copied out (batch-sharded jobs).
    Returns ``out_host`` once every copy has been queued behind the current stream (synchronise it
    or the device before reading).  ``param_grads`` holds
    ``dA | dD | ddelta_bias`` laid out by ``ops.param_grad_layout``.
    The device buffers of the last shape used are kept (``HostPipeline``).
    """
    batch = host["u"].size(0)
    chunk = _auto_chunk(host, batch) if chunks is None else -(-batch // max(1, min(int(chunks), batch)))
    pipe = _cache.get("pipe")
    if pipe is None or pipe.key != _key(host, chunk, delta_softplus, out_float, params) or pipe.A is not params["A"] \
            or pipe.D is not params.get("D") or pipe.bias is not params.get("delta_bias"):
        _cache.clear()
        pipe = HostPipeline(host, params, delta_softplus, out_float, chunk, device=device)
        _cache["pipe"] = pipe
    return pipe.run(host, out_host, allreduce)


# ---- the four-corner operator on host-resident data ---------------------------------------------------
# Through the drop-in operator a caller with K = 4 corner directions moves u, out, dout and du with K*D
# channels although the four groups of u are flips of one image.  The four-corner operator takes the
# image once: (2 + K)*D + 2*K*N values per pixel in, (2 + K)*D + 2*K*N out, instead of 3*K*D + 2*K*N
# each way (53 % of the bytes at K4 D192 N16).
_XBIG = ("u", "delta", "B", "C", "dy")


def alloc_cross_host_outputs(u, delta, B, A, has_D, has_bias):
    """Pinned host buffers for every output of one four-corner forward + backward step."""
    dim, n = A.shape
    total, _ = ops.param_grad_layout(dim, n, has_D, has_bias, False)
    pin = lambda shape, dt: torch.empty(shape, dtype=dt, pin_memory=True)
    return {"y": pin(tuple(u.shape), u.dtype), "du": pin(tuple(u.shape), u.dtype), "ddelta": pin(tuple(delta.shape), u.dtype),
            "dB": pin(tuple(B.shape), B.dtype), "dC": pin(tuple(B.shape), B.dtype),
            "param_grads": pin((total,), torch.float32), "dw": pin((B.size(1), dim // B.size(1)), torch.float32)}


class CrossHostPipeline:
    """``HostPipeline`` for ``cross_scan_2d``: u (b, D, h, w) and dy (b, D, h, w) cross the bus once for all K
    directions; delta (b, K*D, h, w), B and C (b, K, n, h, w) as in the plain operator.  The merged images y and
    du are formed on the device in fp32 (the directions' CTAs add onto them) and leave in the input type."""

    def __init__(self, host, params, delta_softplus=True, chunk=None, depth=3, device=None):
        from . import cross
        self.dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.A, self.D, self.bias, self.w = params["A"], params.get("D"), params.get("delta_bias"), params["w"]
        self.softplus = delta_softplus
        u, delta, B = host["u"], host["delta"], host["B"]
        cross._check_shapes(u, delta, self.A, B, self.w)
        self.batch, self.K = u.size(0), B.size(1)
        per_sample = sum(host[k][0].numel() * host[k].element_size() for k in _XBIG)
        auto = -(-self.batch // min(64, max(1, round(self.batch * per_sample / 32e6))))   # about 32 MB of input per chunk
        self.chunk = max(1, min(chunk or auto, self.batch))
        dim, n = self.A.shape
        self.total, self.parts = ops.param_grad_layout(dim, n, self.D is not None, self.bias is not None, False)
        self.rows, self.cols = cross._masks(self.K)
        c, dev = self.chunk, self.dev
        with torch.cuda.device(dev):
            self.flat = torch.zeros(self.total, dtype=torch.float32, device=dev)
            self.dw = torch.zeros(dim, dtype=torch.float32, device=dev)
            self.wf = self.w.detach().float().contiguous().view(-1)
            self.s_in, self.s_out = torch.cuda.Stream(), torch.cuda.Stream()
            mk = lambda ref, dt=None: torch.empty((c,) + tuple(ref.shape[1:]), dtype=dt or ref.dtype, device=dev)
            self.slots = []
            for _ in range(max(2, depth)):
                s = {k: mk(host[k]) for k in _XBIG}
                s.update(y32=mk(u, torch.float32), du32=mk(u, torch.float32), y=mk(u), du=mk(u), ddelta=mk(delta, u.dtype),
                         dB32=mk(B, torch.float32), dC32=mk(B, torch.float32))
                if B.dtype != torch.float32:
                    s.update(dB=mk(B), dC=mk(B))
                s["free"], s["loaded"], s["done"] = torch.cuda.Event(), torch.cuda.Event(), torch.cuda.Event()
                self.slots.append(s)
            s0 = self.slots[0]
            p = ops._problem(s0["u"], s0["delta"], self.A, s0["B"], s0["C"], self.D, self.bias, None, delta_softplus,
                             torch.float32, "host pipeline", shared_u_dim=dim)
            L = _lib.lib()
            nsaved, nscr = L.cs2d_saved_bytes(ctypes.byref(p)), L.cs2d_bwd_scratch_bytes(ctypes.byref(p))
            if nsaved == 0 or nscr == 0:
                raise RuntimeError(f"cs2d host pipeline: {_lib.last_error()}")
            for s in self.slots:
                s["saved"] = torch.empty(nsaved // 4, dtype=torch.float32, device=dev)
                s["scratch"] = torch.empty(nscr // 4, dtype=torch.float32, device=dev)

    def _part(self, name):
        if name not in self.parts:
            return None
        off, n = self.parts[name]
        return self.flat[off:off + n]

    def run(self, host, out_host, allreduce=False):
        """One forward + backward step; returns ``out_host`` with every copy queued behind the current stream."""
        L = _lib.lib()
        vp = lambda t: ctypes.c_void_p(t.data_ptr()) if t is not None else None
        dim = self.A.size(0)
        with torch.cuda.device(self.dev):
            main = torch.cuda.current_stream()
            stream = ctypes.c_void_p(main.cuda_stream)
            self.flat.zero_()
            self.dw.zero_()
            self.s_in.wait_stream(main)
            nslots = len(self.slots)
            bounds = [(lo, min(lo + self.chunk, self.batch)) for lo in range(0, self.batch, self.chunk)]
            for i, (lo, hi) in enumerate(bounds):
                s, n = self.slots[i % nslots], hi - lo
                with torch.cuda.stream(self.s_in):
                    if i >= nslots:
                        self.s_in.wait_event(s["free"])     # the slot's previous results have left the device
                    for k in _XBIG:
                        s[k][:n].copy_(host[k][lo:hi], non_blocking=True)
                    s["loaded"].record(self.s_in)
                main.wait_event(s["loaded"])
                if i >= nslots:
                    main.wait_event(s["free"])
                t = {k: s[k][:n] for k in _XBIG + ("y32", "du32", "y", "du", "ddelta", "dB32", "dC32")}
                for k in ("y32", "du32", "dB32", "dC32"):   # the directions add onto these
                    t[k].zero_()
                p = ops._problem(t["u"], t["delta"], self.A, t["B"], t["C"], self.D, self.bias, None, self.softplus,
                                 torch.float32, "host pipeline", shared_u_dim=dim)
                dirs = _lib.Dirs(self.rows, self.cols, 1, 0, self.wf.data_ptr(), None)
                rc = L.cs2d_fwd_dir(ctypes.byref(p), ctypes.byref(dirs), vp(t["y32"]), t["y32"].stride(0), t["y32"].stride(1),
                                    t["y32"].stride(2), vp(s["saved"]), stream)
                ops._raise_on(rc, "forward")
                p.out_dtype = ops._DT[t["dy"].dtype]
                dirs = _lib.Dirs(self.rows, self.cols, 3, 0, self.wf.data_ptr(), self.dw.data_ptr())
                rc = L.cs2d_bwd_dir(ctypes.byref(p), ctypes.byref(dirs), vp(t["dy"]), t["dy"].stride(0), t["dy"].stride(1),
                                    t["dy"].stride(2), vp(s["saved"]), vp(s["scratch"]), vp(t["du32"]), vp(t["ddelta"]),
                                    vp(self._part("dA")), vp(t["dB32"]), vp(t["dC32"]), vp(self._part("dD")),
                                    vp(self._part("ddelta_bias")), None, stream)
                ops._raise_on(rc, "backward")
                t["y"].copy_(t["y32"])
                t["du"].copy_(t["du32"])
                dB, dC = t["dB32"], t["dC32"]
                if "dB" in s:
                    dB, dC = s["dB"][:n], s["dC"][:n]
                    dB.copy_(t["dB32"])
                    dC.copy_(t["dC32"])
                s["done"].record(main)
                with torch.cuda.stream(self.s_out):
                    self.s_out.wait_event(s["done"])
                    for name, src in (("y", t["y"]), ("du", t["du"]), ("ddelta", t["ddelta"]), ("dB", dB), ("dC", dC)):
                        out_host[name][lo:hi].copy_(src, non_blocking=True)
                    s["free"].record(self.s_out)
            if allreduce:
                from . import parallel
                parallel.allreduce_param_grads(self.flat)
                parallel.allreduce_param_grads(self.dw)
            out_host["param_grads"].copy_(self.flat, non_blocking=True)
            out_host["dw"].copy_(self.dw.view(self.K, dim // self.K), non_blocking=True)
            main.wait_stream(self.s_out)
        return out_host
