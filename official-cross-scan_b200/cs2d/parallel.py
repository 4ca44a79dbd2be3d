"""Batch-sharded (data-parallel) use of the 2D-CrossScan selective scan.

Every (batch, channel) recurrence is independent, so a job is split across
GPUs by batch with no exchange on the data path: u, delta, B, C, dout and
du, ddelta, dB, dC stay on the rank that owns the samples.  Only the
per-channel parameter gradients dA, dD, ddelta_bias (and dA_decay) sum over the
batch.  The backward writes them into ONE flat fp32 buffer and a single
all-reduce over that buffer (NCCL over NVLink on GPUs, gloo in CPU tests),
issued on the same stream right after the kernel, completes the step.  The
reference has no distributed code; its kernels accumulate these gradients with
atomics across the batch inside one GPU
(``selective_scan_bwd_kernel_oflex.cuh:886,891,896``).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import ops


def shard_bounds(batch: int, rank: int, world: int):
    """Contiguous, balanced [lo, hi) slice of the batch owned by ``rank``."""
    if not (0 <= rank < world) or batch < 0:
        raise ValueError("bad rank/world/batch")
    base, rem = divmod(batch, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def allreduce_param_grads(flat: torch.Tensor, group=None, async_op: bool = False):
    """Sums the flat parameter-gradient buffer over the ranks, in place."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return None
    return dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group, async_op=async_op)


def unpack_param_grads(flat, dim, dstate, has_D, has_bias, has_decay, delta_dim=None):
    """Views of dA, dD, ddelta_bias, dA_decay inside ``flat`` (None where absent)."""
    total, parts = ops.param_grad_layout(dim, dstate, has_D, has_bias, has_decay)
    if flat.numel() != total:
        raise ValueError("flat buffer does not match the layout")

    def part(name):
        if name not in parts:
            return None
        off, n = parts[name]
        return flat[off:off + n]

    dA = part("dA").view(dim, dstate)
    dbias = part("ddelta_bias")
    if dbias is not None and delta_dim is not None and delta_dim != dim:
        dbias = dbias.view(delta_dim, dim // delta_dim).sum(1)
    return dA, part("dD"), dbias, part("dA_decay")


def bwd_data_parallel(u, delta, A, B, C, D_, delta_bias_, dout, x_, x_v_, delta_softplus, A_decay_=None,
                      x_sd_=None, group=None):
    """``ops.bwd`` on this rank's batch shard followed by the one all-reduce.

    Returns the same list as ``ops.bwd``; dA, dD, ddelta_bias, dA_decay hold the
    sums over all ranks.
    """
    dim, dstate = A.shape
    total, _ = ops.param_grad_layout(dim, dstate, D_ is not None, delta_bias_ is not None, A_decay_ is not None)
    flat = torch.zeros(total, dtype=torch.float32, device=u.device)
    res = ops.bwd(u, delta, A, B, C, D_, delta_bias_, dout, x_, x_v_, delta_softplus, A_decay_, x_sd_,
                  param_grads=flat)
    allreduce_param_grads(flat, group)
    dA, dD, dbias, ddecay = unpack_param_grads(flat, dim, dstate, D_ is not None, delta_bias_ is not None,
                                               A_decay_ is not None, delta.size(1))
    res[2], res[5], res[6], res[7] = dA, dD, dbias, ddecay
    return res


class ResidentStep:
    """Forward + backward (+ the one all-reduce) on device-resident tensors, with every buffer
    preallocated: a step allocates nothing and issues, on the current stream, the forward kernel,
    two zero fills, the backward kernel, the all-reduce of the flat parameter-gradient buffer and
    the cast of dB / dC to the input type.  The collective is started before the casts and waited
    for after them, so that it overlaps them.  At small per-GPU batches (a batch of 32 split over
    8 GPUs leaves about a millisecond of kernels per step) this is what keeps the allocator, the
    fills and the collective off the critical path.

    ``t`` is a dict of device tensors ``u, delta, A, B, C, D, delta_bias, dout`` (``D`` and
    ``delta_bias`` may be None); the buffers are sized for exactly these shapes.
    """

    def __init__(self, t, delta_softplus=True, group=None):
        import ctypes
        from . import _lib
        self.group, self.softplus = group, bool(delta_softplus)
        u, B = t["u"], t["B"]
        dev = u.device
        dim, n = t["A"].shape
        self.total, self.parts = ops.param_grad_layout(dim, n, t.get("D") is not None, t.get("delta_bias") is not None,
                                                       False)
        L = _lib.lib()
        p = ops._problem(u, t["delta"], t["A"], B, t["C"], t.get("D"), t.get("delta_bias"), None, delta_softplus, u.dtype,
                         "resident step")
        nsaved, nscr = L.cs2d_saved_bytes(ctypes.byref(p)), L.cs2d_bwd_scratch_bytes(ctypes.byref(p))
        if nsaved == 0 or nscr == 0:
            raise RuntimeError(f"cs2d resident step: {_lib.last_error()}")
        with torch.cuda.device(dev):
            f32 = lambda ref: torch.empty(tuple(ref.shape), dtype=torch.float32, device=dev)
            self.out, self.du, self.ddelta = torch.empty_like(u), torch.empty_like(u), torch.empty_like(u)
            self.dB32, self.dC32 = f32(B), f32(B)
            self.dB = self.dB32 if B.dtype == torch.float32 else torch.empty_like(B)
            self.dC = self.dC32 if B.dtype == torch.float32 else torch.empty_like(B)
            self.flat = torch.zeros(self.total, dtype=torch.float32, device=dev)
            self.saved = torch.empty(nsaved // 4, dtype=torch.float32, device=dev)
            self.scratch = torch.empty(max(4, nscr // 4), dtype=torch.float32, device=dev)
        self.p = p

    def _part(self, name):
        if name not in self.parts:
            return None
        off, n = self.parts[name]
        return self.flat[off:off + n]

    def run(self, t, allreduce=True):
        """One step on the tensors of ``t`` (same shapes as at construction).  Returns self; the results
        are ``out, du, ddelta, dB, dC`` and ``flat`` (dA | dD | ddelta_bias, summed over the ranks)."""
        import ctypes
        from . import _lib
        L = _lib.lib()
        vp = lambda x: ctypes.c_void_p(x.data_ptr()) if x is not None else None
        u, dout = t["u"], t["dout"]
        with torch.cuda.device(u.device):
            stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
            p = ops._problem(u, t["delta"], t["A"], t["B"], t["C"], t.get("D"), t.get("delta_bias"), None, self.softplus,
                             u.dtype, "resident step")
            rc = L.cs2d_fwd(ctypes.byref(p), vp(self.out), self.out.stride(0), self.out.stride(1), self.out.stride(2),
                            vp(self.saved), stream)
            ops._raise_on(rc, "forward")
            self.dB32.zero_()
            self.dC32.zero_()
            self.flat.zero_()
            p.out_dtype = ops._DT[dout.dtype]
            rc = L.cs2d_bwd(ctypes.byref(p), vp(dout), dout.stride(0), dout.stride(1), dout.stride(2), vp(self.saved),
                            vp(self.scratch), vp(self.du), vp(self.ddelta), vp(self._part("dA")), vp(self.dB32),
                            vp(self.dC32), vp(self._part("dD")), vp(self._part("ddelta_bias")), None, stream)
            ops._raise_on(rc, "backward")
            work = allreduce_param_grads(self.flat, self.group, async_op=True) if allreduce else None
            if self.dB is not self.dB32:
                self.dB.copy_(self.dB32)
                self.dC.copy_(self.dC32)
            if work is not None:
                work.wait()
        return self
