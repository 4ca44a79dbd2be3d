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
