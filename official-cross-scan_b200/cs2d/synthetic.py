"""Seeded synthetic inputs for the 2D-CrossScan selective scan.

The shapes stand in for the activations of the networks the reference targets
(VMamba-style backbones on ImageNet-224, detection- and segmentation-scale
feature maps); only the feature-map shapes and the parameter initialisation
are reproduced, no dataset is involved.  Everything is generated on the CPU
from one ``torch.Generator`` so that every implementation sees identical bits.

Distributions: ``u0, B, C, delta ~ N(0,1)``; the K directions of ``u`` are the
four corner flips of ``u0``; ``delta`` is passed raw (softplus is applied by
the operator); ``delta_bias = inv_softplus(dt)`` with ``dt`` log-uniform in
``[1e-3, 1e-1]``; ``A[d, n] = -(n+1)``; ``D = 1``.
"""
from __future__ import annotations

import math

import torch

# name -> (B, K, D, N, H, W, io dtype)
CONFIGS = {
    "c1_cpu_correctness": (1, 4, 8, 4, 8, 8, torch.float32),
    "c2_vmamba_t_stage1": (32, 4, 192, 16, 56, 56, torch.float32),
    "c3_s1_n16": (128, 4, 192, 16, 56, 56, torch.bfloat16),
    "c3_s2_n16": (128, 4, 384, 16, 28, 28, torch.bfloat16),
    "c3_s3_n16": (128, 4, 768, 16, 14, 14, torch.bfloat16),
    "c3_s4_n16": (128, 4, 1536, 16, 7, 7, torch.bfloat16),
    "c3_s1_n1": (128, 4, 192, 1, 56, 56, torch.bfloat16),
    "c3_s2_n1": (128, 4, 384, 1, 28, 28, torch.bfloat16),
    "c3_s3_n1": (128, 4, 768, 1, 14, 14, torch.bfloat16),
    "c3_s4_n1": (128, 4, 1536, 1, 7, 7, torch.bfloat16),
    "c4_detection": (2, 4, 192, 16, 200, 336, torch.bfloat16),
    "c5_segmentation": (16, 4, 384, 16, 128, 128, torch.bfloat16),
}

_FLIPS = ((), (3,), (2,), (2, 3))


def make_inputs(batch, k, d, n, h, w, dtype=torch.float32, seed=0, delta_dim=None,
                with_D=True, with_bias=True, a_decay=None):
    """Returns a dict of CPU tensors: u, delta, A, B, C, D, delta_bias, A_decay, dout."""
    gen = torch.Generator().manual_seed(seed)
    dim = k * d
    ddim = dim if delta_dim is None else delta_dim
    u0 = torch.randn(batch, d, h, w, generator=gen)
    u = torch.cat([torch.flip(u0, _FLIPS[i % 4]) if _FLIPS[i % 4] else u0 for i in range(k)], 1)
    delta = torch.randn(batch, ddim, h, w, generator=gen)
    dt = torch.exp(torch.rand(ddim, generator=gen) * (math.log(0.1) - math.log(1e-3)) + math.log(1e-3))
    dt = dt.clamp_min(1e-4)
    delta_bias = dt + torch.log(-torch.expm1(-dt))
    A = -torch.arange(1, n + 1, dtype=torch.float32).repeat(dim, 1).contiguous()
    Bm = torch.randn(batch, k, n, h, w, generator=gen)
    Cm = torch.randn(batch, k, n, h, w, generator=gen)
    gen2 = torch.Generator().manual_seed(seed + 1)
    dout = torch.randn(batch, dim, h, w, generator=gen2)
    return {
        "u": u.to(dtype).contiguous(), "delta": delta.to(dtype).contiguous(), "A": A,
        "B": Bm.to(dtype).contiguous(), "C": Cm.to(dtype).contiguous(),
        "D": torch.ones(dim) if with_D else None,
        "delta_bias": delta_bias.float() if with_bias else None,
        "A_decay": None if a_decay is None else torch.tensor([float(a_decay)]),
        "dout": dout.to(dtype).contiguous(),
    }


def elements(batch, k, d, n, h, w):
    """Scanned elements of one forward (or backward) pass: B*K*D*H*W*N."""
    return batch * k * d * n * h * w


def algorithmic_bytes(batch, k, d, n, h, w, s, fwd=True, bwd=True):
    """HBM bytes the operator must move at the reference boundary.

    Forward reads u, delta, B, C and writes out; backward reads u, delta, dout,
    B, C and writes du, ddelta, dB, dC; ``s`` is bytes per I/O element.
    """
    px = batch * h * w * k * s
    total = 0
    if fwd:
        total += px * (3 * d + 2 * n)
    if bwd:
        total += px * (5 * d + 4 * n)
    return total
