"""Module level of the four-corner CrossScan: the parameters a VMamba-style SS2D block
keeps around the scan (``A_log``, ``D``, ``dt_bias``) plus the trainable direction-fusion
weights the reference's README describes ("trainable weights to fuse the directions") but
ships no code for.  The projections that produce ``delta``, ``B`` and ``C`` from the
features are the caller's; this module owns only what the scan itself needs.
"""
from __future__ import annotations

import math

import torch
from torch import nn

from .cross import cross_scan_2d


class CrossScan2D(nn.Module):
    """y = sum_k w[k] * scan_k(u; delta_k, A_k, B_k, C_k, D_k) over K corner directions.

    Inputs of ``forward``: ``u (b, d_inner, h, w)``, ``delta (b, K*d_inner, h, w)`` (raw, the
    softplus and ``dt_bias`` are applied inside the kernels), ``B, C (b, K, d_state, h, w)``.
    Initialisation follows the S4D-real / Mamba convention: ``A = -(1..d_state)``,
    ``dt`` log-uniform in ``[dt_min, dt_max]`` through the inverse softplus, ``D = 1``,
    fusion weights ``1/K``.
    """

    def __init__(self, d_inner: int, d_state: int = 16, directions: int = 4, dt_min: float = 1e-3,
                 dt_max: float = 1e-1, dt_init_floor: float = 1e-4, device=None, dtype=torch.float32):
        super().__init__()
        if d_state > 16:
            raise ValueError("d_state must be <= 16")
        self.d_inner, self.d_state, self.K = d_inner, d_state, directions
        dim = directions * d_inner
        A = torch.arange(1, d_state + 1, dtype=torch.float32, device=device).repeat(dim, 1)
        self.A_log = nn.Parameter(torch.log(A))
        self.D = nn.Parameter(torch.ones(dim, dtype=torch.float32, device=device))
        dt = torch.exp(torch.rand(dim, device=device) * (math.log(dt_max) - math.log(dt_min)) + math.log(dt_min))
        dt = dt.clamp_min(dt_init_floor)
        self.dt_bias = nn.Parameter(dt + torch.log(-torch.expm1(-dt)))           # inverse softplus
        self.fusion = nn.Parameter(torch.full((directions, d_inner), 1.0 / directions, dtype=torch.float32,
                                              device=device))
        self.io_dtype = dtype

    def forward(self, u, delta, B, C):
        A = -torch.exp(self.A_log.float())
        return cross_scan_2d(u, delta, A, B, C, self.fusion, self.D, self.dt_bias, True)

    def extra_repr(self):
        return f"d_inner={self.d_inner}, d_state={self.d_state}, directions={self.K}"
