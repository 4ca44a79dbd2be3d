"""Module level of the four-corner CrossScan: the parameters a VMamba-style SS2D block
keeps around the scan (``A_log``, ``D``, ``dt_bias``) plus the trainable direction-fusion
weights the reference's README describes ("trainable weights to fuse the directions") but
ships no code for (``CrossScan2D``), and the block around it - projections that emit ``delta``,
``B`` and ``C`` in the layout the kernels read, convolution, normalisation, gate (``SS2D``).
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


class SS2D(nn.Module):
    """A VMamba-style 2-D selective-scan block around the four-corner CrossScan - the caller the
    reference leaves to its forks (its README names them; the snapshot ships only the extension).

    ``x (b, h, w, d_model)`` ->  in_proj -> (features, gate) -> depthwise 3x3 conv + SiLU ->
    x_proj (one 1x1 convolution that emits, per direction, a low-rank ``dt`` code and ``B``, ``C``
    directly in the ``(b, K, ., h, w)`` layout the kernels read: the three are strided views of its
    output, nothing is copied or transposed) -> dt_proj (per direction, rank -> d_inner; the
    softplus and ``dt_bias`` are applied inside the kernels) -> CrossScan2D (all directions and the
    fusion weights in one launch each way) -> LayerNorm -> gate with SiLU -> out_proj.
    """

    def __init__(self, d_model: int, d_state: int = 16, expand: int = 2, dt_rank: int | None = None, d_conv: int = 3,
                 directions: int = 4, device=None):
        super().__init__()
        self.d_model, self.d_inner, self.d_state, self.K = d_model, expand * d_model, d_state, directions
        self.dt_rank = dt_rank or max(1, math.ceil(d_model / 16))
        d, R, N, K = self.d_inner, self.dt_rank, d_state, directions
        self.in_proj = nn.Linear(d_model, 2 * d, bias=False, device=device)
        self.conv2d = nn.Conv2d(d, d, d_conv, padding=d_conv // 2, groups=d, bias=True, device=device)
        self.x_proj = nn.Conv2d(d, K * (R + 2 * N), 1, bias=False, device=device)
        self.dt_proj = nn.Parameter(torch.randn(K, d, R, device=device) * R ** -0.5)
        self.scan = CrossScan2D(d, N, K, device=device)
        self.out_norm = nn.LayerNorm(d, device=device)
        self.out_proj = nn.Linear(d, d_model, bias=False, device=device)

    def _scan(self, u, delta, A, B, C, w, D, dt_bias):
        return cross_scan_2d(u, delta, A, B, C, w, D, dt_bias, True)

    def forward(self, x):
        b, h, w, _ = x.shape
        d, R, N, K = self.d_inner, self.dt_rank, self.d_state, self.K
        xz = self.in_proj(x)
        u, z = xz[..., :d], xz[..., d:]
        u = torch.nn.functional.silu(self.conv2d(u.permute(0, 3, 1, 2))).contiguous()        # (b, d, h, w)
        code = self.x_proj(u).view(b, K, R + 2 * N, h, w)
        dts, Bm, Cm = code[:, :, :R], code[:, :, R:R + N], code[:, :, R + N:]                  # views, no copies
        delta = torch.einsum("bkrhw,kdr->bkdhw", dts, self.dt_proj.to(dts.dtype)).reshape(b, K * d, h, w)
        A = -torch.exp(self.scan.A_log.float())
        y = self._scan(u, delta, A, Bm, Cm, self.scan.fusion, self.scan.D, self.scan.dt_bias)
        y = self.out_norm(y.permute(0, 2, 3, 1).to(x.dtype))
        return self.out_proj(y * torch.nn.functional.silu(z))
