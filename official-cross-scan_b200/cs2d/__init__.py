"""cs2d - B200-native 2D-CrossScan selective scan (forward + backward).

Drop-in for the ``fwd`` / ``bwd`` operators of the reference CUDA extension
``selective_nd_scan_cuda_oflex`` plus an autograd Function.
"""
from .ops import SelectiveScan2D, bwd, fwd, fwd_only, selective_scan_2d  # noqa: F401
from .cross import CrossScan2D, cross_scan_2d  # noqa: F401
from .host import (CrossHostPipeline, HostPipeline, alloc_cross_host_outputs, alloc_host_outputs,  # noqa: F401
                   fwd_bwd_from_host)
from ._lib import LIB_PATH, build, device_status, launch_count  # noqa: F401
