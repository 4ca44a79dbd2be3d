"""Module with the name and the two functions of the reference extension.

``import selective_nd_scan_cuda_oflex as ext; ext.fwd(...); ext.bwd(...)`` works
unchanged for a caller written against the reference's pybind module
(``kernels/selective_nd_scan/src/cusoflex/selective_scan_oflex.cpp:442-445``).
"""
from cs2d.ops import bwd, fwd  # noqa: F401
