"""ctypes binding of the cs2d C-ABI library (``include/cs2d.h``)."""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libcs2d.so")

F32, F16, BF16 = 0, 1, 2
NOALLOC_SCRATCH_BYTES = 32 << 20  # CS2D_NOALLOC_SCRATCH_BYTES
DIRS_SERIAL = 1                   # CS2D_DIRS_SERIAL


_i32, _i64, _p = ctypes.c_int32, ctypes.c_int64, ctypes.c_void_p


class Dirs(ctypes.Structure):
    """Mirror of ``cs2d_dirs``."""
    _fields_ = [("flip_rows_mask", ctypes.c_uint32), ("flip_cols_mask", ctypes.c_uint32),
                ("shared_input", ctypes.c_int32), ("flags", ctypes.c_int32),
                ("merge_w", ctypes.c_void_p), ("merge_dw", ctypes.c_void_p)]


class Problem(ctypes.Structure):
    """Mirror of ``cs2d_problem``."""
    _fields_ = (
        [(n, _i32) for n in ("batch", "dim", "nrows", "ncols", "dstate", "n_groups", "delta_dim",
                             "io_dtype", "out_dtype", "delta_softplus")]
        + [("u", _p), ("u_bs", _i64), ("u_ds", _i64), ("u_hs", _i64)]
        + [("delta", _p), ("delta_bs", _i64), ("delta_ds", _i64), ("delta_hs", _i64)]
        + [("A", _p), ("A_ds", _i64), ("A_ns", _i64)]
        + [("B", _p), ("B_bs", _i64), ("B_gs", _i64), ("B_ns", _i64), ("B_hs", _i64)]
        + [("C", _p), ("C_bs", _i64), ("C_gs", _i64), ("C_ns", _i64), ("C_hs", _i64)]
        + [("D", _p), ("delta_bias", _p), ("A_decay", _p)]
    )


_lib = None


def build() -> str:
    """Compile the library in-tree with nvcc for sm_100a (no GPU needed)."""
    import subprocess
    subprocess.run([os.path.join(_HERE, "..", "csrc", "build.sh")], check=True)
    return LIB_PATH


def lib():
    """Loads the library.  There is no fallback: a missing build is an error."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"cs2d: {LIB_PATH} is missing - build it with official-cross-scan_b200/csrc/build.sh; "
                "there is no CPU or PyTorch fallback for this operator")
        L = ctypes.CDLL(LIB_PATH)
        vp, i64 = ctypes.c_void_p, ctypes.c_int64
        L.cs2d_saved_bytes.restype = ctypes.c_size_t
        L.cs2d_saved_bytes.argtypes = [ctypes.POINTER(Problem)]
        L.cs2d_bwd_scratch_bytes.restype = ctypes.c_size_t
        L.cs2d_bwd_scratch_bytes.argtypes = [ctypes.POINTER(Problem)]
        L.cs2d_fwd_only_scratch_bytes.restype = ctypes.c_size_t
        L.cs2d_fwd_only_scratch_bytes.argtypes = [ctypes.POINTER(Problem)]
        L.cs2d_fwd.restype = ctypes.c_int
        L.cs2d_fwd.argtypes = [ctypes.POINTER(Problem), vp, i64, i64, i64, vp, vp]
        L.cs2d_bwd.restype = ctypes.c_int
        L.cs2d_bwd.argtypes = [ctypes.POINTER(Problem), vp, i64, i64, i64, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp]
        dp = ctypes.POINTER(Dirs)
        L.cs2d_fwd_dir.restype = ctypes.c_int
        L.cs2d_fwd_dir.argtypes = [ctypes.POINTER(Problem), dp, vp, i64, i64, i64, vp, vp]
        L.cs2d_fwd_only.restype = ctypes.c_int
        L.cs2d_fwd_only.argtypes = [ctypes.POINTER(Problem), dp, vp, i64, i64, i64, vp, vp]
        L.cs2d_bwd_det_scratch_bytes.restype = ctypes.c_size_t
        L.cs2d_bwd_det_scratch_bytes.argtypes = [ctypes.POINTER(Problem)]
        L.cs2d_bwd_det.restype = ctypes.c_int
        L.cs2d_bwd_det.argtypes = [ctypes.POINTER(Problem), dp, vp, i64, i64, i64, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp,
                                   vp, vp]
        L.cs2d_bwd_dir.restype = ctypes.c_int
        L.cs2d_bwd_dir.argtypes = [ctypes.POINTER(Problem), dp, vp, i64, i64, i64, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp,
                                   vp]
        L.cs2d_bwd_noalloc.restype = ctypes.c_int
        L.cs2d_bwd_noalloc.argtypes = [ctypes.POINTER(Problem), vp, i64, i64, i64, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp]
        L.cs2d_last_error.restype = ctypes.c_char_p
        L.cs2d_abi_version.restype = ctypes.c_int
        L.cs2d_launch_count.restype = ctypes.c_int64
        L.cs2d_device_status.restype = ctypes.c_int
        if L.cs2d_abi_version() != 2:
            raise RuntimeError("cs2d: ABI version mismatch between libcs2d.so and the Python binding")
        _lib = L
    return _lib


def last_error() -> str:
    return lib().cs2d_last_error().decode()


def device_status() -> int:
    """Reads and clears the device status word (0 = fine); synchronises."""
    return int(lib().cs2d_device_status())


def launch_count() -> int:
    return int(lib().cs2d_launch_count())
