"""ctypes binding of the C-ABI in `include/kcg_capi.h`.

The library is loaded from the package directory (`libkcg_b200.so`, built in-tree by
`kernelcodegen_b200.build`).  There is no fallback: if the library is missing, loading raises.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_uint32, c_uint64, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libkcg_b200.so"
BOUNDS_LIB_PATH = Path(__file__).resolve().parent / "libkcg_b200_bounds.so"   # -DKCG_DEBUG_BOUNDS build

# enum kcg_status_t
KCG_OK = 0
KCG_BAD_SHAPE = 1
KCG_BAD_ALIGN = 2
KCG_UNSUPPORTED = 3
KCG_CUDA_ERROR = 4
KCG_DEVICE_TIMEOUT = 5
KCG_PEER_TIMEOUT = 6
KCG_BAD_WORKSPACE = 8
KCG_BAD_ARGUMENT = 9
KCG_TOO_LARGE = 10
KCG_STATIC_SCRATCH_BYTES = 32 << 20

# enum kcg_dtype_t / kcg_precision_t / kcg_epilogue_t / kcg_layout_t
KCG_F32, KCG_BF16 = 0, 1
KCG_PREC_3XTF32, KCG_PREC_TF32, KCG_PREC_BF16 = 0, 1, 2
KCG_EPI_NONE, KCG_EPI_RELU = 0, 1
KCG_ROW_MAJOR, KCG_COL_MAJOR = 0, 1

EXPORTED_SYMBOLS = (
    "kcg_gemm_workspace_bytes",
    "kcg_fmha_workspace_bytes",
    "kcg_gemm_shared_k_tiles",
    "kcg_gemm_shared_k_plan",
    "kcg_gemm_launch_geometry",
    "kcg_fmha_launch_geometry",
    "kcg_gemm_launch",
    "kcg_gemm_launch_static",
    "kcg_fmha_fwd_launch",
    "kcg_softmax_launch",
    "kcg_batched_gemm_launch",
    "kcg_batched_gemm_workspace_bytes",
    "kcg_transpose_launch",
    "kcg_gemm_host",
    "kcg_gemm_host_staged",
    "kcg_fmha_fwd_host",
    "kcg_gemm_time",
    "kcg_fmha_time",
    "kcg_peer_alloc",
    "kcg_peer_open",
    "kcg_peer_close",
    "kcg_peer_free",
    "kcg_peer_wait_launch",
    "kcg_peer_wait_status",
    "kcg_last_device_status",
    "kcg_set_spin_limit",
    "kcg_debug_bounds_enabled",
    "kcg_debug_set_extent_limit",
    "kcg_debug_bounds_detail",
    "kcg_selftest_wait_timeout",
    "kcg_launch_count",
    "kcg_status_str",
    "kcg_version",
)


class GemmDesc(Structure):
    """Mirror of `struct kcg_gemm_desc`."""

    _fields_ = [
        ("M", c_int64), ("N", c_int64), ("K", c_int64),
        ("lda", c_int64), ("ldb", c_int64), ("ldc", c_int64),
        ("dtype_in", c_int32), ("dtype_out", c_int32),
        ("precision", c_int32), ("epilogue", c_int32), ("b_layout", c_int32),
        ("tile_n", c_int32), ("stages", c_int32), ("group_m", c_int32),
        ("n_peers", c_int32), ("cta_group", c_int32),
        ("peer_c", c_void_p * 8),
        ("mc_c", c_void_p),
        ("n_done_flags", c_int32), ("done_value", c_uint32),
        ("done_flags", c_void_p * 9),
    ]


class FmhaDesc(Structure):
    """Mirror of `struct kcg_fmha_desc`."""

    _fields_ = [
        ("B", c_int32), ("H", c_int32), ("Sq", c_int32), ("Skv", c_int32), ("D", c_int32),
        ("dtype_in", c_int32), ("dtype_out", c_int32), ("causal", c_int32),
        ("scale", c_float), ("reserved", c_int32),
    ]


class KcgError(RuntimeError):
    def __init__(self, status: int, what: str):
        self.status = status
        super().__init__(f"{what}: {status_str(status)}")


_lib = None


def load() -> ctypes.CDLL:
    """Load the native library once; raise if it is not built."""
    global _lib
    if _lib is not None:
        return _lib
    import os

    # KCG_DEBUG_BOUNDS=1 in the environment selects the bounds-checking build of the same sources
    path = BOUNDS_LIB_PATH if os.environ.get("KCG_DEBUG_BOUNDS") == "1" else LIB_PATH
    if not path.exists():
        raise ImportError(
            f"{path} is missing: build it with `python -m kernelcodegen_b200.build` "
            "(there is no CPU or PyTorch fallback)")
    lib = ctypes.CDLL(str(path))
    lib.kcg_gemm_workspace_bytes.restype = c_size_t
    lib.kcg_gemm_workspace_bytes.argtypes = [POINTER(GemmDesc)]
    lib.kcg_fmha_workspace_bytes.restype = c_size_t
    lib.kcg_gemm_shared_k_tiles.restype = c_int
    lib.kcg_gemm_shared_k_tiles.argtypes = [POINTER(GemmDesc)]
    lib.kcg_gemm_shared_k_plan.restype = None
    lib.kcg_gemm_shared_k_plan.argtypes = [c_int32, c_int32, c_int32, c_int32, POINTER(c_int32)]
    lib.kcg_fmha_workspace_bytes.argtypes = [POINTER(FmhaDesc)]
    lib.kcg_gemm_launch_geometry.restype = c_int
    lib.kcg_gemm_launch_geometry.argtypes = [POINTER(GemmDesc), POINTER(c_int32)]
    lib.kcg_fmha_launch_geometry.restype = c_int
    lib.kcg_fmha_launch_geometry.argtypes = [POINTER(FmhaDesc), POINTER(c_int32)]
    lib.kcg_gemm_launch.restype = c_int
    lib.kcg_gemm_launch.argtypes = [POINTER(GemmDesc), c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]
    lib.kcg_gemm_launch_static.restype = c_int
    lib.kcg_gemm_launch_static.argtypes = [POINTER(GemmDesc), c_void_p, c_void_p, c_void_p, c_void_p]
    lib.kcg_fmha_fwd_launch.restype = c_int
    lib.kcg_fmha_fwd_launch.argtypes = [POINTER(FmhaDesc), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p]
    lib.kcg_softmax_launch.restype = c_int
    lib.kcg_softmax_launch.argtypes = [c_int64, c_int64, c_void_p, c_void_p, c_void_p]
    lib.kcg_batched_gemm_launch.restype = c_int
    lib.kcg_batched_gemm_launch.argtypes = [POINTER(GemmDesc), c_int64, c_int64, c_int64, c_int64, c_void_p, c_void_p,
                                            c_void_p, c_void_p, c_size_t, c_void_p]
    lib.kcg_batched_gemm_workspace_bytes.restype = c_size_t
    lib.kcg_batched_gemm_workspace_bytes.argtypes = [POINTER(GemmDesc), c_int64, c_int64, c_int64]
    lib.kcg_transpose_launch.restype = c_int
    lib.kcg_transpose_launch.argtypes = [c_int64, c_int64, c_int64, c_int32, c_void_p, c_void_p, c_void_p]
    lib.kcg_gemm_host.restype = c_int
    lib.kcg_gemm_host.argtypes = [POINTER(GemmDesc), c_void_p, c_void_p, c_void_p]
    lib.kcg_gemm_host_staged.restype = c_int
    lib.kcg_gemm_host_staged.argtypes = [POINTER(GemmDesc), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                         c_void_p, c_void_p, c_size_t, c_int, c_void_p]
    lib.kcg_fmha_fwd_host.restype = c_int
    lib.kcg_fmha_fwd_host.argtypes = [POINTER(FmhaDesc), c_void_p, c_void_p, c_void_p, c_void_p]
    lib.kcg_gemm_time.restype = c_int
    lib.kcg_gemm_time.argtypes = [POINTER(GemmDesc), c_int, POINTER(c_float)]
    lib.kcg_fmha_time.restype = c_int
    lib.kcg_fmha_time.argtypes = [POINTER(FmhaDesc), c_int, POINTER(c_float)]
    lib.kcg_peer_alloc.restype = c_int
    lib.kcg_peer_alloc.argtypes = [c_size_t, POINTER(c_void_p), c_void_p]
    lib.kcg_peer_open.restype = c_int
    lib.kcg_peer_open.argtypes = [c_void_p, POINTER(c_void_p)]
    lib.kcg_peer_close.restype = c_int
    lib.kcg_peer_close.argtypes = [c_void_p]
    lib.kcg_peer_free.restype = c_int
    lib.kcg_peer_free.argtypes = [c_void_p]
    lib.kcg_peer_wait_launch.restype = c_int
    lib.kcg_peer_wait_launch.argtypes = [c_void_p, c_int32, c_int32, c_uint32, c_uint32, c_void_p]
    lib.kcg_peer_wait_status.restype = c_int
    lib.kcg_peer_wait_status.argtypes = []
    lib.kcg_last_device_status.restype = c_int
    lib.kcg_last_device_status.argtypes = []
    lib.kcg_selftest_wait_timeout.restype = c_int
    lib.kcg_selftest_wait_timeout.argtypes = [c_uint32]
    lib.kcg_set_spin_limit.restype = None
    lib.kcg_set_spin_limit.argtypes = [c_uint32]
    lib.kcg_debug_bounds_enabled.restype = c_int
    lib.kcg_debug_bounds_enabled.argtypes = []
    lib.kcg_debug_set_extent_limit.restype = None
    lib.kcg_debug_set_extent_limit.argtypes = [c_uint64]
    lib.kcg_debug_bounds_detail.restype = c_int
    lib.kcg_debug_bounds_detail.argtypes = [POINTER(c_uint64)]
    lib.kcg_launch_count.restype = c_uint64
    lib.kcg_launch_count.argtypes = []
    lib.kcg_status_str.restype = c_char_p
    lib.kcg_status_str.argtypes = [c_int]
    lib.kcg_version.restype = c_char_p
    lib.kcg_version.argtypes = []
    _lib = lib
    return lib


def status_str(status: int) -> str:
    return load().kcg_status_str(int(status)).decode()


def check(status: int, what: str) -> None:
    if status != KCG_OK:
        raise KcgError(status, what)
