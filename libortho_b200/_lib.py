"""ctypes loader of ``libortho_b200.so`` -- the C-ABI CUDA library behind ``OrthoLinear``.

Takes the place of the pybind11 module ``libortho._C_ops`` (``torch_bind/bindings.cpp:46-49``
in the reference).  There is no fallback of any kind: if the shared library is missing or does
not load, importing the operator fails with an error that says how to build it.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libortho_b200.so")

OK = 0
DECODE_MAX_M = 64

_lib = None


class LayerDesc(ctypes.Structure):
    """``ortho_b200_layer_desc`` of ``include/ortho_b200.h``."""
    _fields_ = [("q_weight", ctypes.c_void_p), ("q_scales_f16", ctypes.c_void_p),
                ("ortho_values_f16", ctypes.c_void_p), ("ortho_col_indices", ctypes.c_void_p),
                ("ortho_row_ptr", ctypes.c_void_p), ("nnz", ctypes.c_int64),
                ("plan", ctypes.c_void_p), ("bias_f32", ctypes.c_void_p), ("y_f16", ctypes.c_void_p),
                ("N", ctypes.c_int64), ("ldy", ctypes.c_int64), ("alpha", ctypes.c_float), ("reserved", ctypes.c_int32)]


class OrthoB200Error(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        msg = lib().ortho_b200_strerror(status).decode()
        if status == 6:
            msg += f" [cudaError {lib().ortho_b200_last_cuda_error()}]"
        super().__init__(f"{where}: {msg} (status {status})")


def _declare(l):
    c = ctypes
    vp, i64, i32p = c.c_void_p, c.c_int64, c.c_void_p
    l.ortho_b200_strerror.restype = c.c_char_p
    l.ortho_b200_strerror.argtypes = [c.c_int]
    l.ortho_b200_version.restype = c.c_int
    l.ortho_b200_version.argtypes = []
    l.ortho_b200_last_cuda_error.restype = c.c_int
    l.ortho_b200_last_cuda_error.argtypes = []
    l.ortho_b200_plan_create.restype = c.c_int
    l.ortho_b200_plan_create.argtypes = [c.POINTER(vp), i32p, i32p, vp, i64, i64, i64, vp]
    l.ortho_b200_plan_destroy.restype = c.c_int
    l.ortho_b200_plan_destroy.argtypes = [vp]
    l.ortho_b200_plan_nnz.restype = i64
    l.ortho_b200_plan_nnz.argtypes = [vp]
    l.ortho_b200_plan_max_row_nnz.restype = i64
    l.ortho_b200_plan_max_row_nnz.argtypes = [vp]
    l.ortho_b200_plan_rows_ordered.restype = ctypes.c_int
    l.ortho_b200_plan_rows_ordered.argtypes = [vp]
    l.ortho_b200_plan_decode_dump.restype = c.c_int
    l.ortho_b200_plan_decode_dump.argtypes = [vp, i32p, i32p, vp, vp]
    l.ortho_b200_dequant_dump.restype = c.c_int
    l.ortho_b200_dequant_dump.argtypes = [vp, vp, i64, i64, vp, vp, vp]
    l.ortho_b200_workspace_bytes.restype = i64
    l.ortho_b200_workspace_bytes.argtypes = [i64, i64, i64]
    l.ortho_b200_plan_workspace_bytes.restype = i64
    l.ortho_b200_plan_workspace_bytes.argtypes = [vp, i64]
    l.ortho_b200_forward.restype = c.c_int
    l.ortho_b200_forward.argtypes = [vp, vp, vp, i32p, i32p, i64, vp, vp, i64, i64, i64, c.c_float,
                                     vp, vp, i64, vp]
    l.ortho_b200_forward_multi.restype = c.c_int
    l.ortho_b200_forward_multi.argtypes = [c.POINTER(LayerDesc), c.c_int, vp, i64, i64, vp, i64, vp]
    l.ortho_b200_multi_workspace_bytes.restype = i64
    l.ortho_b200_multi_workspace_bytes.argtypes = [c.POINTER(LayerDesc), c.c_int, i64, i64]
    l.ortho_b200_forward_static_scratch.restype = c.c_int
    l.ortho_b200_forward_static_scratch.argtypes = [vp, vp, vp, i32p, i32p, i64, vp, vp, i64, i64, i64, c.c_float, vp]
    l.ortho_b200_set_decode_config.restype = c.c_int
    l.ortho_b200_set_decode_config.argtypes = [c.c_int, c.c_int, c.c_int, c.c_int]
    l.ortho_b200_query_kernel_status.restype = c.c_int
    l.ortho_b200_query_kernel_status.argtypes = []
    l.ortho_b200_launch_count.restype = i64
    l.ortho_b200_launch_count.argtypes = []
    l.ortho_b200_pack_base.restype = c.c_int
    l.ortho_b200_pack_base.argtypes = [vp, i64, i64, vp, vp, vp, vp]
    l.ortho_b200_csr_count.restype = c.c_int
    l.ortho_b200_csr_count.argtypes = [vp, i64, i64, vp, vp]
    l.ortho_b200_csr_fill.restype = c.c_int
    l.ortho_b200_csr_fill.argtypes = [vp, i64, i64, vp, vp, vp, vp]
    l.ortho_b200_sieve_scratch_bytes.restype = i64
    l.ortho_b200_sieve_scratch_bytes.argtypes = [i64]
    l.ortho_b200_sieve.restype = c.c_int
    l.ortho_b200_sieve.argtypes = [vp, vp, i64, i64, c.c_float, i64, vp, vp, vp, i64, vp]
    l.ortho_b200_comm_create.restype = c.c_int
    l.ortho_b200_comm_create.argtypes = [c.c_int, c.c_int, i64, c.POINTER(vp)]
    l.ortho_b200_comm_export.restype = c.c_int
    l.ortho_b200_comm_export.argtypes = [vp, vp]
    l.ortho_b200_comm_connect.restype = c.c_int
    l.ortho_b200_comm_connect.argtypes = [vp, vp]
    l.ortho_b200_comm_local.restype = vp
    l.ortho_b200_comm_local.argtypes = [vp]
    l.ortho_b200_comm_set_timeout_ms.restype = c.c_int
    l.ortho_b200_comm_set_timeout_ms.argtypes = [vp, i64]
    l.ortho_b200_comm_set_deferred.restype = c.c_int
    l.ortho_b200_comm_set_deferred.argtypes = [vp, c.c_int]
    l.ortho_b200_comm_wait.restype = c.c_int
    l.ortho_b200_comm_wait.argtypes = [vp, vp]
    l.ortho_b200_comm_destroy.restype = c.c_int
    l.ortho_b200_comm_destroy.argtypes = [vp]
    l.ortho_b200_forward_gather.restype = c.c_int
    l.ortho_b200_forward_gather.argtypes = [vp, vp, vp, i32p, i32p, i64, vp, i64, i64, i64, c.c_float,
                                            vp, vp, i64, vp, i64, i64, i64, vp]


# every symbol include/ortho_b200.h declares
EXPORTS = [
    "ortho_b200_strerror", "ortho_b200_version", "ortho_b200_last_cuda_error",
    "ortho_b200_plan_create", "ortho_b200_plan_destroy", "ortho_b200_plan_nnz",
    "ortho_b200_plan_max_row_nnz", "ortho_b200_plan_rows_ordered", "ortho_b200_plan_decode_dump", "ortho_b200_dequant_dump",
    "ortho_b200_workspace_bytes", "ortho_b200_plan_workspace_bytes", "ortho_b200_forward", "ortho_b200_set_decode_config",
    "ortho_b200_launch_count", "ortho_b200_query_kernel_status", "ortho_b200_forward_static_scratch",
    "ortho_b200_comm_create", "ortho_b200_comm_export", "ortho_b200_comm_connect", "ortho_b200_comm_local",
    "ortho_b200_comm_set_timeout_ms", "ortho_b200_comm_destroy", "ortho_b200_forward_gather",
    "ortho_b200_comm_set_deferred", "ortho_b200_comm_wait",
    "ortho_b200_pack_base", "ortho_b200_csr_count", "ortho_b200_csr_fill",
    "ortho_b200_sieve_scratch_bytes", "ortho_b200_sieve",
    "ortho_b200_forward_multi", "ortho_b200_multi_workspace_bytes",
]


def lib():
    """The loaded library.  Raises ``ImportError`` if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: the CUDA extension is required (there is no CPU or "
                "PyTorch fallback). Build it with `python -m libortho_b200.build`.")
        l = ctypes.CDLL(LIB_PATH)
        _declare(l)
        _lib = l
    return _lib


def check(status: int, where: str) -> None:
    if status != OK:
        raise OrthoB200Error(status, where)
