"""ctypes binding of libsla_b200.so, the C-ABI library declared in include/sla_b200.h.

The library is the product: there is no Python or CPU fallback. Importing this module without the
built shared object raises, and every call converts a negative status into an exception.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libsla_b200.so")

SLA_BF16, SLA_FP16, SLA_FP32 = 0, 1, 2
PHI = {"softmax": 0, "relu": 1, "elu": 2}
OP_BLOCK_MAP, OP_FWD, OP_BWD, OP_LINEAR_STATE, OP_SAGE_FWD, OP_SPARSE_BWD = 0, 1, 2, 3, 4, 5
FLAG_SPARSE_ONLY, FLAG_LEGACY_MMA, FLAG_LINEAR_UNSELECTED, FLAG_STATE_READY, FLAG_LINEAR_ONLY = 1, 2, 4, 8, 16

# every symbol include/sla_b200.h declares
EXPORTS = (
    "sla_version", "sla_status_string", "sla_last_cuda_error", "sla_launch_count", "sla_poll_device_error", "sla_debug_set_trace", "sla_debug_set_wait_limit_ns", "sla_debug_drop_first_k_tile", "sla_topk_count", "sla_workspace_bytes", "sla_kernel_path",
    "sla_block_map", "sla_column_lists", "sla_index_convert", "sla_pooled_sums_bytes", "sla_qk_norm_rope_pool",
    "sla_block_map_pooled", "sla_sparse_fwd", "sla_sparse_bwd", "sla_linear_state", "sla_linear_state_static", "sla_fwd", "sla_fwd_gather", "sla_enable_peer_access", "sla_ipc_export", "sla_ipc_open", "sla_ipc_close", "sla_fwd_prepare", "sla_bwd",
    "sage_sla_fwd", "sage_sla_fwd_gather", "sage_sla_prepare",
)


class SlaShape(C.Structure):
    _fields_ = [
        ("B", C.c_int32), ("H", C.c_int32), ("L", C.c_int32), ("D", C.c_int32),
        ("BLKQ", C.c_int32), ("BLKK", C.c_int32), ("topk", C.c_int32), ("dtype", C.c_int32),
        ("feature_map", C.c_int32), ("flags", C.c_int32), ("qk_scale", C.c_float),
    ]


class SlaError(RuntimeError):
    def __init__(self, status: int, text: str):
        super().__init__(f"sla_b200 status {status}: {text}")
        self.status = status


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python sla_b200/build.py` (needs nvcc). "
            "sla_b200 has no fallback path.")
    lib = C.CDLL(LIB_PATH)
    vp, i32p, f32p, i8p = C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p
    sp = C.POINTER(SlaShape)
    lib.sla_version.restype = C.c_int
    lib.sla_status_string.restype = C.c_char_p
    lib.sla_status_string.argtypes = [C.c_int]
    lib.sla_last_cuda_error.restype = C.c_char_p
    lib.sla_launch_count.restype = C.c_longlong
    lib.sla_debug_set_trace.restype = C.c_int
    lib.sla_debug_set_trace.argtypes = [C.c_void_p]
    lib.sla_debug_set_wait_limit_ns.restype = C.c_int
    lib.sla_debug_set_wait_limit_ns.argtypes = [C.c_ulonglong]
    lib.sla_debug_drop_first_k_tile.restype = C.c_int
    lib.sla_debug_drop_first_k_tile.argtypes = [C.c_int]
    lib.sla_poll_device_error.restype = C.c_int
    lib.sla_poll_device_error.argtypes = [C.POINTER(C.c_int), C.c_int]
    lib.sla_topk_count.restype = C.c_int
    lib.sla_topk_count.argtypes = [C.c_int, C.c_double]
    lib.sla_kernel_path.restype = C.c_int
    lib.sla_kernel_path.argtypes = [sp, C.c_int]
    lib.sla_workspace_bytes.restype = C.c_size_t
    lib.sla_workspace_bytes.argtypes = [sp, C.c_int]
    lib.sla_block_map.restype = C.c_int
    lib.sla_block_map.argtypes = [sp, C.c_int, vp, vp, i32p, i8p, i32p, i32p, vp, C.c_size_t, vp]
    lib.sla_pooled_sums_bytes.restype = C.c_size_t
    lib.sla_pooled_sums_bytes.argtypes = [sp]
    lib.sla_qk_norm_rope_pool.restype = C.c_int
    lib.sla_qk_norm_rope_pool.argtypes = [sp, vp, vp, f32p, f32p, f32p, f32p, C.c_float, C.c_int, vp, vp, vp, C.c_size_t, vp]
    lib.sla_block_map_pooled.restype = C.c_int
    lib.sla_block_map_pooled.argtypes = [sp, vp, i32p, i8p, i32p, i32p, vp, C.c_size_t, vp]
    lib.sla_index_convert.restype = C.c_int
    lib.sla_index_convert.argtypes = [vp, C.c_int, vp, C.c_int, C.c_size_t, vp]
    lib.sla_column_lists.restype = C.c_int
    lib.sla_column_lists.argtypes = [sp, i8p, i32p, i32p, vp]
    lib.sla_sparse_fwd.restype = C.c_int
    lib.sla_sparse_fwd.argtypes = [sp, vp, vp, vp, i32p, vp, f32p, vp]
    lib.sla_sparse_bwd.restype = C.c_int
    lib.sla_sparse_bwd.argtypes = [sp, vp, vp, vp, vp, f32p, vp, i32p, i32p, i32p, vp, vp, vp, vp, C.c_size_t, vp]
    lib.sla_linear_state.restype = C.c_int
    lib.sla_linear_state.argtypes = [sp, vp, vp, vp, vp, C.c_size_t, vp]
    lib.sla_linear_state_static.restype = C.c_int
    lib.sla_linear_state_static.argtypes = [sp, vp, vp, vp, vp]
    lib.sla_fwd_prepare.restype = C.c_int
    lib.sla_fwd_prepare.argtypes = [sp, vp, vp, f32p, f32p, vp, vp, C.c_size_t, vp]
    lib.sla_fwd.restype = C.c_int
    lib.sla_fwd.argtypes = [sp, vp, vp, vp, i32p, f32p, f32p, vp, vp, f32p, vp, vp, C.c_size_t, vp]
    lib.sla_fwd_gather.restype = C.c_int
    lib.sla_fwd_gather.argtypes = [sp, vp, vp, vp, i32p, f32p, f32p, vp, vp, f32p, vp, vp, C.c_size_t,
                                   C.POINTER(C.c_void_p), C.c_int, vp]
    lib.sla_ipc_export.restype = C.c_int
    lib.sla_ipc_export.argtypes = [C.c_void_p, C.c_char_p, C.POINTER(C.c_size_t)]
    lib.sla_ipc_open.restype = C.c_int
    lib.sla_ipc_open.argtypes = [C.c_char_p, C.POINTER(C.c_void_p)]
    lib.sla_ipc_close.restype = C.c_int
    lib.sla_ipc_close.argtypes = [C.c_void_p]
    lib.sla_enable_peer_access.restype = C.c_int
    lib.sla_enable_peer_access.argtypes = [C.c_int]
    lib.sla_bwd.restype = C.c_int
    lib.sla_bwd.argtypes = [sp, vp, vp, vp, vp, f32p, vp, i32p, i32p, i32p, f32p, vp, vp, vp, vp, f32p, f32p,
                            vp, C.c_size_t, vp]
    lib.sage_sla_prepare.restype = C.c_int
    lib.sage_sla_prepare.argtypes = [sp, vp, vp, vp, f32p, f32p, vp, vp, C.c_size_t, vp]
    lib.sage_sla_fwd_gather.restype = C.c_int
    lib.sage_sla_fwd_gather.argtypes = [sp, vp, vp, vp, i32p, f32p, f32p, vp, vp, vp, C.c_size_t,
                                        C.POINTER(C.c_void_p), C.c_int, vp]
    lib.sage_sla_fwd.restype = C.c_int
    lib.sage_sla_fwd.argtypes = [sp, vp, vp, vp, i32p, f32p, f32p, vp, vp, vp, C.c_size_t, vp]
    return lib


lib = _load()


def check(status: int) -> None:
    if status == 0:
        return
    text = lib.sla_status_string(status).decode()
    if status == -7:
        text += " -- " + lib.sla_last_cuda_error().decode()
    if status == -10:
        raise NotImplementedError(f"sla_b200 status {status}: {text}")
    raise SlaError(status, text)


def poll_device_error(clear: bool = True) -> int:
    """Synchronise and return the device error code of the tcgen05 kernels (0 = none)."""
    code = C.c_int(0)
    rc = lib.sla_poll_device_error(C.byref(code), 1 if clear else 0)
    if rc not in (0, -8):          # -8 = SLA_ERR_TIMEOUT: the code says which wait
        check(rc)
    return code.value


def raise_on_device_error() -> None:
    """Synchronise, and raise if a bounded device-side wait ran out since the last poll (the word is cleared)."""
    code = poll_device_error(clear=True)
    if code != 0:
        raise SlaError(-8, f"a device-side wait of a tcgen05 kernel ran out (code {code}); the outputs of that "
                           "launch and of every tcgen05 launch after it are not valid")


def topk_count(n_blocks: int, ratio: float) -> int:
    return int(lib.sla_topk_count(int(n_blocks), float(ratio)))
