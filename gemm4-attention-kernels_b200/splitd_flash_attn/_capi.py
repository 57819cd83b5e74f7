"""ctypes binding of libsplitd_attn.so (the C-ABI declared in include/splitd_attn.h).

The library is built in-tree by ``build.py`` (nvcc, sm_100a). There is no fallback: if the
shared object is missing or a call fails, an exception is raised.
"""

from __future__ import annotations

import ctypes
import os
from typing import Optional

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(os.path.dirname(_PKG_DIR), "csrc", "libsplitd_attn.so")

SPLITD_DTYPE_BF16 = 0
SPLITD_DTYPE_FP16 = 1

EXPORTED_SYMBOLS = (
    "splitd_device_supported",
    "splitd_fwd",
    "splitd_fwd_workspace_bytes",
    "splitd_bwd_rowstat_elems",
    "splitd_out_resid_bytes",
    "splitd_bwd_workspace_bytes",
    "splitd_bwd_workspace_bytes_limit",
    "splitd_bwd_num_chunks",
    "splitd_bwd_chunk",
    "splitd_wait_probe",
    "splitd_bwd_preprocess",
    "splitd_bwd_dq",
    "splitd_bwd_dkdv",
    "splitd_bwd_tiles",
    "splitd_bwd_grads",
    "splitd_bwd",
    "splitd_bwd_static_scratch",
    "splitd_bwd_static_scratch_limit_rowstat",
    "splitd_bwd_static_scratch_limit_workspace",
    "splitd_last_error",
    "splitd_version",
)


class SplitdParams(ctypes.Structure):
    """Mirror of ``splitd_params`` (include/splitd_attn.h); field order must match."""

    _fields_ = [
        ("q", ctypes.c_void_p),
        ("k", ctypes.c_void_p),
        ("v", ctypes.c_void_p),
        ("o", ctypes.c_void_p),
        ("lse", ctypes.c_void_p),
        ("dout", ctypes.c_void_p),
        ("dlse", ctypes.c_void_p),
        ("dq", ctypes.c_void_p),
        ("dk", ctypes.c_void_p),
        ("dv", ctypes.c_void_p),
        ("dpsum", ctypes.c_void_p),
        ("lse_log2", ctypes.c_void_p),
        ("workspace", ctypes.c_void_p),
        ("workspace_bytes", ctypes.c_size_t),
        ("cu_seqlens_q", ctypes.c_void_p),
        ("cu_seqlens_k", ctypes.c_void_p),
        ("batch", ctypes.c_int32),
        ("seqlen_q", ctypes.c_int32),
        ("seqlen_k", ctypes.c_int32),
        ("total_q", ctypes.c_int32),
        ("total_k", ctypes.c_int32),
        ("max_seqlen_q", ctypes.c_int32),
        ("max_seqlen_k", ctypes.c_int32),
        ("heads_q", ctypes.c_int32),
        ("heads_kv", ctypes.c_int32),
        ("head_dim", ctypes.c_int32),
        ("q_strides", ctypes.c_int64 * 3),
        ("k_strides", ctypes.c_int64 * 3),
        ("v_strides", ctypes.c_int64 * 3),
        ("o_strides", ctypes.c_int64 * 3),
        ("do_strides", ctypes.c_int64 * 3),
        ("dq_strides", ctypes.c_int64 * 3),
        ("dk_strides", ctypes.c_int64 * 3),
        ("dv_strides", ctypes.c_int64 * 3),
        ("softmax_scale", ctypes.c_float),
        ("causal", ctypes.c_int32),
        ("dtype", ctypes.c_int32),
        ("status_flag", ctypes.c_void_p),
        ("debug", ctypes.c_void_p),
        ("softcap", ctypes.c_float),
        ("local", ctypes.c_int32),
        ("window_left", ctypes.c_int32),
        ("window_right", ctypes.c_int32),
        ("o_resid", ctypes.c_void_p),
        ("o_resid_all", ctypes.c_int32),
    ]


class SplitdError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"splitd_attn error {code}: {message}")
        self.code = code


_lib: Optional[ctypes.CDLL] = None


def load_library() -> ctypes.CDLL:
    """Load the shared object once; raise if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} not found: build it with `python gemm4-attention-kernels_b200/build.py` "
            "(there is no CPU or PyTorch fallback for the attention kernels)"
        )
    lib = ctypes.CDLL(LIB_PATH)
    pp = ctypes.POINTER(SplitdParams)
    lib.splitd_device_supported.argtypes = [ctypes.c_int]
    lib.splitd_device_supported.restype = ctypes.c_int
    for name in (
        "splitd_fwd",
        "splitd_bwd_preprocess",
        "splitd_bwd_dq",
        "splitd_bwd_dkdv",
        "splitd_bwd_tiles",
        "splitd_bwd_grads",
        "splitd_bwd",
        "splitd_bwd_static_scratch",
    ):
        fn = getattr(lib, name)
        fn.argtypes = [pp, ctypes.c_void_p]
        fn.restype = ctypes.c_int
    for name in (
        "splitd_fwd_workspace_bytes",
        "splitd_bwd_rowstat_elems",
        "splitd_out_resid_bytes",
        "splitd_bwd_workspace_bytes",
    ):
        fn = getattr(lib, name)
        fn.argtypes = [pp]
        fn.restype = ctypes.c_size_t
    lib.splitd_bwd_workspace_bytes_limit.argtypes = [pp, ctypes.c_size_t]
    lib.splitd_bwd_workspace_bytes_limit.restype = ctypes.c_size_t
    lib.splitd_bwd_num_chunks.argtypes = [pp]
    lib.splitd_bwd_num_chunks.restype = ctypes.c_int
    lib.splitd_bwd_chunk.argtypes = [pp, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    lib.splitd_bwd_chunk.restype = ctypes.c_int
    lib.splitd_wait_probe.argtypes = [ctypes.c_void_p, ctypes.c_uint, ctypes.c_void_p, ctypes.c_void_p]
    lib.splitd_wait_probe.restype = ctypes.c_int
    for name in ("splitd_bwd_static_scratch_limit_rowstat", "splitd_bwd_static_scratch_limit_workspace"):
        fn = getattr(lib, name)
        fn.argtypes = []
        fn.restype = ctypes.c_size_t
    lib.splitd_last_error.restype = ctypes.c_char_p
    lib.splitd_version.restype = ctypes.c_char_p
    _lib = lib
    return lib


def check(code: int) -> None:
    if code != 0:
        msg = load_library().splitd_last_error().decode("utf-8", "replace")
        raise SplitdError(code, msg)
