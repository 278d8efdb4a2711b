"""ctypes view of libmxdsa.so (the C ABI declared in include/mxdsa.h).

Raw device pointers in, status codes out.  The library is built in-tree by ``mxdsa_b200.build``;
if it is missing this module raises -- there is no fallback implementation.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libmxdsa.so")

EXPORTS = (
    "mxdsa_status_string", "mxdsa_last_cuda_error", "mxdsa_device_fault", "mxdsa_prefill_fwd",
    "mxdsa_num_sm_parts", "mxdsa_decode_sched", "mxdsa_decode_workspace_bytes", "mxdsa_decode_fwd",
    "mxdsa_decode_sched_whole", "mxdsa_decode_fwd_nocombine",
    "mxdsa_decode_fwd_static", "mxdsa_decode_combine", "mxdsa_pack_q", "mxdsa_pack_kv", "mxdsa_pack_last_cuda_error",
    "mxdsa_topk_select", "mxdsa_topk_last_cuda_error", "mxdsa_selftest_bounded_wait", "mxdsa_selftest_teardowns", "mxdsa_selftest_mma_rate",
)
DTYPE_BF16, DTYPE_F32 = 0, 1
STATIC_SCRATCH_BYTES = 32 << 20


class PrefillParams(C.Structure):
    _fields_ = [
        ("s_q", C.c_int32), ("s_kv", C.c_int32), ("topk", C.c_int32), ("sm_scale", C.c_float),
        ("q", C.c_void_p), ("stride_q_token", C.c_int64), ("kv", C.c_void_p),
        ("indices", C.c_void_p), ("stride_indices_pair", C.c_int64),
        ("attn_sink", C.c_void_p), ("topk_length", C.c_void_p),
        ("w1", C.c_uint32 * 8), ("w2", C.c_uint32 * 8),
        ("out", C.c_void_p), ("max_logits", C.c_void_p), ("lse", C.c_void_p), ("stream", C.c_void_p),
    ]


class SchedParams(C.Structure):
    _fields_ = [
        ("b", C.c_int32), ("s_q", C.c_int32), ("topk", C.c_int32), ("extra_topk", C.c_int32),
        ("topk_length", C.c_void_p), ("extra_topk_length", C.c_void_p), ("num_sm_parts", C.c_int32),
        ("sched_meta", C.c_void_p), ("num_splits", C.c_void_p), ("stream", C.c_void_p),
    ]


class DecodeParams(C.Structure):
    _fields_ = [
        ("b", C.c_int32), ("s_q", C.c_int32), ("topk", C.c_int32), ("extra_topk", C.c_int32),
        ("sm_scale", C.c_float),
        ("q", C.c_void_p), ("stride_q_b", C.c_int64), ("stride_q_s", C.c_int64),
        ("kv", C.c_void_p), ("num_blocks", C.c_int32), ("page_block_size", C.c_int32),
        ("stride_kv_block", C.c_int64),
        ("indices", C.c_void_p), ("stride_indices_b", C.c_int64), ("stride_indices_s", C.c_int64),
        ("topk_length", C.c_void_p), ("attn_sink", C.c_void_p),
        ("extra_kv", C.c_void_p), ("extra_num_blocks", C.c_int32), ("extra_page_block_size", C.c_int32),
        ("stride_extra_kv_block", C.c_int64),
        ("extra_indices", C.c_void_p), ("stride_extra_indices_b", C.c_int64),
        ("stride_extra_indices_s", C.c_int64), ("extra_topk_length", C.c_void_p),
        ("w1", C.c_uint32 * 8), ("w2", C.c_uint32 * 8),
        ("out", C.c_void_p), ("lse", C.c_void_p),
        ("sched_meta", C.c_void_p), ("num_splits", C.c_void_p), ("num_sm_parts", C.c_int32),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("stream", C.c_void_p),
    ]


class CombineParams(C.Structure):
    _fields_ = [
        ("b", C.c_int32), ("s_q", C.c_int32), ("num_sm_parts", C.c_int32),
        ("sched_meta", C.c_void_p), ("num_splits", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("attn_sink", C.c_void_p),
        ("out", C.c_void_p), ("lse", C.c_void_p), ("stream", C.c_void_p),
    ]


class PackQParams(C.Structure):
    _fields_ = [
        ("rows", C.c_int64), ("src", C.c_void_p), ("src_dtype", C.c_int32), ("src_stride_row", C.c_int64),
        ("dst", C.c_void_p), ("dst_stride_row", C.c_int64), ("paired_storage", C.c_int32), ("stream", C.c_void_p),
    ]


class PackKVParams(C.Structure):
    _fields_ = [
        ("rows", C.c_int64), ("src", C.c_void_p), ("src_dtype", C.c_int32), ("src_stride_row", C.c_int64),
        ("dst", C.c_void_p), ("rows_per_page", C.c_int32), ("dst_stride_page", C.c_int64), ("stream", C.c_void_p),
    ]


class TopkParams(C.Structure):
    _fields_ = [
        ("scores", C.c_void_p), ("score_stride", C.c_int64), ("lengths", C.c_void_p), ("row_offset", C.c_void_p),
        ("indices", C.c_void_p), ("index_stride", C.c_int64), ("topk_length", C.c_void_p),
        ("rows", C.c_int32), ("group", C.c_int32), ("s_kv", C.c_int32), ("topk", C.c_int32), ("stream", C.c_void_p),
    ]


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.isfile(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m mxdsa_b200.build`")
        L = C.CDLL(LIB_PATH)
        L.mxdsa_status_string.restype = C.c_char_p
        L.mxdsa_status_string.argtypes = [C.c_int]
        L.mxdsa_last_cuda_error.restype = C.c_int
        L.mxdsa_device_fault.argtypes = [C.c_void_p]
        L.mxdsa_prefill_fwd.argtypes = [C.POINTER(PrefillParams)]
        L.mxdsa_num_sm_parts.argtypes = [C.c_int, C.c_int]
        L.mxdsa_decode_sched.argtypes = [C.POINTER(SchedParams)]
        L.mxdsa_decode_sched_whole.argtypes = [C.POINTER(SchedParams)]
        L.mxdsa_decode_workspace_bytes.restype = C.c_size_t
        L.mxdsa_decode_workspace_bytes.argtypes = [C.c_int, C.c_int, C.c_int]
        L.mxdsa_decode_fwd.argtypes = [C.POINTER(DecodeParams)]
        L.mxdsa_decode_fwd_nocombine.argtypes = [C.POINTER(DecodeParams)]
        L.mxdsa_decode_fwd_static.argtypes = [C.POINTER(DecodeParams)]
        L.mxdsa_decode_combine.argtypes = [C.POINTER(CombineParams)]
        L.mxdsa_pack_q.argtypes = [C.POINTER(PackQParams)]
        L.mxdsa_pack_kv.argtypes = [C.POINTER(PackKVParams)]
        L.mxdsa_pack_last_cuda_error.restype = C.c_int
        L.mxdsa_topk_select.argtypes = [C.POINTER(TopkParams)]
        L.mxdsa_topk_last_cuda_error.restype = C.c_int
        L.mxdsa_selftest_bounded_wait.argtypes = [C.c_void_p]
        L.mxdsa_selftest_teardowns.argtypes = [C.c_void_p]
        L.mxdsa_selftest_mma_rate.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p]
        _lib = L
    return _lib


def check(status: int, what: str) -> None:
    if status != 0:
        L = lib()
        msg = L.mxdsa_status_string(status).decode()
        raise RuntimeError(f"{what}: {msg} (status {status}, cuda error {L.mxdsa_last_cuda_error()})")
