"""mxdsa_b200: B200-native MXFP8 DeepSeek-Sparse-Attention (prefill + split-KV decode).

Public surface = the two operator entry points of the reference extension plus the packers that
define the uint8 wire format:

    dual_mxfp8_head64_sparse_prefill_fwd(q, kv, indices, sm_scale, w1, w2, attn_sink, topk_length)
    dual_mxfp8_sparse_decode_fwd(q, kv, indices, topk_length, attn_sink, tile_scheduler_metadata,
                                 num_splits, extra_kv, extra_indices, extra_topk_length,
                                 d_qk, d_v, sm_scale, w1, w2)

They come from the C++ extension module ``lib/mxdsa_ext.so`` (``ext``; importable as ``mxdsa_ext``,
the reference's module name, or as ``mxdsa_b200_ext``), which calls the C ABI of
``lib/libmxdsa.so`` (include/mxdsa.h).  ``mxdsa_b200.api`` holds the same two functions written
against the C ABI with ctypes.  All compute is in the CUDA library; if it has not been built
(``python -m mxdsa_b200.build``) the first call raises -- there is no fallback path.
"""
from __future__ import annotations

import importlib.util
import os

from . import api, capi, packing  # noqa: F401

_EXT_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "mxdsa_ext.so")
_ext = None


def ext():
    """The compiled extension module (loaded on first use)."""
    global _ext
    if _ext is None:
        if not os.path.isfile(_EXT_PATH):
            raise RuntimeError(f"{_EXT_PATH} is missing: build it with `python -m mxdsa_b200.build`")
        import torch  # noqa: F401  (libtorch must be loaded before the extension)
        spec = importlib.util.spec_from_file_location("mxdsa_b200_ext", _EXT_PATH)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        _ext = mod
    return _ext


def dual_mxfp8_head64_sparse_prefill_fwd(q, kv, indices, sm_scale, w1, w2, attn_sink=None, topk_length=None):
    return ext().dual_mxfp8_head64_sparse_prefill_fwd(q, kv, indices, sm_scale, list(w1), list(w2), attn_sink,
                                                      topk_length)


def dual_mxfp8_head64_sparse_prefill_fwd_ex(q, kv, indices, sm_scale, w1, w2, attn_sink=None, topk_length=None):
    """The prefill operator with an odd number of query tokens, any positive topk and float8_e4m3fn inputs allowed
    (no counterpart in the reference; indices [ceil(s_q/2), 1, topk])."""
    return ext().dual_mxfp8_head64_sparse_prefill_fwd_ex(q, kv, indices, sm_scale, list(w1), list(w2), attn_sink,
                                                         topk_length)


def dual_mxfp8_sparse_decode_fwd(q, kv, indices, topk_length, attn_sink, tile_scheduler_metadata, num_splits,
                                 extra_kv, extra_indices, extra_topk_length, d_qk, d_v, sm_scale, w1, w2):
    return ext().dual_mxfp8_sparse_decode_fwd(q, kv, indices, topk_length, attn_sink, tile_scheduler_metadata,
                                              num_splits, extra_kv, extra_indices, extra_topk_length, d_qk, d_v,
                                              sm_scale, list(w1), list(w2))


def dual_mxfp8_sparse_decode_fwd_whole(q, kv, indices, topk_length, attn_sink, tile_scheduler_metadata, num_splits,
                                       extra_kv, extra_indices, extra_topk_length, d_qk, d_v, sm_scale, w1, w2):
    """The decode operator without a combine pass: every request is given to one part, no scratch is allocated
    (no counterpart in the reference; same arguments and return values as dual_mxfp8_sparse_decode_fwd)."""
    return ext().dual_mxfp8_sparse_decode_fwd_whole(q, kv, indices, topk_length, attn_sink, tile_scheduler_metadata,
                                                    num_splits, extra_kv, extra_indices, extra_topk_length, d_qk, d_v,
                                                    sm_scale, list(w1), list(w2))


def device_fault() -> None:
    """Synchronise the current stream; raise if a kernel abandoned one of its bounded waits."""
    ext().device_fault()


__all__ = ["dual_mxfp8_head64_sparse_prefill_fwd", "dual_mxfp8_head64_sparse_prefill_fwd_ex",
           "dual_mxfp8_sparse_decode_fwd", "dual_mxfp8_sparse_decode_fwd_whole", "device_fault", "ext", "api",
           "capi", "packing"]
