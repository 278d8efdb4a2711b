"""mxdsa_b200: B200-native MXFP8 DeepSeek-Sparse-Attention (prefill + split-KV decode).

Public surface = the two operator entry points of the reference extension plus the packers that
define the uint8 wire format.  The compute lives in ``lib/libmxdsa.so`` (C ABI, include/mxdsa.h);
import fails loudly on first use if that library has not been built.
"""
from .api import (device_fault, dual_mxfp8_head64_sparse_prefill_fwd,  # noqa: F401
                  dual_mxfp8_sparse_decode_fwd)

__all__ = ["dual_mxfp8_head64_sparse_prefill_fwd", "dual_mxfp8_sparse_decode_fwd", "device_fault"]
