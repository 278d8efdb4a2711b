"""Fused quantise-and-pack on the GPU: one kernel per tensor instead of the chain of torch kernels
that the reference's helpers launch (reference tests/mxfp8_test_utils.py:30-104).

Same function names as those helpers and byte-identical packed tensors for the same input values;
the dequantised copy that the helpers also return is not produced here (``mxdsa_b200.packing``
keeps the torch versions, which do).  Inputs: CUDA tensors, bf16 or fp32, last dimension 512 and
contiguous.  All compute is in libmxdsa.so (``mxdsa_pack_q`` / ``mxdsa_pack_kv``); there is no
fallback.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import capi

D = 512
ROW = 528


def _src(t: torch.Tensor, name: str):
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be on CUDA")
    if t.dtype not in (torch.bfloat16, torch.float32):
        raise RuntimeError(f"{name} must be bf16 or fp32")
    if t.dim() < 2 or t.size(-1) != D:
        raise RuntimeError(f"{name} must have a last dimension of {D}")
    t = t.contiguous()
    return t, (capi.DTYPE_BF16 if t.dtype == torch.bfloat16 else capi.DTYPE_F32)


def pack_dual_q64(q: torch.Tensor, paired_storage: bool = False) -> torch.Tensor:
    """q [..., 64, 512] -> u8 [..., 64, 528]: 512 E4M3 bytes + 8 UE8M0 scale bytes stored twice; scale g is
    shared by dims [32g,32g+32) and [256+32g,256+32g+32) (reference pack_dual_q64)."""
    src, dt = _src(q, "q")
    out = torch.empty((*src.shape[:-1], ROW), dtype=torch.uint8, device=src.device)
    rows = src.numel() // D
    p = capi.PackQParams(rows=rows, src=src.data_ptr(), src_dtype=dt, src_stride_row=D, dst=out.data_ptr(),
                         dst_stride_row=ROW, paired_storage=int(bool(paired_storage)),
                         stream=torch.cuda.current_stream(src.device).cuda_stream)
    with torch.cuda.device(src.device):
        capi.check(capi.lib().mxdsa_pack_q(C.byref(p)), "mxdsa_pack_q")
    return out


def pack_dual_prefill_kv64(kv: torch.Tensor) -> torch.Tensor:
    """kv [s_kv, 1, 512] -> u8 [s_kv, 1, 528] view of one flat buffer: all data rows, then all 16-byte scale
    slots; scale g covers dims [64g,64g+64) (reference pack_dual_prefill_kv64)."""
    if kv.dim() != 3 or kv.size(1) != 1:
        raise RuntimeError("kv must have shape [s_kv, 1, 512]")
    src, dt = _src(kv, "kv")
    n = src.size(0)
    out = torch.empty(n * ROW, dtype=torch.uint8, device=src.device)
    if n:
        p = capi.PackKVParams(rows=n, src=src.data_ptr(), src_dtype=dt, src_stride_row=D, dst=out.data_ptr(),
                              rows_per_page=n, dst_stride_page=0,
                              stream=torch.cuda.current_stream(src.device).cuda_stream)
        with torch.cuda.device(src.device):
            capi.check(capi.lib().mxdsa_pack_kv(C.byref(p)), "mxdsa_pack_kv")
    return out.view(n, 1, ROW)


def pack_dual_decode_kv_pages(kv: torch.Tensor) -> torch.Tensor:
    """kv [pages, page_size, 1, 512] -> u8 [pages, page_size, 1, 528]: per page, page_size*512 data bytes and
    then page_size 16-byte scale slots (reference pack_dual_decode_kv_pages)."""
    if kv.dim() != 4 or kv.size(2) != 1:
        raise RuntimeError("kv must have shape [pages, page_size, 1, 512]")
    src, dt = _src(kv, "kv")
    pages, psz = src.size(0), src.size(1)
    out = torch.empty((pages, psz * ROW), dtype=torch.uint8, device=src.device)
    if pages * psz:
        p = capi.PackKVParams(rows=pages * psz, src=src.data_ptr(), src_dtype=dt, src_stride_row=D,
                              dst=out.data_ptr(), rows_per_page=psz, dst_stride_page=psz * ROW,
                              stream=torch.cuda.current_stream(src.device).cuda_stream)
        with torch.cuda.device(src.device):
            capi.check(capi.lib().mxdsa_pack_kv(C.byref(p)), "mxdsa_pack_kv")
    return out.view(pages, psz, 1, ROW)
