"""Operator API: the two entry points of the reference's extension module, same positional
arguments, same validation rules, same return values (reference csrc/bindings/binding.cpp:12-118
and csrc/bindings/dual_mxfp8_sparse_decode.h:13-243), implemented over the C ABI of libmxdsa.so.

torch is used for device memory and the current stream only; all compute is in the library.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence, Tuple

import torch

from . import capi

D = 512
ROW = 528
HEADS = 64
_SCHED_INTS = 8


def _req(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _opt_ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _check_opt(t: Optional[torch.Tensor], name: str, dtype, shape: Sequence[int]) -> None:
    if t is None:
        return
    _req(t.is_cuda, f"{name} must be on CUDA")
    _req(t.dtype == dtype, f"{name} must have dtype {dtype}")
    _req(tuple(t.shape) == tuple(shape), f"{name} must have shape {tuple(shape)}")
    _req(t.dim() == 0 or t.size(-1) == 1 or t.stride(-1) == 1, f"{name} must have contiguous last dimension")


def _words(w: Sequence[int], name: str):
    _req(len(w) == 8, "w1 and w2 must each contain 8 pre-expanded TMEM scale words")
    return (C.c_uint32 * 8)(*[int(x) & 0xFFFFFFFF for x in w])


def _stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def dual_mxfp8_head64_sparse_prefill_fwd(q: torch.Tensor, kv: torch.Tensor, indices: torch.Tensor,
                                         sm_scale: float, w1: Sequence[int], w2: Sequence[int],
                                         attn_sink: Optional[torch.Tensor] = None,
                                         topk_length: Optional[torch.Tensor] = None) -> List[torch.Tensor]:
    """Sparse MXFP8 prefill attention.  q u8 [s_q,64,528], kv u8 [s_kv,1,528] (contiguous
    envelope), indices i32 [s_q/2,1,topk]; returns [out bf16 [s_q,64,512], max_logits f32 [s_q,64],
    lse f32 [s_q,64]].  Does not synchronise."""
    return _prefill(q, kv, indices, sm_scale, w1, w2, attn_sink, topk_length, extended=False)


def dual_mxfp8_head64_sparse_prefill_fwd_ex(q: torch.Tensor, kv: torch.Tensor, indices: torch.Tensor,
                                            sm_scale: float, w1: Sequence[int], w2: Sequence[int],
                                            attn_sink: Optional[torch.Tensor] = None,
                                            topk_length: Optional[torch.Tensor] = None) -> List[torch.Tensor]:
    """The prefill operator without three restrictions of the reference's (which has no counterpart of
    this entry point): s_q may be odd (indices [ceil(s_q/2),1,topk]; the last pair then has one token),
    topk may be any positive number, and q / kv may be torch.float8_e4m3fn as well as uint8."""
    return _prefill(q, kv, indices, sm_scale, w1, w2, attn_sink, topk_length, extended=True)


def _prefill(q, kv, indices, sm_scale, w1, w2, attn_sink, topk_length, extended: bool) -> List[torch.Tensor]:
    _req(q.dim() == 3, "q must have 3 dimensions")
    _req(kv.dim() == 3, "kv must have 3 dimensions")
    _req(indices.dim() == 3, "indices must have 3 dimensions")
    s_q, h_q = q.size(0), q.size(1)
    s_kv, h_kv = kv.size(0), kv.size(1)
    topk = indices.size(2)
    _req(s_q > 0 and (extended or s_q % 2 == 0), "q must contain an even, positive number of query tokens")
    pairs = (s_q + 1) // 2
    _req(h_q == HEADS, "q must have shape [s_q, 64, 528]")
    _req(h_kv == 1, "kv must have shape [s_kv, 1, 528]")
    _req(q.size(2) == ROW, "q must store 512 E4M3 bytes followed by a replicated 16-byte UE8M0 scale slot per head")
    _req(kv.size(2) == ROW, "kv must provide a 528-byte envelope per token for replicated page-tail scales")
    _req(topk > 0 and (extended or topk % 64 == 0), "topk must be a positive multiple of 64")
    w1c, w2c = _words(w1, "w1"), _words(w2, "w2")
    for t, n in ((q, "q"), (kv, "kv"), (indices, "indices")):
        _req(t.is_cuda, f"{n} must be on CUDA")
    bytes_ok = (torch.uint8, torch.float8_e4m3fn) if extended else (torch.uint8,)
    _req(q.dtype in bytes_ok, "q must have dtype torch.uint8")
    _req(kv.dtype in bytes_ok, "kv must have dtype torch.uint8")
    _req(indices.dtype == torch.int32, "indices must have dtype torch.int32")
    _req(q.stride(-1) == 1, "q must have contiguous last dimension")
    _req(kv.is_contiguous(), "kv must be contiguous")
    _req(indices.stride(-1) == 1, "indices must have contiguous last dimension")
    _req(tuple(indices.shape) == (pairs, 1, topk), "indices must have shape (num_q_pairs, h_kv, topk)")
    _check_opt(attn_sink, "attn_sink", torch.float32, (HEADS,))
    _check_opt(topk_length, "topk_length", torch.int32, (pairs,))
    _req(q.stride(1) == ROW, "Q head stride must be 512 e4m3 bytes + an aligned 16-byte scale slot")
    for t in (q, indices):
        for st in t.stride():
            _req(st <= 2**31 - 1, f"Stride exceeds int32 limit: {st}")
    with torch.cuda.device(q.device):
        _req(torch.cuda.get_device_capability(q.device)[0] == 10,
             "Dual MXFP8 head64 sparse prefill requires SM100f.")
        out = torch.empty((s_q, h_q, D), dtype=torch.bfloat16, device=q.device)
        max_logits = torch.empty((s_q, h_q), dtype=torch.float32, device=q.device)
        lse = torch.empty((s_q, h_q), dtype=torch.float32, device=q.device)
        p = capi.PrefillParams(
            s_q=s_q, s_kv=s_kv, topk=topk, sm_scale=float(sm_scale), q=q.data_ptr(),
            stride_q_token=q.stride(0), kv=kv.data_ptr(), indices=indices.data_ptr(),
            stride_indices_pair=indices.stride(0), attn_sink=_opt_ptr(attn_sink),
            topk_length=_opt_ptr(topk_length), w1=w1c, w2=w2c, out=out.data_ptr(),
            max_logits=max_logits.data_ptr(), lse=lse.data_ptr(), stream=_stream_ptr(q.device))
        capi.check(capi.lib().mxdsa_prefill_fwd(C.byref(p)), "mxdsa_prefill_fwd")
    return [out, max_logits, lse]


def dual_mxfp8_sparse_decode_fwd(q: torch.Tensor, kv: torch.Tensor, indices: torch.Tensor,
                                 topk_length: Optional[torch.Tensor], attn_sink: Optional[torch.Tensor],
                                 tile_scheduler_metadata: Optional[torch.Tensor],
                                 num_splits: Optional[torch.Tensor], extra_kv: Optional[torch.Tensor],
                                 extra_indices: Optional[torch.Tensor],
                                 extra_topk_length: Optional[torch.Tensor], d_qk: int, d_v: int,
                                 sm_scale: float, w1: Sequence[int], w2: Sequence[int]
                                 ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Sparse MXFP8 decode attention with split-KV scheduling.  q [b,s_q,64,528], kv pages
    [blocks,page,1,528], indices i32 [b,s_q,topk] (global slot ids); optional extra cache.
    Returns (out bf16 [b,s_q,64,512], lse f32 as a [b,64,s_q] view, tile_scheduler_metadata i32
    [num_sm_parts,8], num_splits i32 [b+1]); the last two are computed when passed as None and can
    be passed back in on later calls with the same shapes and lengths."""
    return _decode(q, kv, indices, topk_length, attn_sink, tile_scheduler_metadata, num_splits, extra_kv,
                   extra_indices, extra_topk_length, d_qk, d_v, sm_scale, w1, w2, whole=False)


def dual_mxfp8_sparse_decode_fwd_whole(q: torch.Tensor, kv: torch.Tensor, indices: torch.Tensor,
                                 topk_length: Optional[torch.Tensor], attn_sink: Optional[torch.Tensor],
                                 tile_scheduler_metadata: Optional[torch.Tensor],
                                 num_splits: Optional[torch.Tensor], extra_kv: Optional[torch.Tensor],
                                 extra_indices: Optional[torch.Tensor],
                                 extra_topk_length: Optional[torch.Tensor], d_qk: int, d_v: int,
                                 sm_scale: float, w1: Sequence[int], w2: Sequence[int]
                                 ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """The decode operator without a combine pass (no counterpart in the reference): the schedule gives every
    request to one part (mxdsa_decode_sched_whole), the attention kernel writes all outputs itself, no scratch is
    allocated.  Same arguments and return values; scheduling tensors passed back in must come from this function."""
    return _decode(q, kv, indices, topk_length, attn_sink, tile_scheduler_metadata, num_splits, extra_kv,
                   extra_indices, extra_topk_length, d_qk, d_v, sm_scale, w1, w2, whole=True)


def _decode(q: torch.Tensor, kv: torch.Tensor, indices: torch.Tensor,
                                 topk_length: Optional[torch.Tensor], attn_sink: Optional[torch.Tensor],
                                 tile_scheduler_metadata: Optional[torch.Tensor],
                                 num_splits: Optional[torch.Tensor], extra_kv: Optional[torch.Tensor],
                                 extra_indices: Optional[torch.Tensor],
                                 extra_topk_length: Optional[torch.Tensor], d_qk: int, d_v: int,
                                 sm_scale: float, w1: Sequence[int], w2: Sequence[int], whole: bool = False
                                 ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Sparse MXFP8 decode attention with split-KV scheduling.  q [b,s_q,64,528], kv pages
    [blocks,page,1,528], indices i32 [b,s_q,topk] (global slot ids); optional extra cache.
    Returns (out bf16 [b,s_q,64,512], lse f32 as a [b,64,s_q] view, tile_scheduler_metadata i32
    [num_sm_parts,8], num_splits i32 [b+1]); the last two are computed when passed as None and can
    be passed back in on later calls with the same shapes and lengths."""
    _req(q.dim() == 4, "q must have 4 dimensions")
    _req(kv.dim() == 4, "kv must have 4 dimensions")
    _req(indices.dim() == 3, "indices must have 3 dimensions")
    b, s_q, h_q = q.size(0), q.size(1), q.size(2)
    num_blocks, page, h_kv = kv.size(0), kv.size(1), kv.size(2)
    topk = indices.size(2)
    have_extra = extra_kv is not None
    extra_topk = extra_indices.size(2) if extra_indices is not None else 0
    _req(b > 0 and s_q > 0, "b and s_q must be positive")
    _req(h_q == HEADS, f"Dual MXFP8 decode supports head64 only; got h_q={h_q}")
    _req(h_kv == 1, "Dual MXFP8 decode requires h_kv=1")
    _req(d_qk == D and d_v == D, "Dual MXFP8 decode requires d_qk=d_v=512")
    _req(topk > 0 and topk % 64 == 0, "topk must be a positive multiple of 64")
    w1c, w2c = _words(w1, "w1"), _words(w2, "w2")
    _req(q.size(3) == ROW, "q must use the 528-byte head64 envelope")
    _req(kv.size(3) == ROW, "kv must use the 528-byte head64 envelope")
    _req(not have_extra or extra_indices is not None, "extra_indices must be provided with extra_kv")
    _req(have_extra or (extra_indices is None and extra_topk_length is None), "extra indices require extra_kv")
    fp8 = (torch.uint8, torch.float8_e4m3fn)
    for t, n in ((q, "q"), (kv, "kv"), (indices, "indices"), (extra_kv, "extra_kv"),
                 (extra_indices, "extra_indices")):
        _req(t is None or t.is_cuda, f"{n} must be on CUDA")
    _req(q.dtype in fp8, "q must have E4M3 storage (uint8 or float8_e4m3fn)")
    _req(kv.dtype in fp8, "kv must have E4M3 storage (uint8 or float8_e4m3fn)")
    _req(not have_extra or extra_kv.dtype in fp8, "extra_kv must have E4M3 storage")
    _req(indices.dtype == torch.int32, "indices must have dtype torch.int32")
    _req(q.stride(-1) == 1, "q must have contiguous last dimension")
    _req(kv.is_contiguous(), "kv must be contiguous")
    _req(indices.stride(-1) == 1, "indices must have contiguous last dimension")
    _req(tuple(indices.shape) == (b, s_q, topk), "indices must have shape (b, s_q, topk)")
    _check_opt(topk_length, "topk_length", torch.int32, (b,))
    _check_opt(attn_sink, "attn_sink", torch.float32, (HEADS,))
    _check_opt(extra_topk_length, "extra_topk_length", torch.int32, (b,))
    if have_extra:
        _req(extra_kv.dim() == 4 and extra_kv.size(2) == 1 and extra_kv.size(3) == ROW,
             "extra_kv must have shape [blocks, page, 1, 528]")
        _req(extra_kv.stride(-1) == 1, "extra_kv must have contiguous last dimension")
        _req(extra_indices.dtype == torch.int32 and tuple(extra_indices.shape) == (b, s_q, extra_topk),
             "extra_indices must have shape (b, s_q, extra_topk)")
        _req(extra_topk == 0 or extra_indices.stride(-1) == 1, "extra_indices must have contiguous last dimension")
        _req(extra_kv.stride(1) == ROW, "dual extra KV row stride must be 528 bytes")
        _req(extra_kv.stride(0) % 512 == 0, "dual extra KV page stride must be divisible by 512 bytes")
    _req(kv.stride(1) == ROW, f"dual KV row stride must be 528 bytes, got {kv.stride(1)}")
    _req(kv.stride(0) % 512 == 0, f"dual KV page stride must be divisible by 512 bytes, got {kv.stride(0)}")
    _req(q.stride(2) == ROW, "Q head stride must be 512 e4m3 bytes + an aligned 16-byte scale slot")
    with torch.cuda.device(q.device):
        _req(torch.cuda.get_device_capability(q.device)[0] == 10, "Dual MXFP8 head64 decode requires SM100f.")
        L = capi.lib()
        stream = _stream_ptr(q.device)
        out = torch.empty((b, s_q, h_q, D), dtype=torch.bfloat16, device=q.device)
        lse = torch.empty((b, s_q, h_q), dtype=torch.float32, device=q.device)
        parts = L.mxdsa_num_sm_parts(q.device.index if q.device.index is not None else torch.cuda.current_device(), s_q)
        _req(parts > 0, "could not query the device")
        if tile_scheduler_metadata is None:
            tile_scheduler_metadata = torch.empty((parts, _SCHED_INTS), dtype=torch.int32, device=q.device)
            num_splits = torch.empty((b + 1,), dtype=torch.int32, device=q.device)
            sp = capi.SchedParams(b=b, s_q=s_q, topk=topk, extra_topk=extra_topk,
                                  topk_length=_opt_ptr(topk_length),
                                  extra_topk_length=_opt_ptr(extra_topk_length), num_sm_parts=parts,
                                  sched_meta=tile_scheduler_metadata.data_ptr(),
                                  num_splits=num_splits.data_ptr(), stream=stream)
            capi.check((L.mxdsa_decode_sched_whole if whole else L.mxdsa_decode_sched)(C.byref(sp)), "mxdsa_decode_sched")
        _check_opt(tile_scheduler_metadata, "tile_scheduler_metadata", torch.int32, (parts, _SCHED_INTS))
        _req(num_splits is not None, "num_splits must be provided with tile_scheduler_metadata")
        _check_opt(num_splits, "num_splits", torch.int32, (b + 1,))
        _req(tile_scheduler_metadata.is_contiguous() and num_splits.is_contiguous(),
             "scheduling tensors must be contiguous")
        ws_bytes = 0 if whole else L.mxdsa_decode_workspace_bytes(b, s_q, parts)
        workspace = torch.empty((ws_bytes,), dtype=torch.uint8, device=q.device)
        p = capi.DecodeParams(
            b=b, s_q=s_q, topk=topk, extra_topk=extra_topk, sm_scale=float(sm_scale),
            q=q.data_ptr(), stride_q_b=q.stride(0), stride_q_s=q.stride(1),
            kv=kv.data_ptr(), num_blocks=num_blocks, page_block_size=page, stride_kv_block=kv.stride(0),
            indices=indices.data_ptr(), stride_indices_b=indices.stride(0), stride_indices_s=indices.stride(1),
            topk_length=_opt_ptr(topk_length), attn_sink=_opt_ptr(attn_sink),
            extra_kv=_opt_ptr(extra_kv), extra_num_blocks=extra_kv.size(0) if have_extra else 0,
            extra_page_block_size=extra_kv.size(1) if have_extra else 0,
            stride_extra_kv_block=extra_kv.stride(0) if have_extra else 0,
            extra_indices=_opt_ptr(extra_indices) if have_extra else None,
            stride_extra_indices_b=extra_indices.stride(0) if have_extra else 0,
            stride_extra_indices_s=extra_indices.stride(1) if have_extra else 0,
            extra_topk_length=_opt_ptr(extra_topk_length), w1=w1c, w2=w2c,
            out=out.data_ptr(), lse=lse.data_ptr(), sched_meta=tile_scheduler_metadata.data_ptr(),
            num_splits=num_splits.data_ptr(), num_sm_parts=parts, workspace=None if whole else workspace.data_ptr(),
            workspace_bytes=ws_bytes, stream=stream)
        if whole:
            capi.check(L.mxdsa_decode_fwd_nocombine(C.byref(p)), "mxdsa_decode_fwd_nocombine")
            return out, lse.transpose(1, 2), tile_scheduler_metadata, num_splits
        capi.check(L.mxdsa_decode_fwd(C.byref(p)), "mxdsa_decode_fwd")
        # the workspace is consumed by kernels already queued on this stream; record that use so
        # the caching allocator does not hand it to another stream before they finish
        workspace.record_stream(torch.cuda.current_stream(q.device))
    return out, lse.transpose(1, 2), tile_scheduler_metadata, num_splits


def device_fault() -> None:
    """Synchronise the current stream and raise if a kernel abandoned one of its bounded waits."""
    capi.check(capi.lib().mxdsa_device_fault(_stream_ptr(torch.cuda.current_device())), "device check")
