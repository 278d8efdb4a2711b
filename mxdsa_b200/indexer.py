"""Index selection on the GPU: score rows -> the ``indices`` / ``topk_length`` tensors of the attention
operators.

The reference has no producer for ``indices``; its callers fix the conventions (reference
tests/benchmark.py:119-147: int32 rows ``[s_q/2, 1, topk]`` for prefill with one row per PAIR of query
tokens, ``[b, s_q, topk]`` for decode with pool indices offset by ``request * pool_len``; -1 entries are
never attended; ``topk_length`` bounds the attended prefix).  ``select_topk_indices`` produces exactly
those tensors from score rows.  All compute is in libmxdsa.so (``mxdsa_topk_select``); there is no
fallback.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch

from . import capi


def select_topk_indices(scores: torch.Tensor, topk: int, lengths: Optional[torch.Tensor] = None,
                        pair: bool = False, row_offset: Optional[torch.Tensor] = None
                        ) -> Tuple[torch.Tensor, torch.Tensor]:
    """scores f32 [n, s_kv] (CUDA, s_kv a multiple of 4) -> (indices i32 [rows, topk], topk_length i32 [rows]).

    rows = n, or n/2 with ``pair=True`` (score rows 2r and 2r+1 are the two tokens of pair r; a key's
    score is the larger of the two).  Row r selects the min(topk, candidates) best keys among
    ``j < lengths[r]``; NaN and -inf scores are no candidates; ties go to the smaller j.  The selected
    indices are ascending, ``row_offset[r]`` is added to each, and the row is padded with -1.
    """
    if not scores.is_cuda or scores.dtype != torch.float32 or scores.dim() != 2:
        raise RuntimeError("scores must be a CUDA float32 tensor of shape [n, s_kv]")
    if scores.stride(1) != 1:
        scores = scores.contiguous()
    n, s_kv = scores.shape
    group = 2 if pair else 1
    if n % group:
        raise RuntimeError("pair=True needs an even number of score rows")
    if s_kv <= 0 or s_kv % 4 or topk <= 0:
        raise RuntimeError("s_kv must be a positive multiple of 4 and topk positive")
    rows = n // group
    dev = scores.device

    def opt(t, name):
        if t is None:
            return None
        if not t.is_cuda or t.dtype != torch.int32 or t.numel() != rows:
            raise RuntimeError(f"{name} must be a CUDA int32 tensor of {rows} elements")
        return t.contiguous()

    lengths, row_offset = opt(lengths, "lengths"), opt(row_offset, "row_offset")
    indices = torch.empty((rows, topk), dtype=torch.int32, device=dev)
    count = torch.empty((rows,), dtype=torch.int32, device=dev)
    if rows:
        p = capi.TopkParams(scores=scores.data_ptr(), score_stride=scores.stride(0),
                            lengths=lengths.data_ptr() if lengths is not None else None,
                            row_offset=row_offset.data_ptr() if row_offset is not None else None,
                            indices=indices.data_ptr(), index_stride=topk, topk_length=count.data_ptr(),
                            rows=rows, group=group, s_kv=s_kv, topk=topk,
                            stream=torch.cuda.current_stream(dev).cuda_stream)
        with torch.cuda.device(dev):
            capi.check(capi.lib().mxdsa_topk_select(C.byref(p)), "mxdsa_topk_select")
    return indices, count
