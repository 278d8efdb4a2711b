"""Packers for the uint8 wire format of the two entry points (torch, CPU or CUDA tensors).

Same format and the same function names / return values as the reference's helpers
(reference tests/mxfp8_test_utils.py:30-104):

  Q          [..., 64, 528]  512 E4M3 bytes + 8 UE8M0 scale bytes stored twice.  Scale g is shared
                             by the 32-wide chunks [32g,32g+32) and [256+32g,256+32g+32).
  prefill KV [s_kv, 1, 528]  view of one flat buffer: all 512-byte data rows, then all 16-byte
                             scale slots (8 UE8M0 bytes, one per 64 dims, stored twice).
  decode KV  [pages, page, 1, 528]  per page: page*512 data bytes, then page*16 slot bytes.

Every scale is 2^ceil(log2(max(amax/448, 2^-126))); values are divided by it, clamped to +-448
and cast to E4M3.

``pack_dual_q64(..., paired_storage=True)`` stores the data bytes in the order in which the
kernel contracts them with K's natural dimension order ([g][half][32]); the default keeps the
reference packer's natural order.  ``make_rank1_kv`` draws KV whose group scales factor as
token scale x dimension scale, which is what the V path of the kernel assumes, and returns the
matching ``w1``/``w2`` words.
"""
from __future__ import annotations

from typing import List, Tuple

import torch

D_HEAD = 512
FP8_MAX = 448.0
KV_GROUP_SIZE = 64


def _pow2_scale(amax: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    s = (amax / FP8_MAX).clamp_min(2.0 ** -126)
    e = torch.ceil(torch.log2(s))
    return torch.exp2(e), (e + 127).to(torch.uint8)


def _quantize(grouped: torch.Tensor):
    scale, sbyte = _pow2_scale(grouped.abs().amax(dim=-1))
    code = (grouped / scale.unsqueeze(-1)).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return code.view(torch.uint8), sbyte, code.float() * scale.unsqueeze(-1)


def pack_dual_q64(q: torch.Tensor, paired_storage: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    assert q.shape[-1] == D_HEAD
    lead = q.shape[:-1]
    paired = q.float().reshape(*lead, 2, 8, 32).transpose(-3, -2).reshape(*lead, 8, 64)
    code, sbyte, deq = _quantize(paired)
    natural = lambda t: t.reshape(*lead, 8, 2, 32).transpose(-3, -2).reshape(*lead, D_HEAD)
    packed = torch.empty((*lead, D_HEAD + 16), dtype=torch.uint8, device=q.device)
    packed[..., :D_HEAD] = code.reshape(*lead, D_HEAD) if paired_storage else natural(code)
    packed[..., D_HEAD:D_HEAD + 8] = sbyte
    packed[..., D_HEAD + 8:] = sbyte
    return packed, natural(deq)


def _quantize_kv(kv: torch.Tensor):
    g = kv.float().reshape(*kv.shape[:-1], D_HEAD // KV_GROUP_SIZE, KV_GROUP_SIZE)
    code, sbyte, deq = _quantize(g)
    return code.reshape(kv.shape), sbyte, deq.reshape(kv.shape)


def pack_dual_prefill_kv64(kv: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    assert kv.ndim == 3 and kv.shape[-1] == D_HEAD
    code, sbyte, deq = _quantize_kv(kv)
    n = kv.shape[0] * kv.shape[1]
    buf = torch.empty(n * (D_HEAD + 16), dtype=torch.uint8, device=kv.device)
    buf[: n * D_HEAD] = code.reshape(-1)
    buf[n * D_HEAD:] = torch.cat((sbyte, sbyte), dim=-1).reshape(-1)
    return buf.view(*kv.shape[:-1], D_HEAD + 16), deq


def pack_dual_decode_kv_pages(kv: torch.Tensor):
    assert kv.ndim == 4 and kv.shape[2] == 1 and kv.shape[-1] == D_HEAD
    pages, psz = kv.shape[:2]
    code, sbyte, deq = _quantize_kv(kv)
    buf = torch.empty((pages, psz * (D_HEAD + 16)), dtype=torch.uint8, device=kv.device)
    buf[:, : psz * D_HEAD] = code.reshape(pages, -1)
    buf[:, psz * D_HEAD:] = torch.cat((sbyte, sbyte), dim=-1).reshape(pages, -1)
    return (buf.view(pages, psz, 1, D_HEAD + 16), deq,
            sbyte.view(pages, psz, 1, D_HEAD // KV_GROUP_SIZE), code.view(pages, psz, 1, D_HEAD))


def w_words(log2_w: List[int]) -> Tuple[List[int], List[int]]:
    """w1/w2 for eight 64-wide dimension scales 2^log2_w[g]: one UE8M0 byte repeated four times
    per word, two words (2 x 32 dims) per 64-wide group."""
    words = [int((int(e) + 127) * 0x01010101) for e in log2_w]
    return [words[j // 2] for j in range(8)], [words[4 + j // 2] for j in range(8)]


def make_rank1_kv(shape, device="cpu", generator=None, log2_range: int = 2):
    """N(0,1) KV of shape [*shape, 512] rescaled per 64-wide group so that group g's quantisation
    scale is exactly (token scale) x 2^wl[g], wl[0] = 0.  Returns (kv fp32, w1, w2)."""
    x = torch.randn((*shape, D_HEAD), device=device, generator=generator)
    wl = torch.randint(-log2_range, log2_range + 1, (8,), generator=generator, device=device)
    wl[0] = 0
    g = x.reshape(*shape, 8, 64)
    e = torch.ceil(torch.log2((g.abs().amax(-1) / FP8_MAX).clamp_min(2.0 ** -126)))
    g = g * torch.exp2(e[..., :1] + wl - e).unsqueeze(-1)
    w1, w2 = w_words(wl.tolist())
    return g.reshape(*shape, D_HEAD), w1, w2
