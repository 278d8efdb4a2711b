"""CPU baseline of the path for bench.py.  TEST / MEASUREMENT INFRASTRUCTURE ONLY.

The reference project has no CPU implementation of its kernels.  The CPU path that its inputs
define -- and that BASELINE.json names as the host-core comparator -- is the torch
"dequantise-and-gather" computation: de-quantise the packed KV once, and per query pair gather the
selected rows, form fp32 logits, softmax, and multiply by V.  This module is that path, written
over the same operand reading as oracle/mxdsa_oracle.py (which Q bytes meet which K bytes, which
scale bytes apply; reference csrc/attention/common.cuh:84-113) but with torch fp32 matmuls on all
host threads so that it can be timed on a bounded sample.  It is a *port*, not the reference's
own code; the shipped library never imports it.
"""
from __future__ import annotations

import os
from typing import Optional, Sequence

import numpy as np
import torch

from . import mxdsa_oracle as O

_E4M3 = torch.from_numpy(np.nan_to_num(O.E4M3_TABLE, nan=0.0).astype(np.float32))


def _ue8m0(b: torch.Tensor) -> torch.Tensor:
    return torch.exp2(b.float() - 127.0)


def dequant_prefill_kv(kv_u8: torch.Tensor, w1: Sequence[int], w2: Sequence[int]):
    """[s_kv,1,528] envelope -> (K [s_kv,512], V [s_kv,512]) fp32, as the kernel reads them."""
    s_kv = kv_u8.shape[0]
    flat = kv_u8.reshape(-1)
    e = _E4M3[flat[: s_kv * 512].long()].view(s_kv, 512)
    slots = flat[s_kv * 512:].view(s_kv, 16)
    k = e * _ue8m0(slots[:, :8]).repeat_interleave(64, dim=1)
    wb = torch.tensor([w & 0xFF for w in list(w1) + list(w2)], dtype=torch.uint8)
    v = e * _ue8m0(slots[:, :1]) * _ue8m0(wb).repeat_interleave(32)[None, :]
    return k, v


def dequant_q(q_u8: torch.Tensor) -> torch.Tensor:
    """[n,64,528] -> fp32 [n,64,512] in the order in which the kernel contracts Q with K."""
    n = q_u8.shape[0]
    e = _E4M3[q_u8[..., :512].long()].view(n, 64, 8, 2, 32)
    e = e * _ue8m0(q_u8[..., 512:520])[..., None, None]
    return e.transpose(-3, -2).reshape(n, 64, 512)


@torch.no_grad()
def prefill_cpu(q_u8: torch.Tensor, k: torch.Tensor, v: torch.Tensor, indices: torch.Tensor, sm_scale: float,
                threads: Optional[int] = None) -> torch.Tensor:
    """Sparse attention of the given query tokens on host cores; q_u8 [s,64,528] (s even),
    indices [s/2,1,topk] (all valid).  Returns out fp32 [s,64,512]."""
    torch.set_num_threads(threads or os.cpu_count() or 1)
    s = q_u8.shape[0]
    qd = dequant_q(q_u8)
    out = torch.empty((s, 64, 512), dtype=torch.float32)
    for p in range(s // 2):
        idx = indices[p, 0].long()
        valid = idx >= 0
        idx = idx.clamp_min(0)
        kg, vg = k[idx], v[idx]
        logits = (qd[2 * p:2 * p + 2].reshape(128, 512) @ kg.t()) * sm_scale
        logits.masked_fill_(~valid[None, :], float("-inf"))
        prob = torch.softmax(logits, dim=-1)
        out[2 * p:2 * p + 2] = (prob @ vg).view(2, 64, 512)
    return out
