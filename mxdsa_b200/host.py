"""Prefill for callers whose tensors live in (pinned) host memory.

The operator itself takes device tensors, like the reference's.  A caller that holds Q, the index rows
and the outputs on the host pays PCIe for 2.76 GB in and 4.33 GB out per 65 536-token step -- several
times the kernel time -- so the only sensible way to drive the operator from host buffers is in chunks,
with the copy-in of chunk i+1, the attention of chunk i and the copy-out of chunk i-1 in flight at the
same time (PCIe is full duplex).  ``prefill_from_host`` does that with two extra streams and two
device staging buffers; the compute runs on the caller's current stream through the public entry
point ``dual_mxfp8_head64_sparse_prefill_fwd``.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

_state = {}


def _streams(device):
    key = torch.device(device).index
    if key not in _state:
        _state[key] = (torch.cuda.Stream(device=device), torch.cuda.Stream(device=device))
    return _state[key]


def prefill_from_host(hq: torch.Tensor, hkv: torch.Tensor, hidx: torch.Tensor, sm_scale: float, w1: Sequence[int],
                      w2: Sequence[int], h_out: torch.Tensor, h_max_logits: torch.Tensor, h_lse: torch.Tensor,
                      attn_sink: Optional[torch.Tensor] = None, chunk_tokens: int = 8192, device=None) -> None:
    """hq u8 [s_q,64,528], hkv u8 [s_kv,1,528], hidx i32 [s_q/2,1,topk] in pinned host memory; results are
    written to the pinned host tensors h_out bf16 [s_q,64,512], h_max_logits / h_lse f32 [s_q,64].
    Returns when everything has been enqueued; the caller's current stream is ordered after the last
    copy-out, so synchronising that stream (or an event recorded on it) is enough."""
    from . import dual_mxfp8_head64_sparse_prefill_fwd as prefill
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    assert chunk_tokens % 2 == 0 and hq.size(0) % 2 == 0
    s_q, topk = hq.size(0), hidx.size(-1)
    cur = torch.cuda.current_stream(device)
    s_in, s_out = _streams(device)
    s_in.wait_stream(cur)
    s_out.wait_stream(cur)
    n_max = min(chunk_tokens, s_q)
    with torch.cuda.stream(s_in):
        dkv = hkv.to(device, non_blocking=True)
        dq = [torch.empty((n_max, 64, 528), dtype=torch.uint8, device=device) for _ in range(2)]
        didx = [torch.empty((n_max // 2, 1, topk), dtype=torch.int32, device=device) for _ in range(2)]
    done = []     # per chunk: event "attention of the chunk has finished"
    for c, a in enumerate(range(0, s_q, n_max)):
        b, n = c % 2, min(n_max, s_q - a)
        with torch.cuda.stream(s_in):
            if c >= 2:
                s_in.wait_event(done[c - 2])        # the staging buffer's previous tenant has been consumed
            dq[b][:n].copy_(hq[a:a + n], non_blocking=True)
            didx[b][:n // 2].copy_(hidx[a // 2:(a + n) // 2], non_blocking=True)
            landed = torch.cuda.Event()
            landed.record(s_in)
        cur.wait_event(landed)
        o, mxl, lse = prefill(dq[b][:n], dkv, didx[b][:n // 2], sm_scale, w1, w2, attn_sink, None)
        ev = torch.cuda.Event()
        ev.record(cur)
        done.append(ev)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev)
            h_out[a:a + n].copy_(o, non_blocking=True)
            h_max_logits[a:a + n].copy_(mxl, non_blocking=True)
            h_lse[a:a + n].copy_(lse, non_blocking=True)
        for t in (o, mxl, lse):
            t.record_stream(s_out)
    for t in (dkv, *dq, *didx):
        t.record_stream(cur)
    cur.wait_stream(s_out)
    cur.wait_stream(s_in)
