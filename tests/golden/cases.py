"""Seeded input generators for the golden fixtures and the parity tests (numpy only).

Every case is a pure function of its name: ``build(name)`` returns the packed uint8 tensors, index
tensors and scalars that go into one call of the prefill or decode entry point.  The same
function is used
  * on the GPU box by ``gen_golden.py`` to feed the compiled reference, and
  * by the tests to rebuild bit-identical inputs for the oracle and for the CUDA library,
so the fixtures only have to store the reference's OUTPUTS (plus a hash of the inputs).

Shapes follow the reference benchmark (tests/benchmark.py:119-147 of the reference project):
64 query heads, one 512-wide MXFP8 latent KV head, pair-shared prefill index rows
[s_q/2, 1, topk], decode pools of 64-token pages addressed by global slot id.
"""
from __future__ import annotations

import hashlib
import os
import sys
from typing import Dict

import numpy as np

sys.path.insert(0, os.path.abspath(os.path.join(os.path.dirname(__file__), "..", "..")))
from oracle import mxdsa_oracle as O  # noqa: E402

PAGE = 64


def _distinct_rows(rng, rows: int, pool: int, topk: int) -> np.ndarray:
    out = np.empty((rows, topk), dtype=np.int32)
    for r in range(rows):
        if topk <= pool:
            out[r] = rng.permutation(pool)[:topk]
        else:
            out[r] = rng.integers(0, pool, size=topk)
    return out


def _bf16_normal(rng, shape) -> np.ndarray:
    return O.bf16_round(rng.standard_normal(shape, dtype=np.float32))


# Inputs are produced in slabs of a few hundred thousand elements: the temporaries of the
# quantiser then stay small and the generators run at memory speed on any host.
def _packed_q(rng, lead: tuple, gain: float = 1.0, slab: int = 16) -> np.ndarray:
    n = int(np.prod(lead))
    out = np.empty((n, 64, O.ROW_BYTES), dtype=np.uint8)
    for i in range(0, n, slab):
        m = min(slab, n - i)
        out[i:i + m] = O.pack_q(_bf16_normal(rng, (m, 64, O.D)) * np.float32(gain))[0]
    return out.reshape(*lead, 64, O.ROW_BYTES)


def _draw_wl(rng) -> np.ndarray:
    wl = rng.integers(-2, 3, size=8)
    wl[0] = 0
    return wl


def _packed_pages(rng, pages: int, wl: np.ndarray, slab: int = 16) -> np.ndarray:
    out = np.empty((pages, PAGE, 1, O.ROW_BYTES), dtype=np.uint8)
    for i in range(0, pages, slab):
        m = min(slab, pages - i)
        kv, _, _ = O.rank1_kv(rng, (m, PAGE, 1), wl=wl)
        out[i:i + m] = O.pack_decode_kv_pages(O.bf16_round(kv))[0]
    return out


PREFILL_CASES: Dict[str, dict] = {
    # BASELINE config 0: sq=256, kv_len=1024, topk=128 (64-token tile variant), seed 0
    "prefill_cfg0": dict(seed=0, s_q=256, s_kv=1024, topk=128),
    # 128-token tile variant (topk >= 512) with sink, per-pair lengths, invalid indices
    "prefill_t128_masked": dict(seed=1, s_q=64, s_kv=2048, topk=512, sink=True, lengths=True,
                                invalid=True),
    # topk multiple of 64 but not of 128, large-tile variant (half-empty last tile)
    "prefill_t128_ragged": dict(seed=2, s_q=32, s_kv=4096, topk=640, invalid=True),
    # small-tile variant, three tiles, sink, peaked attention (larger logits)
    "prefill_t64_peaked": dict(seed=3, s_q=32, s_kv=512, topk=192, sink=True, q_gain=4.0),
    # many tiles: exercises the running-max rescale across a long row
    "prefill_long": dict(seed=4, s_q=16, s_kv=16384, topk=4096, q_gain=2.0),
}

DECODE_CASES: Dict[str, dict] = {
    # MTP-style: main cache 128 tokens with topk 128, extra cache with extra topk
    "decode_mtp": dict(seed=10, b=4, s_q=6, main_len=128, topk=128, extra_len=1024, extra_topk=256),
    # odd s_q, per-request lengths, sink, invalid indices, extra_topk not a multiple of 64
    "decode_ragged": dict(seed=11, b=3, s_q=5, main_len=128, topk=128, extra_len=512,
                          extra_topk=200, sink=True, lengths=True, invalid=True),
    # no extra cache
    "decode_main_only": dict(seed=12, b=2, s_q=2, main_len=512, topk=256),
    # many requests per sm-part and splits that straddle parts (b > num_sm_parts on a B200)
    "decode_many": dict(seed=13, b=40, s_q=6, main_len=128, topk=128, extra_len=1024,
                        extra_topk=1024),
    # single query token
    "decode_sq1": dict(seed=14, b=5, s_q=1, main_len=128, topk=64, extra_len=256, extra_topk=128,
                       sink=True),
}


def build_prefill(name: str) -> dict:
    c = PREFILL_CASES[name]
    rng = np.random.default_rng(c["seed"])
    s_q, s_kv, topk = c["s_q"], c["s_kv"], c["topk"]
    q_u8 = _packed_q(rng, (s_q,), c.get("q_gain", 1.0))
    kv, w1, w2 = O.rank1_kv(rng, (s_kv, 1), wl=_draw_wl(rng))
    kv_u8, _ = O.pack_prefill_kv(O.bf16_round(kv))
    idx = _distinct_rows(rng, s_q // 2, s_kv, topk)[:, None, :]
    if c.get("invalid"):
        m = rng.random(idx.shape) < 0.1
        idx = np.where(m, -1, idx).astype(np.int32)
        m2 = rng.random(idx.shape) < 0.02
        idx = np.where(m2, s_kv + rng.integers(0, 1000, idx.shape), idx).astype(np.int32)
        idx[-1, 0, :] = -1  # one pair without any valid key
    sink = (rng.standard_normal(64) * 2).astype(np.float32) if c.get("sink") else None
    lengths = None
    if c.get("lengths"):
        lengths = rng.integers(1, topk + 1, size=s_q // 2).astype(np.int32)
        lengths[0] = 0
        lengths[1] = topk
        lengths[2] = 65
    return dict(kind="prefill", q=q_u8, kv=kv_u8, indices=np.ascontiguousarray(idx),
                sm_scale=float(O.D ** -0.5), w1=w1, w2=w2, attn_sink=sink, topk_length=lengths)


def build_decode(name: str) -> dict:
    c = DECODE_CASES[name]
    rng = np.random.default_rng(c["seed"])
    b, s_q, topk = c["b"], c["s_q"], c["topk"]
    main_len, extra_len, etopk = c["main_len"], c.get("extra_len", 0), c.get("extra_topk", 0)
    q_u8 = _packed_q(rng, (b, s_q))
    # one rank-1 dimension-scale vector shared by both pools (w1/w2 are per call)
    wl = _draw_wl(rng)
    w1, w2 = O.w_log2_to_words(wl)
    kv_u8 = _packed_pages(rng, b * main_len // PAGE, wl)
    off = (np.arange(b, dtype=np.int32) * main_len)[:, None, None]
    idx = _distinct_rows(rng, b * s_q, main_len, topk).reshape(b, s_q, topk) + off
    out = dict(kind="decode", q=q_u8, kv=kv_u8, sm_scale=float(O.D ** -0.5), w1=w1, w2=w2,
               extra_kv=None, extra_indices=None, extra_topk_length=None, topk_length=None,
               attn_sink=None)
    if etopk:
        ekv_u8 = _packed_pages(rng, b * extra_len // PAGE, wl)
        eoff = (np.arange(b, dtype=np.int32) * extra_len)[:, None, None]
        eidx = _distinct_rows(rng, b * s_q, extra_len, etopk).reshape(b, s_q, etopk) + eoff
        out.update(extra_kv=ekv_u8, extra_indices=np.ascontiguousarray(eidx.astype(np.int32)))
    if c.get("invalid"):
        idx = np.where(rng.random(idx.shape) < 0.1, -1, idx)
        if etopk:
            e = out["extra_indices"]
            out["extra_indices"] = np.where(rng.random(e.shape) < 0.1, -1, e).astype(np.int32)
    if c.get("lengths"):
        tl = rng.integers(1, topk + 1, size=b).astype(np.int32)
        tl[0] = 0
        out["topk_length"] = tl
        if etopk:
            el = rng.integers(0, etopk + 1, size=b).astype(np.int32)
            el[0] = 0
            out["extra_topk_length"] = el
    if c.get("sink"):
        out["attn_sink"] = (rng.standard_normal(64) * 2).astype(np.float32)
    out["indices"] = np.ascontiguousarray(idx.astype(np.int32))
    return out


def build(name: str) -> dict:
    return build_prefill(name) if name in PREFILL_CASES else build_decode(name)


def input_hash(case: dict) -> str:
    h = hashlib.sha256()
    for k in sorted(case):
        v = case[k]
        if isinstance(v, np.ndarray):
            h.update(k.encode())
            h.update(np.ascontiguousarray(v).tobytes())
        elif isinstance(v, (list, float, int)):
            h.update(f"{k}={v}".encode())
    return h.hexdigest()


# rows of `out` that the fixtures keep in full (all rows contribute a float64 row-sum as well)
def kept_rows(n_rows: int, keep: int = 12) -> np.ndarray:
    return np.unique(np.linspace(0, n_rows - 1, keep).astype(np.int64))
