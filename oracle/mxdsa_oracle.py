"""CPU oracle for the MXFP8 sparse-attention path.  TEST INFRASTRUCTURE ONLY.

This module is the checker that the tests, ``__graft_entry__.smoke()`` and the CPU-baseline
legs of ``bench.py`` compare the CUDA library against.  The shipped library never imports it.

It is a numpy restatement of what the reference (dingirsu/MXDSA) kernels compute, written from
the reference's sources (paths are relative to the reference project):

* wire format and quantiser ............ tests/mxfp8_test_utils.py:11-104, csrc/attention/config.h:64-76
* which Q bytes meet which K bytes ..... csrc/attention/common.cuh:84-96 (descriptor steps),
                                         csrc/attention/prefill_kernel.cuh:1060-1067 (Q tensor map),
                                         csrc/attention/prefill_kernel.cuh:266-286 (Q scale words)
* K scales, token ("anchor") V scale ... csrc/attention/prefill_kernel.cuh:599-704
* V dimension scales w1/w2 ............. csrc/attention/prefill_kernel.cuh:134-140, common.cuh:97-113
* validity rules ....................... csrc/attention/common.cuh:42-56 (prefill),
                                         csrc/attention/decode_kernel.cuh:660-673 (decode)
* softmax, P requantisation, outputs ... csrc/attention/prefill_kernel.cuh:717-1021,
                                         csrc/attention/decode_kernel.cuh:170-326, 811-971
* decode addressing / pair-row quirk ... csrc/attention/decode_kernel.cuh:105-158, 545-680
* split-KV scheduler ................... csrc/split_kv/scheduler.cu:11-118
* split combine ........................ csrc/split_kv/combine.cu:12-162

PARITY PIN.  The reference ships no golden vectors or known-answer tests, and it has no CPU
path.  The pin is therefore the reference's own kernels, compiled unmodified by
``oracle/build_ref.sh`` and run on a B200 by ``tests/golden/gen_golden.py``; the inputs and the
reference outputs of those runs are committed under ``tests/golden/`` and
``tests/test_oracle_golden.py`` checks this oracle against them.  The integer parts are pinned
bit for bit as well: the packers against the bytes of the reference's own Python packers
(``tests/golden/packers.npz``, written by ``tests/golden/gen_packer_golden.py`` from the
unmodified ``tests/mxfp8_test_utils.py`` of the reference; checked by
``tests/test_packers_reference_pin.py``), the scheduler metadata against the records of the
reference's scheduler kernel in the same golden fixtures.

Two levels of fidelity:
  level 0  exact softmax attention on the de-quantised operands in float64 (the ideal the kernel
           approximates; the reference kernel itself is ~0.1-0.5 max-abs away from it because the
           probabilities go through E4M3);
  level 1  the kernel's numerical contract: 64- or 128-key tiles, lazy running-max rescale
           (threshold 6 in log2 units, decided per 32 rows), probabilities times token scale
           re-quantised to E4M3 with one round-up UE8M0 scale per 32 keys (floor 61), and for
           decode the split-KV schedule with fp32 partials merged by the combine step.  This is
           the level that is pinned against the reference kernel's outputs (agreement ~1e-3).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Sequence, Tuple

import numpy as np

D = 512
SLOT = 16
ROW_BYTES = D + SLOT  # 528
FP8_MAX = 448.0
LOG2E = 1.4426950408889634


# --------------------------------------------------------------------------------------
# number formats
# --------------------------------------------------------------------------------------
def _build_e4m3_table() -> np.ndarray:
    """float32 value of every E4M3FN byte (bias 7, no inf, 0x7f/0xff are NaN)."""
    t = np.zeros(256, dtype=np.float64)
    for b in range(256):
        s = -1.0 if b & 0x80 else 1.0
        e = (b >> 3) & 0xF
        m = b & 7
        if e == 0xF and m == 7:
            v = float("nan")
        elif e == 0:
            v = m / 8.0 * 2.0 ** (-6)
        else:
            v = (1.0 + m / 8.0) * 2.0 ** (e - 7)
        t[b] = s * v
    return t.astype(np.float32)


E4M3_TABLE = _build_e4m3_table()
_E4M3_POS = E4M3_TABLE[:0x7F].astype(np.float64)  # 0 .. 448, ascending, 127 entries


def e4m3_decode(b: np.ndarray) -> np.ndarray:
    return E4M3_TABLE[np.asarray(b, dtype=np.uint8)]


def _chunked(fn, x: np.ndarray, out_dtype, chunk: int = 1 << 19) -> np.ndarray:
    """Apply an element-wise function over a flat view in pieces, so that its temporaries stay
    small and are recycled by the allocator (first-touch page faults dominate otherwise)."""
    x = np.ascontiguousarray(x)
    flat = x.reshape(-1)
    if flat.size <= chunk:
        return fn(x)
    out = np.empty(flat.size, dtype=out_dtype)
    for i in range(0, flat.size, chunk):
        out[i:i + chunk] = fn(flat[i:i + chunk])
    return out.reshape(x.shape)


def e4m3_encode(x: np.ndarray) -> np.ndarray:
    return _chunked(_e4m3_encode, np.asarray(x, dtype=np.float32), np.uint8)


def _e4m3_encode(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even, saturating-to-finite float -> E4M3FN byte
    (what ``tensor.to(torch.float8_e4m3fn)`` does for |x| <= 448, mxfp8_test_utils.py:20-21, and
    what ``cvt.rn.satfinite.e4m3x2.f32`` does in the kernel, prefill_kernel.cuh:828-829)."""
    x = np.asarray(x, dtype=np.float32)
    a = np.minimum(np.abs(x), np.float32(FP8_MAX)).astype(np.float64)
    _, ex = np.frexp(a)                      # a = m * 2^ex, m in [0.5, 1)
    e = np.maximum(ex - 1, -6)               # exponent of the binade, clamped to the subnormal one
    step = np.exp2((e - 3).astype(np.float64))
    qv = np.rint(a / step) * step            # rint rounds half to even
    _, ex2 = np.frexp(qv)
    e2 = np.maximum(ex2 - 1, -6)
    normal = qv >= 2.0 ** -6
    mant = np.where(normal, qv / np.exp2(e2.astype(np.float64)) - 1.0, qv * 64.0) * 8.0
    code = np.where(normal, (e2 + 7) << 3, 0).astype(np.int64) | mant.astype(np.int64)
    code = np.where(np.signbit(x), code | 0x80, code).astype(np.uint8)
    return code


def ue8m0_decode(b: np.ndarray) -> np.ndarray:
    """UE8M0 byte -> 2^(b-127) as float64 (b = 255 is NaN in the format; never produced here)."""
    return np.exp2(np.asarray(b, dtype=np.float64) - 127.0)


def ue8m0_roundup(x: np.ndarray) -> np.ndarray:
    """Smallest UE8M0 byte whose value is >= x (``cvt.rp.satfinite.ue8m0x2.f32``,
    csrc/ptx/types.cuh:14-29)."""
    x = np.asarray(x, dtype=np.float64)
    e = np.ceil(np.log2(np.maximum(x, 2.0 ** -127)))
    return np.clip(e + 127, 0, 254).astype(np.uint8)


def bf16_round(x: np.ndarray) -> np.ndarray:
    """float -> nearest-even bf16, returned as float32."""
    return _chunked(_bf16_round, np.asarray(x, dtype=np.float32), np.float32)


def _bf16_round(x: np.ndarray) -> np.ndarray:
    u = np.asarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return r.astype(np.uint32).view(np.float32)


# --------------------------------------------------------------------------------------
# wire format (tests/mxfp8_test_utils.py)
# --------------------------------------------------------------------------------------
def _pow2_scale(amax: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    """scale = 2^ceil(log2(max(amax/448, 2^-126))) and its UE8M0 byte (mxfp8_test_utils.py:15-18)."""
    s = np.maximum(amax.astype(np.float32) / np.float32(FP8_MAX), np.float32(2.0 ** -126))
    e = np.ceil(np.log2(s.astype(np.float32)).astype(np.float32)).astype(np.int32)
    return np.exp2(e.astype(np.float64)).astype(np.float32), (e + 127).astype(np.uint8)


def quantize_groups(x: np.ndarray, group: int) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    """Independent per-group quantiser (mxfp8_test_utils.py:11-27): bytes, scale bytes, dequantised."""
    x = np.asarray(x, dtype=np.float32)
    g = x.reshape(*x.shape[:-1], D // group, group)
    scale, sbyte = _pow2_scale(np.abs(g).max(-1))
    qv = np.clip(g / scale[..., None], -FP8_MAX, FP8_MAX)
    code = e4m3_encode(qv)
    deq = (e4m3_decode(code) * scale[..., None]).reshape(x.shape)
    return code.reshape(x.shape), sbyte, deq.astype(np.float32)


def pack_q(q: np.ndarray, paired_storage: bool = False) -> Tuple[np.ndarray, np.ndarray]:
    """Q packer (mxfp8_test_utils.py:30-63).  One scale per pair of 32-wide chunks
    ``[32g,32g+32)`` and ``[256+32g,256+32g+32)``.  With ``paired_storage=False`` the data bytes
    are stored in natural dimension order exactly as the reference packer does; with ``True``
    they are stored in the order ``[g][half][32]`` which is the order in which the kernel
    contracts them (see ``q_kernel_order``).  Returns (packed [...,528] u8, dequantised natural)."""
    q = np.asarray(q, dtype=np.float32)
    lead = q.shape[:-1]
    paired = q.reshape(*lead, 2, 8, 32).swapaxes(-3, -2).reshape(*lead, 8, 64)
    scale, sbyte = _pow2_scale(np.abs(paired).max(-1))
    code = e4m3_encode(np.clip(paired / scale[..., None], -FP8_MAX, FP8_MAX))
    deq = (e4m3_decode(code) * scale[..., None]).astype(np.float32)
    deq_nat = deq.reshape(*lead, 8, 2, 32).swapaxes(-3, -2).reshape(*lead, D)
    if paired_storage:
        data = code.reshape(*lead, D)
    else:
        data = code.reshape(*lead, 8, 2, 32).swapaxes(-3, -2).reshape(*lead, D)
    packed = np.empty((*lead, ROW_BYTES), dtype=np.uint8)
    packed[..., :D] = data
    packed[..., D:D + 8] = sbyte
    packed[..., D + 8:] = sbyte
    return packed, deq_nat


def pack_prefill_kv(kv: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    """Prefill KV packer (mxfp8_test_utils.py:66-78): a flat buffer holding every token's 512 data
    bytes followed by every token's 16-byte scale slot, viewed as [s_kv, 1, 528]."""
    assert kv.ndim == 3 and kv.shape[1] == 1
    data, sb, deq = quantize_groups(kv, 64)
    n = kv.shape[0]
    buf = np.empty(n * ROW_BYTES, dtype=np.uint8)
    buf[: n * D] = data.reshape(-1)
    buf[n * D:] = np.concatenate([sb, sb], -1).reshape(-1)
    return buf.reshape(n, 1, ROW_BYTES), deq


def pack_decode_kv_pages(kv: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    """Decode KV packer (mxfp8_test_utils.py:81-104): per page, page_size*512 data bytes and then
    page_size 16-byte scale slots."""
    assert kv.ndim == 4 and kv.shape[2] == 1
    pages, psz = kv.shape[:2]
    data, sb, deq = quantize_groups(kv, 64)
    buf = np.empty((pages, psz * ROW_BYTES), dtype=np.uint8)
    buf[:, : psz * D] = data.reshape(pages, -1)
    buf[:, psz * D:] = np.concatenate([sb, sb], -1).reshape(pages, -1)
    return buf.reshape(pages, psz, 1, ROW_BYTES), deq


def w_words_to_log2(w1: Sequence[int], w2: Sequence[int]) -> np.ndarray:
    """log2 of the eight 64-wide dimension scales encoded by w1/w2 (word 2i of each list)."""
    return np.array([(w1[2 * i] & 0xFF) - 127 for i in range(4)] +
                    [(w2[2 * i] & 0xFF) - 127 for i in range(4)])


def w_log2_to_words(wl: Sequence[int]) -> Tuple[list, list]:
    """w1/w2 word lists for eight 64-wide dimension scales 2^wl[g]: each word repeats one UE8M0
    byte four times and adjacent words (32 dims each) share it (reference params.h:386-388)."""
    words = [int((int(e) + 127) * 0x01010101) for e in wl]
    return [words[j // 2] for j in range(8)], [words[4 + j // 2] for j in range(8)]


def rank1_kv(rng: np.random.Generator, shape: Sequence[int], w_log2_range: int = 2,
             wl: Optional[np.ndarray] = None):
    """Synthetic KV whose 64-wide group scales factor as token scale x dimension scale, which is
    what the kernel's V path assumes (reference README "rank-1 factorization").  Returns
    (kv float32 [..., 512], w1 words[8], w2 words[8]).  W[g] are random powers of two in
    [2^-r, 2^r] with W[0] = 1 (or the given ``wl`` = log2 W); every group of a token is rescaled so that its own power-of-two
    quantisation scale is exactly tok * W[g]."""
    x = rng.standard_normal((*shape, D), dtype=np.float32)
    if wl is None:
        wl = rng.integers(-w_log2_range, w_log2_range + 1, size=8)
        wl[0] = 0
    wl = np.asarray(wl)
    g = x.reshape(*shape, 8, 64)
    amax = np.abs(g).max(-1)
    _, sb = _pow2_scale(amax)
    e = sb.astype(np.int32) - 127
    target = e[..., :1] + wl
    g = g * np.exp2((target - e).astype(np.float32))[..., None]
    kv = g.reshape(*shape, D)
    w1, w2 = w_log2_to_words(wl)
    return kv, w1, w2


# --------------------------------------------------------------------------------------
# de-quantisation exactly as the kernel consumes the bytes
# --------------------------------------------------------------------------------------
def q_kernel_order(q_u8: np.ndarray) -> np.ndarray:
    """De-quantise packed Q rows [...,528] into the order in which the kernel contracts them with
    K's natural dimension order.

    QK step kk (0..15) multiplies Q memory bytes [(kk%8)*64 + (kk//8)*32, +32) with K bytes
    [32kk, +32) and uses Q scale byte kk%8 (common.cuh:84-96 with the natural-order Q tensor map,
    prefill_kernel.cuh:1060-1067, and the scale words of prefill_kernel.cuh:276-286).  So Q memory
    block 2g+h lines up with K block 8h+g and carries scale g."""
    q_u8 = np.asarray(q_u8, dtype=np.uint8)
    lead = q_u8.shape[:-1]
    val = e4m3_decode(q_u8[..., :D]).astype(np.float64).reshape(*lead, 8, 2, 32)
    sc = ue8m0_decode(q_u8[..., D:D + 8])  # first copy of the slot (LDG_128 .x/.y)
    val = val * sc[..., :, None, None]
    return val.swapaxes(-3, -2).reshape(*lead, D)  # [h][g][32] == K block 8h+g


def kv_rows_dequant(data: np.ndarray, slot: np.ndarray, w1: Sequence[int], w2: Sequence[int],
                    v_sf_byte: int = 0) -> Tuple[np.ndarray, np.ndarray]:
    """K and V values of gathered rows.  ``data`` [...,512] u8, ``slot`` [...,16] u8.
    K uses scale byte j for dims [64j, 64j+64) (prefill_kernel.cuh:676-691, common.cuh:88-95).
    V uses only scale byte 0 of the token, times the dimension scale taken from w1 (dims 0-255)
    or w2 (dims 256-511), word (d%256)//32 (prefill_kernel.cuh:134-140, 693-695)."""
    e = e4m3_decode(data).astype(np.float64)
    ks = np.repeat(ue8m0_decode(slot[..., :8]), 64, axis=-1)
    k = e * ks
    wbytes = np.array([(w >> (8 * v_sf_byte)) & 0xFF for w in list(w1) + list(w2)], dtype=np.uint8)
    wd = np.repeat(ue8m0_decode(wbytes), 32)
    v = e * ue8m0_decode(slot[..., 0:1]) * wd
    return k, v


# --------------------------------------------------------------------------------------
# attention core shared by prefill and decode
# --------------------------------------------------------------------------------------
def _attend_exact(qk, k, v, valid, sm_scale, sink):
    """Level 0: plain softmax attention in float64.  qk [R,512], k/v [T,512], valid [T].
    Returns out [R,512], max_logits [R], lse [R] (natural log; the sink only enters `out`)."""
    R = qk.shape[0]
    if not valid.any():
        return np.zeros((R, D)), np.full(R, -np.inf), np.full(R, np.inf)
    logits = np.where(valid[None, :], (qk @ k.T) * sm_scale, -np.inf)
    mx = logits.max(-1)
    p = np.exp(logits - mx[:, None])
    l = p.sum(-1)
    denom = l if sink is None else l + np.exp(np.tile(sink, R // 64) - mx)
    return (p @ v) / denom[:, None], mx, mx + np.log(l)


def _tile_pass(qk, k, vq, tok, valid, sm_scale, tile):
    """Level 1: one pass of the kernel's main loop over the given keys (a whole index row, or the
    block range of one decode split), in the kernel's own arithmetic order
    (prefill_kernel.cuh:732-986, decode_kernel.cuh:827-958):

      x       = logit * (sm_scale * log2e)               fp32
      tile max, and per group of 32 rows (one warp): adopt max(m, tile max) as the new running
      max m only if some row of the group has tile max - m > 6; m starts at -1e30
      p       = exp2(x - m); l = l * 2^(m_old - m) + sum p; O *= 2^(m_old - m)
      s       = p * token scale; per 32 keys e = max(roundup_ue8m0(amax(s)/448), 61)
      S8      = e4m3(s * 2^(127 - e));  O += (S8 * 2^(e-127)) @ (E4M3 values * dimension scale)

    Returns O [R,512] (un-normalised), m [R] (base 2, -inf when no key was valid), l [R],
    true max [R] (base 2)."""
    R = qk.shape[0]
    f32 = np.float32
    scale_log2 = f32(f32(sm_scale) * f32(1.44269504))    # bindings/common.h:11, binding.cpp:86
    x_all = (qk @ k.T).astype(f32) * scale_log2          # fp32 accumulators times fp32 scale
    x_all = np.where(valid[None, :], x_all, f32(-np.inf))
    m = np.full(R, f32(-1e30), dtype=f32)
    l = np.zeros(R, dtype=f32)
    real = np.full(R, f32(-np.inf), dtype=f32)
    o = np.zeros((R, D), dtype=np.float64)
    T = k.shape[0]
    tok32 = tok.astype(f32)
    for t0 in range(0, T, tile):
        xt = x_all[:, t0:t0 + tile]
        tmax = xt.max(-1)
        real = np.maximum(real, tmax)
        grow = (tmax - m > f32(6.0)).reshape(-1, 32).any(-1).repeat(32)
        newm = np.where(grow, np.maximum(m, tmax), m)
        so = np.where(grow, np.exp2((m - newm).astype(np.float64)), 1.0).astype(f32)
        m = newm
        p = np.exp2((xt - m[:, None]).astype(np.float64)).astype(f32)
        l = (l * so + p.sum(-1, dtype=f32)).astype(f32)
        o = o * so[:, None].astype(np.float64)
        sv = (p * tok32[None, t0:t0 + tile]).astype(f32)
        for b0 in range(0, xt.shape[1], 32):
            sb = sv[:, b0:b0 + 32]
            amax = sb.max(-1)
            e = np.where(amax > 0, ue8m0_roundup(amax.astype(np.float64) / FP8_MAX), 127).astype(np.int32)
            e = np.maximum(e, 61)
            s8 = e4m3_decode(e4m3_encode(sb * np.exp2(127.0 - e)[:, None].astype(f32))).astype(np.float64)
            o += (s8 * np.exp2(e - 127.0)[:, None]) @ vq[t0 + b0:t0 + b0 + 32]
    none = np.isneginf(real)
    l = np.where(none, f32(0), l)
    m = np.where(none, f32(-np.inf), m)
    return o, m, l, real


LN2 = 0.6931471805599453


def _finish(o, m, l, real, sink, R):
    """Epilogue of an un-split pass (prefill_kernel.cuh:988-1019, decode_kernel.cuh:187-214):
    out = O / (l + 2^(sink*log2e - m)), 0 when l == 0; lse = m*ln2 + ln(l), +inf when no key."""
    with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
        sk = np.full(R, -np.inf) if sink is None else np.tile(sink, R // 64).astype(np.float64)
        denom = l.astype(np.float64) + np.exp2(sk * LOG2E - m.astype(np.float64))
        out = np.where((l == 0)[:, None], 0.0, o / denom[:, None])
        lse = m.astype(np.float64) * LN2 + np.log(l.astype(np.float64))
        lse = np.where(np.isneginf(lse) | np.isnan(lse), np.inf, lse)
    return out, real.astype(np.float64) * LN2, lse


def prefill_ref(q_u8: np.ndarray, kv_u8: np.ndarray, indices: np.ndarray, sm_scale: float,
                w1: Sequence[int], w2: Sequence[int], attn_sink: Optional[np.ndarray] = None,
                topk_length: Optional[np.ndarray] = None, level: int = 1):
    """Restatement of ``dual_mxfp8_head64_sparse_prefill_fwd`` (csrc/bindings/binding.cpp:12-113).
    q_u8 [s_q,64,528], kv_u8 [s_kv,1,528] (flat envelope), indices [s_q/2,1,topk] int32.
    Returns (out [s_q,64,512] float32 rounded to bf16, max_logits [s_q,64] f32, lse [s_q,64] f32).
    The reference demands an even s_q (binding.cpp:36); an odd one is taken here as "the last index row
    serves one token" (indices [ceil(s_q/2),1,topk]): the token is evaluated twice and one copy dropped."""
    s_q_given = q_u8.shape[0]
    if s_q_given % 2:
        q_u8 = np.concatenate([q_u8, q_u8[-1:]])
    s_q = q_u8.shape[0]
    s_kv = kv_u8.shape[0]
    topk = indices.shape[-1]
    flat = np.ascontiguousarray(kv_u8).reshape(-1)
    data = flat[: s_kv * D].reshape(s_kv, D)
    slots = flat[s_kv * D:].reshape(s_kv, SLOT)
    k_all, v_all = kv_rows_dequant(data, slots, w1, w2)
    tok_all = ue8m0_decode(slots[:, 0])
    vq_all = v_all / tok_all[:, None]
    qk = q_kernel_order(q_u8)  # [s_q,64,512]
    out = np.zeros((s_q, 64, D), dtype=np.float32)
    mxl = np.zeros((s_q, 64), dtype=np.float32)
    lse = np.zeros((s_q, 64), dtype=np.float32)
    tile = 128 if topk >= 512 else 64  # csrc/attention/launch.h:14-19
    for p in range(s_q // 2):
        idx = indices[p, 0].astype(np.int64)
        n = topk if topk_length is None else int(topk_length[p])
        pos = np.arange(topk)
        valid = (idx >= 0) & (idx < s_kv) & (pos < n)  # common.cuh:46-49
        safe = np.where(valid, idx, 0)
        rows = qk[2 * p:2 * p + 2].reshape(128, D)
        if level == 0:
            o, m, l = _attend_exact(rows, k_all[safe], v_all[safe], valid, sm_scale, attn_sink)
        else:
            # the kernel walks max(ceil(n / tile), 1) tiles (prefill_kernel.cuh:120)
            nt = max(-(-n // tile), 1) * tile
            pad = max(nt - topk, 0)
            sl = slice(0, min(nt, topk))
            kk, vv, tt, va = k_all[safe][sl], vq_all[safe][sl], tok_all[safe][sl], valid[sl]
            if pad:
                kk = np.concatenate([kk, np.zeros((pad, D))])
                vv = np.concatenate([vv, np.zeros((pad, D))])
                tt = np.concatenate([tt, np.ones(pad)])
                va = np.concatenate([va, np.zeros(pad, bool)])
            o, m, l = _finish(*_tile_pass(rows, kk, vv, tt, va, sm_scale, tile), attn_sink, 128)
        out[2 * p:2 * p + 2] = bf16_round(o.reshape(2, 64, D))
        mxl[2 * p:2 * p + 2] = m.reshape(2, 64)
        lse[2 * p:2 * p + 2] = l.reshape(2, 64)
    return out[:s_q_given], mxl[:s_q_given], lse[:s_q_given]


def _pool_views(pool_u8: np.ndarray):
    """Split a decode page pool [pages, page, 1, 528] into data [pages*page,512] and
    slots [pages*page,16] (decode_kernel.cuh:674-680: slot offset = page*stride + page_size*512 +
    idx_in_page*16)."""
    pages, psz = pool_u8.shape[:2]
    flat = np.ascontiguousarray(pool_u8).reshape(pages, psz * ROW_BYTES)
    data = flat[:, : psz * D].reshape(pages * psz, D)
    slots = flat[:, psz * D:].reshape(pages * psz, SLOT)
    return data, slots


def _decode_row_keys(r, row, indices, topk_length, kvd, extra_indices, extra_topk_length, ekvd):
    """Key sequence of one (request, index row) in the kernel's block order: the main keys padded
    to whole 64-key blocks (max(ceil(len/64),1) blocks), then the extra keys padded likewise
    (decode_kernel.cuh:121-129, 599-701).  Returns data rows, slot rows, valid mask."""
    topk = indices.shape[-1]
    data, slots = kvd
    n = topk if topk_length is None else int(topk_length[r])
    nblk = max(-(-n // 64), 1)
    pos = np.arange(nblk * 64)
    idx = np.full(nblk * 64, -1, dtype=np.int64)
    m = min(topk, nblk * 64)
    idx[:m] = indices[r, row, :m]
    # decode_kernel.cuh:666-669 attends every index != -1.  An index outside the pool is undefined behaviour
    # there (the scale slot is read out of bounds); the library under test skips such a key, and so does this.
    valid = (idx >= 0) & (idx < data.shape[0]) & (pos < n)
    safe = np.where(valid, idx, 0)
    d_rows, s_rows = data[safe], slots[safe]
    if ekvd is not None and extra_indices is not None and extra_indices.shape[-1] > 0:
        edata, eslots = ekvd
        etopk = extra_indices.shape[-1]
        en = etopk if extra_topk_length is None else int(extra_topk_length[r])
        enblk = -(-en // 64)
        epos = np.arange(enblk * 64)
        eidx = np.full(enblk * 64, -1, dtype=np.int64)
        em = min(etopk, enblk * 64)
        eidx[:em] = extra_indices[r, row, :em]
        evalid = (eidx >= 0) & (eidx < edata.shape[0]) & (epos < en)
        esafe = np.where(evalid, eidx, 0)
        d_rows = np.concatenate([d_rows, edata[esafe]])
        s_rows = np.concatenate([s_rows, eslots[esafe]])
        valid = np.concatenate([valid, evalid])
    return d_rows, s_rows, valid


def decode_ref(q_u8: np.ndarray, kv_u8: np.ndarray, indices: np.ndarray,
               topk_length: Optional[np.ndarray], attn_sink: Optional[np.ndarray],
               extra_kv_u8: Optional[np.ndarray], extra_indices: Optional[np.ndarray],
               extra_topk_length: Optional[np.ndarray], sm_scale: float, w1: Sequence[int],
               w2: Sequence[int], level: int = 1, sched: Optional["SchedMeta"] = None,
               per_query_rows: bool = False):
    """Restatement of ``dual_mxfp8_sparse_decode_fwd`` (csrc/bindings/dual_mxfp8_sparse_decode.h).
    q_u8 [b,s_q,64,528]; kv pools [pages,page,1,528]; indices [b,s_q,topk] of global slot ids
    (page*page_size + slot).  Queries 2p and 2p+1 of a request both follow index row p
    (decode_kernel.cuh:108, 554-558) unless ``per_query_rows``.  A slot is attended when its
    index != -1 and its position < the request's length (decode_kernel.cuh:666-669).

    Level 1 with ``sched`` walks the split-KV schedule the way the kernel does
    (decode_kernel.cuh:105-158): every sm-part processes its block range of each of its requests
    as an independent pass; passes of a split request are written as fp32 partials
    (O/l, log2(l)+m) and merged by ``combine_ref``.  Without ``sched`` every row is one pass.

    Returns (out [b,s_q,64,512] f32 bf16-rounded, lse [b,s_q,64] f32); lse excludes the sink
    (decode_kernel.cuh:199-213, combine.cu:99-101)."""
    b, s_q = q_u8.shape[:2]
    kvd = _pool_views(kv_u8)
    ekvd = _pool_views(extra_kv_u8) if extra_kv_u8 is not None else None
    qk = q_kernel_order(q_u8)
    out = np.zeros((b, s_q, 64, D), dtype=np.float32)
    lse = np.zeros((b, s_q, 64), dtype=np.float32)
    if per_query_rows:
        groups = [(s, [s]) for s in range(s_q)]
    else:
        groups = [(p, [t for t in (2 * p, 2 * p + 1) if t < s_q]) for p in range((s_q + 1) // 2)]

    def operands(r, row):
        d_rows, s_rows, valid = _decode_row_keys(r, row, indices, topk_length, kvd, extra_indices,
                                                 extra_topk_length, ekvd)
        k, v = kv_rows_dequant(d_rows, s_rows, w1, w2)
        tok = ue8m0_decode(s_rows[:, 0])
        return k, v, tok, valid

    if level == 0 or sched is None:
        for r in range(b):
            for row, toks in groups:
                k, v, tok, valid = operands(r, row)
                R = len(toks) * 64
                qrows = qk[r, toks].reshape(R, D)
                if level == 0:
                    o, _, l = _attend_exact(qrows, k, v, valid, sm_scale, attn_sink)
                else:
                    o, _, l = _finish(*_tile_pass(_pad128(qrows), k, v / tok[:, None], tok, valid,
                                                  sm_scale, 64), attn_sink, 128)
                    o, l = o[:R], l[:R]
                out[r, toks] = bf16_round(o.reshape(len(toks), 64, D))
                lse[r, toks] = l.reshape(len(toks), 64)
        return out, lse

    partial = {}  # (request, row) -> list of (split index, o [128,512], lse2 [128])
    for part in sched.meta:
        begin_req, end_req, begin_block, end_block, begin_split, first_split, last_split = part[:7]
        if begin_req >= b:
            continue
        for r in range(begin_req, end_req + 1):
            for row, toks in groups:
                k, v, tok, valid = operands(r, row)
                nblocks = k.shape[0] // 64
                s_blk = begin_block if r == begin_req else 0
                e_blk = end_block if r == end_req else nblocks
                is_split = bool(first_split) if r == begin_req else (bool(last_split) if r == end_req else False)
                n_split = int(sched.num_splits[r]) + (begin_split if r == begin_req else 0)
                sl = slice(s_blk * 64, e_blk * 64)
                R = len(toks) * 64
                qrows = _pad128(qk[r, toks].reshape(R, D))
                o, m, l, real = _tile_pass(qrows, k[sl], (v / tok[:, None])[sl], tok[sl], valid[sl],
                                           sm_scale, 64)
                if not is_split:
                    oo, _, ll = _finish(o, m, l, real, attn_sink, 128)
                    out[r, toks] = bf16_round(oo[:R].reshape(len(toks), 64, D))
                    lse[r, toks] = ll[:R].reshape(len(toks), 64)
                else:
                    with np.errstate(divide="ignore", invalid="ignore"):
                        on = np.where((l == 0)[:, None], 0.0, o / l.astype(np.float64)[:, None])
                        l2 = np.log2(l.astype(np.float64)) + m.astype(np.float64)
                    partial.setdefault((r, row), []).append((n_split, on, l2))
    for (r, row), lst in partial.items():
        toks = dict(groups)[row]
        R = len(toks) * 64
        lst.sort(key=lambda t: t[0])
        first = int(sched.num_splits[r])
        assert [t[0] for t in lst] == list(range(first, int(sched.num_splits[r + 1]))), (r, row)
        oacc = np.stack([t[1] for t in lst]).astype(np.float32).astype(np.float64)
        lacc = np.stack([t[2] for t in lst]).astype(np.float32).astype(np.float64)
        sink = None if attn_sink is None else np.tile(attn_sink, 2).astype(np.float64)
        oo, ll = combine_ref(lacc, oacc, sink)
        out[r, toks] = bf16_round(oo[:R].reshape(len(toks), 64, D))
        lse[r, toks] = ll[:R].reshape(len(toks), 64)
    return out, lse


def _pad128(rows: np.ndarray) -> np.ndarray:
    """The kernel always works on 128 rows (2 tokens x 64 heads); with an odd s_q the last pair's
    second token is a clamped copy that is never stored (decode_kernel.cuh:266-267)."""
    if rows.shape[0] == 128:
        return rows
    return np.concatenate([rows, rows[-64:]])


# --------------------------------------------------------------------------------------
# split-KV scheduler and combine
# --------------------------------------------------------------------------------------
@dataclass
class SchedMeta:
    meta: np.ndarray        # [num_sm_parts, 8] int32: begin_req, end_req, begin_block, end_block,
                            #   begin_split, first_req_splitted, last_req_splitted, pad
    num_splits: np.ndarray  # [b+1] int32 prefix sums


def sched_meta_ref(b: int, topk: int, extra_topk: int, num_sm_parts: int,
                   topk_length: Optional[np.ndarray] = None,
                   extra_topk_length: Optional[np.ndarray] = None,
                   block: int = 64, overhead: int = 5) -> SchedMeta:
    """Integer-exact restatement of ``get_mla_metadata_kernel`` (csrc/split_kv/scheduler.cu:11-118).

    Parts that receive no work (begin_req == b) are skipped by the attention kernel, but the
    reference still fills their records by reading its shared arrays one element past the end:
    first_block[b] aliases last_block[0] and the end fields come from request b-1
    (scheduler.cu:22-26, 70, 98-103).  Those values are reproduced so that the seven meaningful
    ints of every record can be compared bit for bit; the eighth int is uninitialised padding in
    the reference and is written as 0 here."""
    nblk, first, last, seql = [], [], [], []
    total = 0
    for i in range(b):
        s = int(topk_length[i]) if topk_length is not None else topk
        if s == 0:
            s = 1
        if extra_topk:
            s = -(-s // block) * block
            s += int(extra_topk_length[i]) if extra_topk_length is not None else extra_topk
        seql.append(s)
        lb = max(s - 1, 0) // block
        first.append(0)
        last.append(lb)
        nblk.append(lb + 1)
        total += lb + 1 + overhead
    payload = -(-total // num_sm_parts) + overhead
    meta = np.zeros((num_sm_parts, 8), dtype=np.int32)
    splits = np.zeros(b + 1, dtype=np.int32)
    req = blk = nsplit = cum = 0
    for i in range(num_sm_parts):
        begin_req, begin_split = req, nsplit
        begin_block = blk + (first[req] if req < b else last[0])
        first_split = int(blk != 0)
        remain = payload
        while req < b:
            rem_blocks = nblk[req] - blk
            if remain >= rem_blocks + overhead:
                cum += nsplit + 1
                splits[req + 1] = cum
                remain -= rem_blocks + overhead
                req += 1
                blk = 0
                nsplit = 0
            else:
                if remain - overhead > 0:
                    blk += remain - overhead
                    nsplit += 1
                    remain = 0
                break
        end_req = req if blk > 0 else req - 1
        if blk > 0:
            end_block = blk + first[req]
        else:
            end_block = 0 if seql[req - 1] == 0 else last[req - 1] + 1
        last_split = int(end_block != last[end_req] + 1 and seql[end_req] != 0)
        if begin_req == end_req:
            first_split = last_split = int(first_split or last_split)
        meta[i] = [begin_req, end_req, begin_block, end_block, begin_split, first_split, last_split, 0]
    assert req == b and blk == 0 and nsplit == 0
    return SchedMeta(meta, splits)


def sched_whole_ref(b: int, topk: int, extra_topk: int, num_sm_parts: int,
                    topk_length: Optional[np.ndarray] = None,
                    extra_topk_length: Optional[np.ndarray] = None, block: int = 64) -> SchedMeta:
    """Whole-request schedule (records of the layout of ``sched_meta_ref``; no request is divided, so decode needs
    no combine pass).  The reference has no such schedule -- its scheduler (csrc/split_kv/scheduler.cu:61-112)
    always fills parts to an equal budget and splits -- so the rule is this library's own, restated here for the
    tests: part i takes the consecutive requests whose midpoint, in prefix-summed 64-key blocks, lies in the i-th
    of ``num_sm_parts`` equal shares of the total (the last part takes what is left); num_splits[i] = i."""
    nblk = []
    for i in range(b):
        s = int(topk_length[i]) if topk_length is not None else topk
        if s == 0:
            s = 1
        if extra_topk:
            s = -(-s // block) * block
            s += int(extra_topk_length[i]) if extra_topk_length is not None else extra_topk
        nblk.append(max(s - 1, 0) // block + 1)
    total = sum(nblk)
    meta = np.zeros((num_sm_parts, 8), dtype=np.int32)
    req, before = 0, 0
    for i in range(num_sm_parts):
        first = req
        while req < b and (i == num_sm_parts - 1 or (2 * before + nblk[req]) * num_sm_parts < 2 * total * (i + 1)):
            before += nblk[req]
            req += 1
        meta[i] = [first, req - 1, 0, nblk[req - 1] if req > first else 0, 0, 0, 0, 0]
    assert req == b
    return SchedMeta(meta, np.arange(b + 1, dtype=np.int32))


def combine_ref(lse_accum: np.ndarray, o_accum: np.ndarray, sink: Optional[np.ndarray]):
    """Merge of split partials (csrc/split_kv/combine.cu:66-125).  lse_accum [n,R] base-2,
    o_accum [n,R,512].  Returns (out [R,512] f64, lse [R] natural log, +inf when empty)."""
    with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
        mx = lse_accum.max(0)
        mx = np.where(np.isneginf(mx), 0.0, mx)
        s = np.exp2(lse_accum - mx).sum(0)
        g = np.where(s == 0, np.inf, np.log2(s) + mx)
        lse = g / LOG2E
        if sink is not None:
            g = np.where(np.isinf(g), np.where(np.isneginf(sink), np.inf, sink * LOG2E),
                         g + np.log2(1 + np.exp2(sink * LOG2E - g)))
        w = np.exp2(lse_accum - g)
    return (w[..., None] * o_accum).sum(0), lse


# --------------------------------------------------------------------------------------
# index selection (the producer of `indices`)
# --------------------------------------------------------------------------------------
def topk_select_ref(scores: np.ndarray, topk: int, lengths: Optional[np.ndarray] = None, pair: bool = False,
                    row_offset: Optional[np.ndarray] = None) -> Tuple[np.ndarray, np.ndarray]:
    """Index selection feeding ``indices`` (no counterpart in the reference: "parity unpinned"; the
    definition follows the conventions of the reference's callers, tests/benchmark.py:119-147 --
    one row per pair, -1 never attended, pool offsets added to the slot index).

    scores f32 [n, s_kv] -> (indices i32 [rows, topk], topk_length i32 [rows]); rows = n/2 with
    ``pair`` (a key's score = the larger of the two tokens', NaN on one side ignored).  Row r keeps the
    min(topk, candidates) best keys among j < lengths[r]; NaN / -inf are no candidates; ties go to the
    smaller j (stable sort); selected indices ascending (+ row_offset[r]), then -1.
    """
    s = np.asarray(scores, dtype=np.float32)
    if pair:
        s = np.fmax(s[0::2], s[1::2])
    rows, s_kv = s.shape
    idx = np.full((rows, topk), -1, dtype=np.int32)
    cnt = np.zeros((rows,), dtype=np.int32)
    for r in range(rows):
        n = s_kv if lengths is None else int(min(max(int(lengths[r]), 0), s_kv))
        row = s[r, :n]
        cand = np.nonzero(~np.isnan(row) & (row != -np.inf))[0]
        order = cand[np.argsort(-row[cand].astype(np.float64), kind="stable")]   # descending score, ascending j in ties
        keep = np.sort(order[:topk])
        cnt[r] = keep.size
        idx[r, :keep.size] = keep + (0 if row_offset is None else int(row_offset[r]))
    return idx, cnt


# --------------------------------------------------------------------------------------
# error measures used by the tests (north-star tolerances)
# --------------------------------------------------------------------------------------
def max_abs(a: np.ndarray, b: np.ndarray) -> float:
    return float(np.max(np.abs(np.asarray(a, np.float64) - np.asarray(b, np.float64))))


def cosine(a: np.ndarray, b: np.ndarray) -> float:
    a = np.asarray(a, np.float64).ravel()
    b = np.asarray(b, np.float64).ravel()
    d = math.sqrt(float(a @ a)) * math.sqrt(float(b @ b))
    return float(a @ b) / d if d > 0 else 1.0
