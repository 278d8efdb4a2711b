"""Parity of the CUDA path on a B200 (run with -m gpu).

Every case goes through the C ABI of libmxdsa.so -- once via the C++ extension module and once
via the ctypes operator implementation -- and is compared with
  * the reference kernel's own outputs (golden fixtures), at the north-star tolerances
    (bf16 out: max-abs <= 2e-2, cosine >= 0.9999; lse / max_logits: 1e-3 abs), and
  * the CPU oracle (level 1) on the same inputs.
Larger shapes are covered through size-independent properties (determinism, exact power-of-two
linearity in the V dimension scales, equivalence of the two masking mechanisms) plus an oracle
check on a sample of query pairs.
"""
import numpy as np
import pytest
import torch

import cases
from helpers import check_against_golden, check_against_oracle, load_golden
from oracle import mxdsa_oracle as O

pytestmark = pytest.mark.gpu


def _impl(name):
    import mxdsa_b200
    return mxdsa_b200 if name == "extension" else mxdsa_b200.api


def _t(x):
    return None if x is None else torch.from_numpy(np.ascontiguousarray(x)).cuda()


def _run_prefill(impl, c):
    import mxdsa_b200
    out, mxl, lse = impl.dual_mxfp8_head64_sparse_prefill_fwd(
        _t(c["q"]), _t(c["kv"]), _t(c["indices"]), c["sm_scale"], c["w1"], c["w2"], _t(c["attn_sink"]),
        _t(c["topk_length"]))
    mxdsa_b200.device_fault()
    assert out.dtype == torch.bfloat16 and tuple(out.shape) == (c["q"].shape[0], 64, 512)
    return out.float().cpu().numpy(), mxl.cpu().numpy(), lse.cpu().numpy()


def _run_decode(impl, c, meta=None, splits=None):
    import mxdsa_b200
    out, lse, meta, splits = impl.dual_mxfp8_sparse_decode_fwd(
        _t(c["q"]), _t(c["kv"]), _t(c["indices"]), _t(c["topk_length"]), _t(c["attn_sink"]), meta, splits,
        _t(c["extra_kv"]), _t(c["extra_indices"]), _t(c["extra_topk_length"]), 512, 512, c["sm_scale"], c["w1"],
        c["w2"])
    mxdsa_b200.device_fault()
    return out, lse, meta, splits


@pytest.mark.parametrize("impl", ["extension", "ctypes"])
@pytest.mark.parametrize("name", list(cases.PREFILL_CASES))
def test_prefill_matches_reference_kernel_and_oracle(name, impl):
    c = cases.build(name)
    g = load_golden(name)
    assert str(g["input_hash"]) == cases.input_hash(c)
    out, mxl, lse = _run_prefill(_impl(impl), c)
    check_against_golden(g, out, lse, mxl)
    ro, rm, rl = O.prefill_ref(c["q"], c["kv"], c["indices"], c["sm_scale"], c["w1"], c["w2"], c["attn_sink"],
                               c["topk_length"], level=1)
    check_against_oracle(out, ro)
    fin = np.isfinite(rl)
    assert np.array_equal(np.isposinf(lse), np.isposinf(rl)) and np.abs(lse[fin] - rl[fin]).max() <= 1e-3
    assert np.array_equal(np.isneginf(mxl), np.isneginf(rm)) and np.abs(mxl[fin] - rm[fin]).max() <= 1e-3
    # pairs without any valid key: zeros, lse = +inf, max_logits = -inf
    none = np.isposinf(rl)
    assert np.all(out[none] == 0) and np.all(np.isneginf(mxl[none]))


@pytest.mark.parametrize("impl", ["extension", "ctypes"])
@pytest.mark.parametrize("name", list(cases.DECODE_CASES))
def test_decode_matches_reference_kernel_and_oracle(name, impl):
    c = cases.build(name)
    cc = cases.DECODE_CASES[name]
    g = load_golden(name)
    assert str(g["input_hash"]) == cases.input_hash(c)
    out, lse, meta, splits = _run_decode(_impl(impl), c)
    assert tuple(lse.shape) == (cc["b"], 64, cc["s_q"]) and lse.stride(1) == 1   # [b,64,s_q] view of [b,s_q,64]
    parts = meta.shape[0]
    # integer work: bit exact against the reference's scheduler (fixture) and the oracle
    if parts == int(g["num_sm_parts"]):
        assert np.array_equal(meta.cpu().numpy()[:, :7], g["sched_meta"][:, :7])
        assert np.array_equal(splits.cpu().numpy(), g["num_splits"])
    sm = O.sched_meta_ref(cc["b"], cc["topk"], cc.get("extra_topk", 0), parts, c["topk_length"],
                          c["extra_topk_length"])
    assert np.array_equal(meta.cpu().numpy()[:, :7], sm.meta[:, :7])
    assert np.array_equal(splits.cpu().numpy(), sm.num_splits)
    o = out.float().cpu().numpy()
    l = lse.transpose(1, 2).contiguous().cpu().numpy()
    check_against_golden(g, o, l, lse_is_b_h_s=True)
    ro, rl = O.decode_ref(c["q"], c["kv"], c["indices"], c["topk_length"], c["attn_sink"], c["extra_kv"],
                          c["extra_indices"], c["extra_topk_length"], c["sm_scale"], c["w1"], c["w2"], level=1,
                          sched=sm)
    check_against_oracle(o, ro)
    fin = np.isfinite(rl)
    assert np.array_equal(np.isposinf(l), np.isposinf(rl)) and np.abs(l[fin] - rl[fin]).max() <= 1e-3
    # the returned scheduling info can be passed back in: same bits
    out2, lse2, meta2, splits2 = _run_decode(_impl(impl), c, meta, splits)
    assert meta2.data_ptr() == meta.data_ptr() and splits2.data_ptr() == splits.data_ptr()
    assert torch.equal(out.view(torch.int16), out2.view(torch.int16)) and torch.equal(lse, lse2)


def test_scheduler_matches_reference_at_benchmark_shapes():
    """mxdsa_decode_sched alone, through the C ABI, against the reference scheduler's records."""
    import ctypes as C
    from mxdsa_b200 import capi
    s = load_golden("sched")
    L = capi.lib()
    for b in (64, 128):
        for extra in (0, 128, 1024, 4096):
            meta = torch.full((24, 8), -7, dtype=torch.int32, device="cuda")
            splits = torch.full((b + 1,), -7, dtype=torch.int32, device="cuda")
            p = capi.SchedParams(b=b, s_q=6, topk=128, extra_topk=extra, topk_length=None, extra_topk_length=None,
                                 num_sm_parts=24, sched_meta=meta.data_ptr(), num_splits=splits.data_ptr(),
                                 stream=torch.cuda.current_stream().cuda_stream)
            capi.check(L.mxdsa_decode_sched(C.byref(p)), "sched")
            torch.cuda.synchronize()
            assert np.array_equal(meta.cpu().numpy()[:, :7], s[f"meta_b{b}_e{extra}"][:, :7]), (b, extra)
            assert np.array_equal(splits.cpu().numpy(), s[f"splits_b{b}_e{extra}"]), (b, extra)


def _big_prefill(s_q, s_kv, topk, seed, tail_invalid=0.0):
    from mxdsa_b200 import packing as P
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.empty((s_q, 64, 528), dtype=torch.uint8, device="cuda")
    for i in range(0, s_q, 512):
        n = min(512, s_q - i)
        q[i:i + n] = P.pack_dual_q64(torch.randn(n, 64, 512, device="cuda", generator=g))[0]
    kvf, w1, w2 = P.make_rank1_kv((s_kv, 1), device="cuda", generator=g)
    kv = P.pack_dual_prefill_kv64(kvf)[0]
    base = torch.stack([torch.randperm(s_kv, device="cuda", generator=g)[:topk] for _ in range(32)]).int()
    idx = base[torch.randint(0, 32, (s_q // 2,), device="cuda", generator=g)]
    idx = (idx + torch.randint(0, s_kv, (s_q // 2, 1), device="cuda", generator=g, dtype=torch.int32)) % s_kv
    if tail_invalid:
        idx[:, int(topk * (1 - tail_invalid)):] = -1
    return q, kv, idx.reshape(s_q // 2, 1, topk).contiguous(), w1, w2


def test_prefill_full_size_addressing():
    """sq = 65 536 query tokens (the headline size; Q alone is 2.2 GB): every byte offset beyond 2^31 must be
    formed in 64 bits.  (The reference forms token x stride in 32 bits, csrc/attention/prefill_kernel.cuh:266-269,
    and cannot run this size.)  The tail of the batch -- tokens past 63 551, where a 32-bit product wraps -- must
    equal what a call on that slice alone returns, bit for bit, and the oracle on sampled pairs."""
    import mxdsa_b200 as M
    s_q, s_kv, topk = 65536, 16384, 128
    q, kv, idx, w1, w2 = _big_prefill(s_q, s_kv, topk, seed=11)
    sc = 512 ** -0.5
    out, mxl, lse = M.dual_mxfp8_head64_sparse_prefill_fwd(q, kv, idx, sc, w1, w2, None, None)
    M.device_fault()
    lo = 63488
    out_t, mxl_t, lse_t = M.dual_mxfp8_head64_sparse_prefill_fwd(q[lo:], kv, idx[lo // 2:], sc, w1, w2, None, None)
    M.device_fault()
    assert torch.equal(out[lo:].view(torch.int16), out_t.view(torch.int16))
    assert torch.equal(lse[lo:], lse_t) and torch.equal(mxl[lo:], mxl_t)
    pairs = [0, 31775, 31776, 32767]          # first pair, the two around the 2^31-byte mark, last pair
    rows = sorted(sum(([2 * p, 2 * p + 1] for p in pairs), []))
    ro, rm, rl = O.prefill_ref(q[rows].cpu().numpy(), kv.cpu().numpy(), idx[pairs].cpu().numpy(), sc, w1, w2,
                               None, None, level=1)
    check_against_oracle(out[rows].float().cpu().numpy(), ro)
    assert np.abs(lse[rows].cpu().numpy() - rl).max() <= 1e-3


def test_prefill_properties_at_headline_topk():
    """sq = 8192 query tokens against kv_len = 16384 with topk = 4096 (the headline tile count),
    10 % of every index row masked with -1 as in the multi-GPU configuration."""
    import mxdsa_b200 as M
    s_q, s_kv, topk = 8192, 16384, 4096
    q, kv, idx, w1, w2 = _big_prefill(s_q, s_kv, topk, seed=7, tail_invalid=0.1)
    sc = 512 ** -0.5
    out, mxl, lse = M.dual_mxfp8_head64_sparse_prefill_fwd(q, kv, idx, sc, w1, w2, None, None)
    # determinism
    out2, mxl2, lse2 = M.dual_mxfp8_head64_sparse_prefill_fwd(q, kv, idx, sc, w1, w2, None, None)
    assert torch.equal(out.view(torch.int16), out2.view(torch.int16)) and torch.equal(lse, lse2)
    # the -1 tail and an explicit length are the same mask
    lens = torch.full((s_q // 2,), int(topk * 0.9), dtype=torch.int32, device="cuda")
    idx_full = idx.clone()
    idx_full[:, :, int(topk * 0.9):] = 5
    out3, mxl3, lse3 = M.dual_mxfp8_head64_sparse_prefill_fwd(q, kv, idx_full, sc, w1, w2, None, lens)
    assert torch.equal(out.view(torch.int16), out3.view(torch.int16))
    assert torch.equal(lse, lse3) and torch.equal(mxl, mxl3)
    # doubling every V dimension scale (a power of two) doubles the output exactly; lse unchanged
    w1d = [(((w & 0xFF) + 1) * 0x01010101) for w in w1]
    w2d = [(((w & 0xFF) + 1) * 0x01010101) for w in w2]
    out4, _, lse4 = M.dual_mxfp8_head64_sparse_prefill_fwd(q, kv, idx, sc, w1d, w2d, None, None)
    assert torch.equal((out.float() * 2).to(torch.bfloat16).view(torch.int16), out4.view(torch.int16))
    assert torch.equal(lse, lse4)
    M.device_fault()
    # oracle on a sample of pairs
    pairs = [0, 1, 2047, 4095]
    rows = sorted(sum(([2 * p, 2 * p + 1] for p in pairs), []))
    ro, rm, rl = O.prefill_ref(q[rows].cpu().numpy(), kv.cpu().numpy(), idx[pairs].cpu().numpy(), sc, w1, w2,
                               None, None, level=1)
    o = out[rows].float().cpu().numpy()
    check_against_oracle(o, ro)
    assert np.abs(lse[rows].cpu().numpy() - rl).max() <= 1e-3
    assert np.abs(mxl[rows].cpu().numpy() - rm).max() <= 1e-3


def test_decode_properties_at_headline_shape():
    """batch 128, sq 6, main 128 + extra 4096 of 16384 per request: determinism, metadata reuse and
    an oracle check of a few requests."""
    import mxdsa_b200 as M
    from mxdsa_b200 import packing as P
    b, s_q, extra = 128, 6, 4096
    g = torch.Generator(device="cuda").manual_seed(11)
    q = P.pack_dual_q64(torch.randn(b * s_q, 64, 512, device="cuda", generator=g))[0].view(b, s_q, 64, 528)
    kvf, w1, w2 = P.make_rank1_kv((2 * b, 64, 1), device="cuda", generator=g)
    kv = P.pack_dual_decode_kv_pages(kvf)[0]
    wl = torch.tensor(O.w_words_to_log2(w1, w2), device="cuda")
    pool = torch.randn(256, 64, 1, 8, 64, device="cuda", generator=g)
    e = torch.ceil(torch.log2((pool.abs().amax(-1) / 448).clamp_min(2.0 ** -126)))
    pool = (pool * torch.exp2(e[..., :1] + wl - e).unsqueeze(-1)).reshape(256, 64, 1, 512)
    ekv = P.pack_dual_decode_kv_pages(pool)[0].repeat(b, 1, 1, 1)
    off = torch.arange(b, device="cuda", dtype=torch.int32)[:, None, None]
    idx = (torch.stack([torch.randperm(128, device="cuda", generator=g) for _ in range(b * s_q)])
           .int().view(b, s_q, 128) + off * 128).contiguous()
    eidx = (torch.stack([torch.randperm(16384, device="cuda", generator=g)[:extra] for _ in range(b * s_q)])
            .int().view(b, s_q, extra) + off * 16384).contiguous()
    sc = 512 ** -0.5
    o1 = M.dual_mxfp8_sparse_decode_fwd(q, kv, idx, None, None, None, None, ekv, eidx, None, 512, 512, sc, w1, w2)
    o2 = M.dual_mxfp8_sparse_decode_fwd(q, kv, idx, None, None, o1[2], o1[3], ekv, eidx, None, 512, 512, sc, w1, w2)
    M.device_fault()
    assert torch.equal(o1[0].view(torch.int16), o2[0].view(torch.int16)) and torch.equal(o1[1], o2[1])
    parts = o1[2].shape[0]
    sm = O.sched_meta_ref(b, 128, extra, parts)
    assert np.array_equal(o1[2].cpu().numpy()[:, :7], sm.meta[:, :7])
    assert np.array_equal(o1[3].cpu().numpy(), sm.num_splits)
    # oracle on requests 0, 5 (straddles parts) and b-1; indices re-based to a 3-request world
    sel = [0, 5, b - 1]
    qs = q[sel].cpu().numpy()
    kvs = torch.cat([kv[2 * r:2 * r + 2] for r in sel]).cpu().numpy()
    ekvs = torch.cat([ekv[256 * r:256 * r + 256] for r in sel]).cpu().numpy()
    idxs = np.stack([(idx[r].cpu().numpy() - r * 128 + i * 128) for i, r in enumerate(sel)])
    eidxs = np.stack([(eidx[r].cpu().numpy() - r * 16384 + i * 16384) for i, r in enumerate(sel)])
    ro, rl = O.decode_ref(qs, kvs, idxs, None, None, ekvs, eidxs, None, sc, w1, w2, level=0)
    o = o1[0][sel].float().cpu().numpy()
    l = o1[1].transpose(1, 2)[sel].cpu().numpy()
    # level 0 (no probability quantisation): the split pattern of the full batch is not reproduced,
    # so compare at the "ideal math" tolerance
    assert O.cosine(o, ro) >= 0.9995
    assert np.abs(l - rl).max() <= 1e-3


def test_entry_points_are_cuda_graph_capturable():
    """The reference's benchmark captures its calls in CUDA graphs (reference tests/benchmark.py:44-46):
    both operators must record into a graph without synchronising and replay to the eager results."""
    import mxdsa_b200 as M
    from mxdsa_b200 import packing as P
    g = torch.Generator(device="cuda").manual_seed(21)
    q = P.pack_dual_q64(torch.randn(32, 64, 512, device="cuda", generator=g))[0]
    kvf, w1, w2 = P.make_rank1_kv((1024, 1), device="cuda", generator=g)
    kv = P.pack_dual_prefill_kv64(kvf)[0]
    idx = torch.stack([torch.randperm(1024, device="cuda", generator=g)[:512] for _ in range(16)]).int().view(16, 1, 512)
    eager = M.dual_mxfp8_head64_sparse_prefill_fwd(q, kv, idx, 512 ** -0.5, w1, w2, None, None)
    # decode inputs: 4 requests, 2 pages of 64 each
    qd = P.pack_dual_q64(torch.randn(4 * 2, 64, 512, device="cuda", generator=g))[0].view(4, 2, 64, 528)
    pool = P.pack_dual_decode_kv_pages(P.make_rank1_kv((8, 64, 1), device="cuda", generator=g)[0])[0]
    didx = (torch.rand(8, 128, device="cuda", generator=g).argsort(1).int().view(4, 2, 128)
            + 128 * torch.arange(4, device="cuda", dtype=torch.int32)[:, None, None]).contiguous()
    first = M.dual_mxfp8_sparse_decode_fwd(qd, pool, didx, None, None, None, None, None, None, None, 512, 512,
                                           512 ** -0.5, w1, w2)
    meta, splits = first[2], first[3]
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):     # warm-up on the capture stream, as torch's graph notes ask
        M.dual_mxfp8_head64_sparse_prefill_fwd(q, kv, idx, 512 ** -0.5, w1, w2, None, None)
        M.dual_mxfp8_sparse_decode_fwd(qd, pool, didx, None, None, meta, splits, None, None, None, 512, 512, 512 ** -0.5,
                                       w1, w2)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        cap = M.dual_mxfp8_head64_sparse_prefill_fwd(q, kv, idx, 512 ** -0.5, w1, w2, None, None)
        capd = M.dual_mxfp8_sparse_decode_fwd(qd, pool, didx, None, None, meta, splits, None, None, None, 512, 512,
                                              512 ** -0.5, w1, w2)
    for _ in range(2):
        for t in (*cap, capd[0], capd[1]):
            t.zero_() if t.is_contiguous() else t.fill_(0)
        graph.replay()
        torch.cuda.synchronize()
        for a, b in zip(cap, eager):
            assert torch.equal(a, b)
        assert torch.equal(capd[0], first[0]) and torch.equal(capd[1], first[1])
    M.device_fault()


def test_host_buffer_prefill_matches_device_call():
    """mxdsa_b200.host.prefill_from_host (chunked, three streams) writes what one device call returns."""
    import mxdsa_b200 as M
    from mxdsa_b200 import host, packing as P
    g = torch.Generator(device="cuda").manual_seed(31)
    s_q = 6 * 64 + 2          # not a multiple of the chunk: ragged last chunk
    q = P.pack_dual_q64(torch.randn(s_q, 64, 512, device="cuda", generator=g))[0]
    kvf, w1, w2 = P.make_rank1_kv((2048, 1), device="cuda", generator=g)
    kv = P.pack_dual_prefill_kv64(kvf)[0]
    idx = torch.stack([torch.randperm(2048, device="cuda", generator=g)[:256] for _ in range(s_q // 2)]).int().view(-1, 1, 256)
    want = M.dual_mxfp8_head64_sparse_prefill_fwd(q, kv, idx, 512 ** -0.5, w1, w2, None, None)
    hq, hkv, hidx = q.cpu().pin_memory(), kv.cpu().pin_memory(), idx.cpu().pin_memory()
    h_out = torch.zeros((s_q, 64, 512), dtype=torch.bfloat16).pin_memory()
    h_mxl = torch.zeros((s_q, 64), dtype=torch.float32).pin_memory()
    h_lse = torch.zeros((s_q, 64), dtype=torch.float32).pin_memory()
    for _ in range(2):
        host.prefill_from_host(hq, hkv, hidx, 512 ** -0.5, w1, w2, h_out, h_mxl, h_lse, chunk_tokens=64)
        torch.cuda.current_stream().synchronize()
        assert torch.equal(h_out, want[0].cpu()) and torch.equal(h_mxl, want[1].cpu()) and torch.equal(h_lse, want[2].cpu())
        h_out.zero_()
