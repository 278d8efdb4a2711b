"""Inputs the reference operator refuses and the extended prefill operator accepts (run with -m gpu).

The reference demands an even number of query tokens, topk % 64 == 0 and uint8 tensors
(csrc/bindings/binding.cpp:36-58).  dual_mxfp8_head64_sparse_prefill_fwd_ex lifts the three rules.  There is no
reference kernel to compare with for those inputs, so the checks are
  * against the CPU oracle, which follows the kernel's tile walk with the missing positions counted as not attended;
  * against the drop-in operator itself on an equivalent input the reference does accept: index rows padded with -1
    to the next multiple of 64 (the same key sequence, bit-equal result when the tile size stays the same), an even
    batch made by repeating the last token, the same bytes viewed as uint8.
"""
import numpy as np
import pytest
import torch

from helpers import check_against_oracle
from oracle import mxdsa_oracle as O

pytestmark = pytest.mark.gpu


def _inputs(s_q, s_kv, topk, seed):
    from mxdsa_b200 import packing as P
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = P.pack_dual_q64(torch.randn(s_q, 64, 512, device="cuda", generator=g))[0]
    kvf, w1, w2 = P.make_rank1_kv((s_kv, 1), device="cuda", generator=g)
    kv = P.pack_dual_prefill_kv64(kvf)[0]
    pairs = (s_q + 1) // 2
    idx = torch.rand(pairs, s_kv, device="cuda", generator=g).argsort(1)[:, :topk].int()
    idx[:, ::7] = -1                                     # holes, as a caller's mask leaves them
    if pairs > 1:
        idx[1, topk // 2:] = -1                          # a row whose second half is empty
    return q, kv, idx.reshape(pairs, 1, topk).contiguous(), w1, w2


def _impls():
    import mxdsa_b200
    return {"extension": mxdsa_b200, "ctypes": mxdsa_b200.api}


@pytest.mark.parametrize("impl", ["extension", "ctypes"])
@pytest.mark.parametrize("s_q,topk", [(5, 200), (7, 1000), (1, 64), (6, 1), (4, 577)])
def test_extended_prefill_against_oracle_and_padded_call(impl, s_q, topk):
    import mxdsa_b200
    M = _impls()[impl]
    s_kv = 2048
    q, kv, idx, w1, w2 = _inputs(s_q, s_kv, topk, seed=31 * s_q + topk)
    sc = 512 ** -0.5
    sink = torch.linspace(-1.0, 1.0, 64, device="cuda")
    lens = torch.full(((s_q + 1) // 2,), topk, device="cuda", dtype=torch.int32)
    lens[0] = max(topk - 3, 1)
    out, mxl, lse = M.dual_mxfp8_head64_sparse_prefill_fwd_ex(q, kv, idx, sc, w1, w2, sink, lens)
    mxdsa_b200.device_fault()
    assert tuple(out.shape) == (s_q, 64, 512) and tuple(lse.shape) == (s_q, 64)

    ro, rm, rl = O.prefill_ref(q.cpu().numpy(), kv.cpu().numpy(), idx.cpu().numpy(), sc, w1, w2,
                               sink.cpu().numpy(), lens.cpu().numpy(), level=1)
    check_against_oracle(out.float().cpu().numpy(), ro)
    lse_h, mxl_h = lse.cpu().numpy(), mxl.cpu().numpy()
    fin = np.isfinite(rl)
    assert np.array_equal(np.isposinf(lse_h), np.isposinf(rl)) and np.abs(lse_h[fin] - rl[fin]).max(initial=0) <= 1e-3
    assert np.array_equal(np.isneginf(mxl_h), np.isneginf(rm)) and np.abs(mxl_h[fin] - rm[fin]).max(initial=0) <= 1e-3

    # the same work phrased within the reference's rules: even batch, index rows padded with -1
    pad_topk = -(-topk // 64) * 64
    qe = torch.cat([q, q[-1:]]) if s_q % 2 else q
    idx_e = torch.full((idx.size(0), 1, pad_topk), -1, device="cuda", dtype=torch.int32)
    idx_e[:, :, :topk] = idx
    out_e, mxl_e, lse_e = M.dual_mxfp8_head64_sparse_prefill_fwd(qe, kv, idx_e, sc, w1, w2, sink, lens)
    mxdsa_b200.device_fault()
    if (topk >= 512) == (pad_topk >= 512):               # same tile size: the same arithmetic, bit for bit
        assert torch.equal(out, out_e[:s_q]) and torch.equal(lse, lse_e[:s_q]) and torch.equal(mxl, mxl_e[:s_q])
    else:                                                # 64-key tiles here, 128-key tiles there
        assert float((out.float() - out_e[:s_q].float()).abs().max()) <= 2e-2
        assert float((lse - lse_e[:s_q]).abs().max()) <= 1e-3


def test_float8_tensors_are_the_same_bytes():
    import mxdsa_b200
    q, kv, idx, w1, w2 = _inputs(4, 1024, 128, seed=5)
    sc = 512 ** -0.5
    a = mxdsa_b200.dual_mxfp8_head64_sparse_prefill_fwd(q, kv, idx, sc, w1, w2, None, None)
    for M in _impls().values():
        b = M.dual_mxfp8_head64_sparse_prefill_fwd_ex(q.view(torch.float8_e4m3fn), kv.view(torch.float8_e4m3fn), idx,
                                                      sc, w1, w2, None, None)
        mxdsa_b200.device_fault()
        assert all(torch.equal(x, y) for x, y in zip(a, b))
        with pytest.raises(RuntimeError, match="(?s).*torch.uint8"):
            M.dual_mxfp8_head64_sparse_prefill_fwd(q.view(torch.float8_e4m3fn), kv, idx, sc, w1, w2, None, None)


def test_decode_accepts_float8_like_the_reference():
    """The decode operator of the reference takes uint8 or float8_e4m3fn (dual_mxfp8_sparse_decode.h:67-74)."""
    import mxdsa_b200
    from mxdsa_b200 import packing as P
    torch.manual_seed(3)
    q = P.pack_dual_q64(torch.randn(4, 64, 512, device="cuda"))[0].view(2, 2, 64, 528)
    kvf, w1, w2 = P.make_rank1_kv((4, 64, 1), device="cuda")
    kv = P.pack_dual_decode_kv_pages(kvf)[0]
    idx = torch.rand(4, 256, device="cuda").argsort(1)[:, :128].int().view(2, 2, 128).contiguous()
    sc = 512 ** -0.5
    for M in _impls().values():
        a = M.dual_mxfp8_sparse_decode_fwd(q, kv, idx, None, None, None, None, None, None, None, 512, 512, sc, w1, w2)
        b = M.dual_mxfp8_sparse_decode_fwd(q.view(torch.float8_e4m3fn), kv.view(torch.float8_e4m3fn), idx, None, None,
                                           None, None, None, None, None, 512, 512, sc, w1, w2)
        mxdsa_b200.device_fault()
        assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
