"""GPU: the failure paths that a healthy run never takes, exercised without faulting or hanging anything.

  * the bounded waits' give-up path: a self-test kernel waits (with the attention kernel's own wait loops,
    limits turned down to about a millisecond) on a barrier that nobody arrives on, gives up, raises the device
    fault record and leaves through its tear-down; the host then sees MXDSA_ERR_DEVICE_TIMEOUT once, and the
    next ordinary call works;
  * decode indices outside the KV pool (stale or corrupt, e.g. -2 or beyond the last page) are skipped like -1
    and nothing is dereferenced.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

MXDSA_ERR_DEVICE_TIMEOUT = 7


def test_bounded_wait_gives_up_reports_and_leaves_the_context_usable():
    import mxdsa_b200
    from mxdsa_b200 import capi, packing as P
    L = capi.lib()
    stream = torch.cuda.current_stream().cuda_stream
    assert L.mxdsa_device_fault(stream) == 0
    before = L.mxdsa_selftest_teardowns(stream)
    assert L.mxdsa_selftest_bounded_wait(stream) == 0
    assert L.mxdsa_selftest_teardowns(stream) == before + 2            # both CTAs left through the tear-down
    assert L.mxdsa_device_fault(stream) == MXDSA_ERR_DEVICE_TIMEOUT      # reported ...
    assert L.mxdsa_device_fault(stream) == 0                             # ... once
    # an ordinary call afterwards
    g = torch.Generator(device="cuda").manual_seed(3)
    q = P.pack_dual_q64(torch.randn(8, 64, 512, device="cuda", generator=g))[0]
    kvf, w1, w2 = P.make_rank1_kv((256, 1), device="cuda", generator=g)
    kv = P.pack_dual_prefill_kv64(kvf)[0]
    idx = torch.stack([torch.randperm(256, device="cuda", generator=g)[:64] for _ in range(4)]).int().view(4, 1, 64)
    out, mxl, lse = mxdsa_b200.dual_mxfp8_head64_sparse_prefill_fwd(q, kv, idx, 512 ** -0.5, w1, w2, None, None)
    mxdsa_b200.device_fault()
    assert torch.isfinite(out.float()).all() and torch.isfinite(lse).all()


def test_decode_indices_outside_the_pool_are_skipped():
    import mxdsa_b200
    from mxdsa_b200 import packing as P
    from oracle import mxdsa_oracle as O
    torch.manual_seed(9)
    b, s, topk = 3, 2, 128
    q = P.pack_dual_q64(torch.randn(b * s, 64, 512, device="cuda"))[0].view(b, s, 64, 528)
    kvf, w1, w2 = P.make_rank1_kv((2 * b, 64, 1), device="cuda")        # 6 pages of 64 keys = 384 keys
    kv = P.pack_dual_decode_kv_pages(kvf)[0]
    pool = 2 * b * 64
    off = torch.arange(b, device="cuda", dtype=torch.int32)[:, None, None]
    idx = (torch.rand(b * s, 128, device="cuda").argsort(1).int().view(b, s, 128) + off * 128).contiguous()
    bad = idx.clone()
    hole = torch.rand(b, s, topk, device="cuda") < 0.2
    junk = torch.tensor([-2, -7, pool, pool + 5, 2 ** 30], device="cuda", dtype=torch.int32)
    bad[hole] = junk[torch.randint(0, junk.numel(), (int(hole.sum()),), device="cuda")]
    clean = idx.clone()
    clean[hole] = -1
    args = (None, None, None, None, None, None, None, 512, 512, 512 ** -0.5, w1, w2)
    o_bad, l_bad, meta, _ = mxdsa_b200.dual_mxfp8_sparse_decode_fwd(q, kv, bad, *args)
    mxdsa_b200.device_fault()
    o_clean, l_clean, _, _ = mxdsa_b200.dual_mxfp8_sparse_decode_fwd(q, kv, clean, *args)
    mxdsa_b200.device_fault()
    assert torch.equal(o_bad, o_clean) and torch.equal(l_bad, l_clean)
    # and the oracle agrees on what "skipped" means
    from helpers import check_against_oracle
    sm = O.sched_meta_ref(b, topk, 0, meta.shape[0], None, None)
    ro, rl = O.decode_ref(q.cpu().numpy(), kv.cpu().numpy(), bad.cpu().numpy(), None, None, None, None, None,
                          512 ** -0.5, w1, w2, level=1, sched=sm)[:2]
    check_against_oracle(o_bad.float().cpu().numpy(), ro)
