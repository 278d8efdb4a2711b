"""mxdsa_decode_fwd_static: decode for callers that cannot allocate device memory.

Collected last on purpose (file name), so that a failure here cannot hide the other tests.  The
entry point keeps the split-KV partials in an array inside the library image instead of taking a
workspace from the caller; it must give bit-identical results to mxdsa_decode_fwd, also on a second
call that finds the previous call's partials still in the array."""
import ctypes as C

import numpy as np
import pytest
import torch

import cases
from helpers import decode_params

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["decode_main_only", "decode_mtp"])
def test_static_scratch_decode_matches_caller_scratch_decode(name):
    from mxdsa_b200 import capi
    L = capi.lib()
    c = cases.build(name)
    t = lambda x: None if x is None else torch.from_numpy(np.ascontiguousarray(x)).cuda()
    q, kv, idx, ekv, eidx = t(c["q"]), t(c["kv"]), t(c["indices"]), t(c["extra_kv"]), t(c["extra_indices"])
    b, s_q = q.shape[:2]
    parts = L.mxdsa_num_sm_parts(torch.cuda.current_device(), s_q)
    need = L.mxdsa_decode_workspace_bytes(b, s_q, parts)
    assert 0 < need <= capi.STATIC_SCRATCH_BYTES, "case must fit the built-in scratch"
    meta = torch.empty((parts, 8), dtype=torch.int32, device="cuda")
    splits = torch.empty((b + 1,), dtype=torch.int32, device="cuda")
    sp = capi.SchedParams(b=b, s_q=s_q, topk=idx.shape[2], extra_topk=eidx.shape[2] if eidx is not None else 0,
                          topk_length=None, extra_topk_length=None, num_sm_parts=parts,
                          sched_meta=meta.data_ptr(), num_splits=splits.data_ptr(),
                          stream=torch.cuda.current_stream().cuda_stream)
    capi.check(L.mxdsa_decode_sched(C.byref(sp)), "sched")

    def run(static):
        out = torch.full((b, s_q, 64, 512), float("nan"), dtype=torch.bfloat16, device="cuda")
        lse = torch.full((b, s_q, 64), float("nan"), dtype=torch.float32, device="cuda")
        ws = None if static else torch.empty(need, dtype=torch.uint8, device="cuda")
        p = decode_params(capi, c, (q, kv, idx, ekv, eidx), out, lse, meta, splits, parts, ws)
        fn = L.mxdsa_decode_fwd_static if static else L.mxdsa_decode_fwd
        capi.check(fn(C.byref(p)), "decode")
        capi.check(L.mxdsa_device_fault(torch.cuda.current_stream().cuda_stream), "fault")
        return out, lse

    ref_out, ref_lse = run(static=False)
    assert not torch.isnan(ref_out.float()).any()
    for _ in range(2):      # the second call finds the first call's partials in the array
        out, lse = run(static=True)
        assert torch.equal(out.view(torch.int16), ref_out.view(torch.int16))
        assert torch.equal(lse, ref_lse)


def test_static_scratch_decode_rejects_oversized_problems():
    from mxdsa_b200 import capi
    L = capi.lib()
    # (b + parts) * s_q partial slots of 64*513*4 bytes: far beyond the built-in array
    p = capi.DecodeParams(b=128, s_q=6, topk=128, num_sm_parts=24)
    assert L.mxdsa_decode_workspace_bytes(128, 6, 24) > capi.STATIC_SCRATCH_BYTES
    assert L.mxdsa_decode_fwd_static(C.byref(p)) == 6      # MXDSA_ERR_WORKSPACE
    assert L.mxdsa_decode_fwd_static(None) == 1            # MXDSA_ERR_NULL
