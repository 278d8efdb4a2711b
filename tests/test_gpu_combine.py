"""GPU: mxdsa_decode_combine on its own reproduces what mxdsa_decode_fwd wrote for the requests that
the schedule splits over several parts (the reference sequences attention and combine as two
launches: reference csrc/bindings/dual_mxfp8_sparse_decode.h:204-241)."""
import ctypes as C

import numpy as np
import pytest
import torch

import cases
from helpers import decode_params

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["decode_many", "decode_mtp"])
def test_combine_alone_matches_decode(name):
    from mxdsa_b200 import capi
    L = capi.lib()
    c = cases.build(name)
    t = lambda x: None if x is None else torch.from_numpy(np.ascontiguousarray(x)).cuda()
    q, kv, idx, ekv, eidx = t(c["q"]), t(c["kv"]), t(c["indices"]), t(c["extra_kv"]), t(c["extra_indices"])
    b, s_q = q.shape[:2]
    parts = L.mxdsa_num_sm_parts(torch.cuda.current_device(), s_q)
    need = L.mxdsa_decode_workspace_bytes(b, s_q, parts)
    meta = torch.empty((parts, 8), dtype=torch.int32, device="cuda")
    splits = torch.empty((b + 1,), dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    sp = capi.SchedParams(b=b, s_q=s_q, topk=idx.shape[2], extra_topk=eidx.shape[2] if eidx is not None else 0,
                          topk_length=None, extra_topk_length=None, num_sm_parts=parts,
                          sched_meta=meta.data_ptr(), num_splits=splits.data_ptr(), stream=stream)
    capi.check(L.mxdsa_decode_sched(C.byref(sp)), "sched")
    out = torch.zeros((b, s_q, 64, 512), dtype=torch.bfloat16, device="cuda")
    lse = torch.zeros((b, s_q, 64), dtype=torch.float32, device="cuda")
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    p = decode_params(capi, c, (q, kv, idx, ekv, eidx), out, lse, meta, splits, parts, ws)
    capi.check(L.mxdsa_decode_fwd(C.byref(p)), "decode")
    capi.check(L.mxdsa_device_fault(stream), "fault")
    n_splits = (splits[1:] - splits[:-1]).cpu().numpy()
    split_req = np.nonzero(n_splits > 1)[0]
    assert len(split_req) > 0, "the case must contain requests that are split"
    # wipe what the combine step wrote and run it again on the same partials
    out2, lse2 = out.clone(), lse.clone()
    out2[split_req] = float("nan")
    lse2[split_req] = float("nan")
    cp = capi.CombineParams(b=b, s_q=s_q, num_sm_parts=parts, sched_meta=meta.data_ptr(), num_splits=splits.data_ptr(),
                            workspace=ws.data_ptr(), workspace_bytes=need, attn_sink=None, out=out2.data_ptr(),
                            lse=lse2.data_ptr(), stream=stream)
    capi.check(L.mxdsa_decode_combine(C.byref(cp)), "combine")
    torch.cuda.synchronize()
    assert torch.equal(out2.view(torch.int16), out.view(torch.int16))
    assert torch.equal(lse2, lse)


def test_combine_argument_rules():
    from mxdsa_b200 import capi
    L = capi.lib()
    assert L.mxdsa_decode_combine(None) == 1
    p = capi.CombineParams(b=1, s_q=1, num_sm_parts=1, sched_meta=16, num_splits=16, workspace=None, workspace_bytes=0,
                           out=32, lse=16)
    assert L.mxdsa_decode_combine(C.byref(p)) == 6      # MXDSA_ERR_WORKSPACE
