"""Decode without a combine pass (run with -m gpu): whole-request schedule + attention only.

No counterpart in the reference, whose scheduler always divides requests between parts.  Checks: the schedule
records equal the oracle's restatement of the rule bit for bit and give every request to exactly one part; the
outputs equal the oracle evaluated without a schedule (every row one pass) within the usual bounds and the reference
kernel's (which divides requests) up to the re-quantisation of divided requests; no scratch is needed; a schedule that does divide a request
raises the device fault record instead of writing through a null pointer."""
import ctypes as C

import numpy as np
import pytest
import torch

import cases
from helpers import LSE_MAX_ABS, check_against_oracle, decode_params, load_golden
from oracle import mxdsa_oracle as O

pytestmark = pytest.mark.gpu


def _t(x):
    return None if x is None else torch.from_numpy(np.ascontiguousarray(x)).cuda()


def _args(c):
    return (_t(c["q"]), _t(c["kv"]), _t(c["indices"]), _t(c["topk_length"]), _t(c["attn_sink"]), None, None,
            _t(c["extra_kv"]), _t(c["extra_indices"]), _t(c["extra_topk_length"]), 512, 512, c["sm_scale"], c["w1"], c["w2"])


@pytest.mark.parametrize("impl", ["extension", "ctypes"])
@pytest.mark.parametrize("name", list(cases.DECODE_CASES))
def test_whole_request_decode_matches_oracle_and_split_operator(name, impl):
    import mxdsa_b200
    M = mxdsa_b200 if impl == "extension" else mxdsa_b200.api
    c = cases.build(name)
    out, lse, meta, splits = M.dual_mxfp8_sparse_decode_fwd_whole(*_args(c))
    mxdsa_b200.device_fault()
    b, s_q = c["q"].shape[:2]
    et = 0 if c["extra_indices"] is None else c["extra_indices"].shape[2]
    ref_sched = O.sched_whole_ref(b, c["indices"].shape[2], et, meta.shape[0], c["topk_length"], c["extra_topk_length"])
    assert np.array_equal(meta.cpu().numpy(), ref_sched.meta) and np.array_equal(splits.cpu().numpy(), ref_sched.num_splits)
    owner = np.full(b, -1)
    for i, rec in enumerate(ref_sched.meta):
        for r in range(rec[0], rec[1] + 1):
            assert owner[r] == -1 and rec[2] == 0 and rec[5] == 0 and rec[6] == 0
            owner[r] = i
    assert (owner >= 0).all() and (np.diff(owner) >= 0).all()

    ro, rl = O.decode_ref(c["q"], c["kv"], c["indices"], c["topk_length"], c["attn_sink"], c["extra_kv"],
                          c["extra_indices"], c["extra_topk_length"], c["sm_scale"], c["w1"], c["w2"], level=1)[:2]
    check_against_oracle(out.float().cpu().numpy(), ro)
    lse_h = lse.transpose(1, 2).contiguous().cpu().numpy()      # back to [b, s_q, 64]
    fin = np.isfinite(rl)
    assert np.array_equal(np.isposinf(lse_h), np.isposinf(rl)) and np.abs(lse_h[fin] - rl[fin]).max(initial=0) <= LSE_MAX_ABS
    # Against the reference kernel's outputs for the same inputs.  Its schedule divides some requests, and a divided
    # request is re-quantised pass by pass (each pass has its own running maximum), so the two legitimately differ
    # at the level of the E4M3 re-quantisation of the probabilities: cosine, not the 2e-2 bound, is the check; the
    # normalisers (lse) are not affected by the re-quantisation and agree to 1e-3.
    g = load_golden(name)
    kept = out.float().cpu().numpy().reshape(-1, 512)[g["out_kept"]]
    gold = (np.asarray(g["out_rows"]).astype(np.uint32) << 16).view(np.float32)
    assert O.cosine(kept, gold) >= 0.9995 and O.max_abs(kept, gold) <= 0.5, (O.cosine(kept, gold), O.max_abs(kept, gold))
    glse = g["lse"].transpose(0, 2, 1)
    gfin = np.isfinite(glse)
    assert np.array_equal(np.isposinf(lse_h), np.isposinf(glse)) and np.abs(lse_h[gfin] - glse[gfin]).max(initial=0) <= LSE_MAX_ABS
    # the records are valid input for the split operator too, whose combine then finds nothing to do: same bits
    out2 = M.dual_mxfp8_sparse_decode_fwd(*(_args(c)[:5] + (meta, splits) + _args(c)[7:]))[0]
    mxdsa_b200.device_fault()
    assert torch.equal(out, out2)
    # and a second call that reuses the scheduling tensors gives the same bits
    out3 = M.dual_mxfp8_sparse_decode_fwd_whole(*(_args(c)[:5] + (meta, splits) + _args(c)[7:]))[0]
    mxdsa_b200.device_fault()
    assert torch.equal(out, out3)


def test_divided_schedule_without_partials_is_flagged_not_dereferenced():
    """mxdsa_decode_fwd_nocombine with the SPLITTING schedule: the kernel must not write partials through the
    null workspace; it raises the device fault record, and the next ordinary call works."""
    import mxdsa_b200
    from mxdsa_b200 import capi
    L = capi.lib()
    c = cases.build("decode_many")
    q, kv, idx, ekv, eidx = _t(c["q"]), _t(c["kv"]), _t(c["indices"]), _t(c["extra_kv"]), _t(c["extra_indices"])
    b, s_q = q.shape[:2]
    parts = L.mxdsa_num_sm_parts(torch.cuda.current_device(), s_q)
    meta = torch.empty((parts, 8), dtype=torch.int32, device="cuda")
    splits = torch.empty((b + 1,), dtype=torch.int32, device="cuda")
    sp = capi.SchedParams(b=b, s_q=s_q, topk=idx.shape[2], extra_topk=eidx.shape[2] if eidx is not None else 0,
                          topk_length=None, extra_topk_length=None, num_sm_parts=parts, sched_meta=meta.data_ptr(),
                          num_splits=splits.data_ptr(), stream=torch.cuda.current_stream().cuda_stream)
    capi.check(L.mxdsa_decode_sched(C.byref(sp)), "sched")
    assert int(splits[-1]) > b, "the case must contain a divided request"
    out = torch.zeros((b, s_q, 64, 512), dtype=torch.bfloat16, device="cuda")
    lse = torch.zeros((b, s_q, 64), dtype=torch.float32, device="cuda")
    p = decode_params(capi, c, (q, kv, idx, ekv, eidx), out, lse, meta, splits, parts, None)
    assert L.mxdsa_decode_fwd_nocombine(C.byref(p)) == 0
    with pytest.raises(RuntimeError):
        mxdsa_b200.device_fault()
    mxdsa_b200.device_fault()          # the record is cleared by the query
    out_ok = mxdsa_b200.dual_mxfp8_sparse_decode_fwd(*_args(c))[0]
    mxdsa_b200.device_fault()
    assert torch.isfinite(out_ok.float()).all()
