"""Whole-request decode schedule (CPU): the oracle's restatement of the rule has the properties the attention
kernel relies on -- every request in exactly one part, in order, never divided -- and stays balanced to within one
request.  (The CUDA scheduler is compared with this restatement bit for bit in tests/test_gpu_decode_whole.py.)"""
import numpy as np
import pytest

from oracle import mxdsa_oracle as O


@pytest.mark.parametrize("b,topk,extra,parts", [(128, 128, 4096, 24), (64, 128, 2048, 24), (3, 128, 0, 24), (40, 64, 512, 74),
                                                (1, 64, 0, 1), (200, 128, 4096, 7)])
def test_whole_schedule_properties(b, topk, extra, parts):
    rng = np.random.default_rng(b * 131 + parts)
    lens = rng.integers(0, topk + 1, size=b).astype(np.int32)
    elens = rng.integers(0, extra + 1, size=b).astype(np.int32) if extra else None
    for tl, el in ((None, None), (lens, elens)):
        s = O.sched_whole_ref(b, topk, extra, parts, tl, el)
        assert s.meta.shape == (parts, 8) and np.array_equal(s.num_splits, np.arange(b + 1))
        nblk = []
        for i in range(b):
            n = topk if tl is None else max(int(tl[i]), 1)
            if extra:
                n = -(-n // 64) * 64 + (extra if el is None else int(el[i]))
            nblk.append(max(n - 1, 0) // 64 + 1)
        nxt, loads = 0, []
        for rec in s.meta:
            assert rec[0] == nxt and rec[2] == 0 and rec[4] == 0 and rec[5] == 0 and rec[6] == 0
            if rec[1] >= rec[0]:
                assert rec[3] == nblk[rec[1]]          # the part ends with the whole last request
                loads.append(sum(nblk[rec[0]:rec[1] + 1]))
                nxt = rec[1] + 1
            else:
                assert rec[1] == rec[0] - 1
                loads.append(0)
        assert nxt == b
        assert max(loads) <= sum(nblk) / parts + max(nblk)
