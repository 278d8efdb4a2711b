"""CPU: the index-selection oracle against an independent statement of the same rule (torch.topk for
distinct scores, a plain Python loop for ties and special values)."""
import numpy as np
import torch

from oracle import mxdsa_oracle as O


def _loop(scores, topk, lengths=None):
    out = []
    for r, row in enumerate(scores):
        n = len(row) if lengths is None else min(max(int(lengths[r]), 0), len(row))
        cand = [(-(float(row[j]) + 0.0), j) for j in range(n) if not np.isnan(row[j]) and row[j] != -np.inf]
        cand.sort()
        out.append(sorted(j for _, j in cand[:topk]))
    return out


def test_distinct_scores_match_torch_topk():
    rng = np.random.default_rng(1)
    s = rng.permuted(np.tile(np.arange(1024, dtype=np.float32), (6, 1)), axis=1) - 400.0
    idx, cnt = O.topk_select_ref(s, 128)
    want = torch.topk(torch.from_numpy(s), 128, dim=1).indices.sort(dim=1).values.numpy()
    assert np.array_equal(idx, want) and (cnt == 128).all()


def test_ties_special_values_lengths_pairs_offsets():
    rng = np.random.default_rng(2)
    s = rng.integers(-2, 3, size=(8, 64)).astype(np.float32)
    s[0, ::3] = np.nan
    s[1, 5:] = -np.inf
    s[2, :] = -np.inf
    s[3, ::2] = -0.0
    lengths = np.array([64, 64, 64, 64, 0, 7, 100, -1], np.int32)
    idx, cnt = O.topk_select_ref(s, 16, lengths)
    want = _loop(s, 16, lengths)
    for r in range(8):
        assert cnt[r] == len(want[r])
        assert list(idx[r, :cnt[r]]) == want[r] and (idx[r, cnt[r]:] == -1).all()
    # pair rows: larger of the two tokens' scores, NaN on one side ignored; offsets added to selected entries only
    pidx, pcnt = O.topk_select_ref(s, 16, pair=True, row_offset=np.array([0, 100, 200, 300]))
    merged = np.fmax(s[0::2], s[1::2])
    want = _loop(merged, 16)
    for r in range(4):
        assert list(pidx[r, :pcnt[r]]) == [j + 100 * r for j in want[r]] and (pidx[r, pcnt[r]:] == -1).all()
