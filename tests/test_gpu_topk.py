"""GPU: the index-selection kernel against the CPU oracle (stable sort), bit for bit: seeded normal
scores at the benchmark's shapes, heavy ties, NaN / -inf / signed zeros, ragged lengths, fewer
candidates than topk, rows longer than one register sweep, pair sharing, pool offsets -- and the
selected rows fed into the attention operator."""
import numpy as np
import pytest
import torch

from oracle import mxdsa_oracle as O

pytestmark = pytest.mark.gpu


def _run(scores, topk, lengths=None, pair=False, row_offset=None):
    from mxdsa_b200.indexer import select_topk_indices
    dev = torch.device("cuda:0")
    t = torch.from_numpy(scores).to(dev)
    ln = None if lengths is None else torch.from_numpy(np.asarray(lengths, np.int32)).to(dev)
    ro = None if row_offset is None else torch.from_numpy(np.asarray(row_offset, np.int32)).to(dev)
    idx, cnt = select_topk_indices(t, topk, ln, pair, ro)
    torch.cuda.synchronize()
    return idx.cpu().numpy(), cnt.cpu().numpy()


def _check(scores, topk, lengths=None, pair=False, row_offset=None):
    got_i, got_c = _run(scores, topk, lengths, pair, row_offset)
    ref_i, ref_c = O.topk_select_ref(scores, topk, lengths, pair, row_offset)
    assert np.array_equal(got_c, ref_c)
    assert np.array_equal(got_i, ref_i)


@pytest.mark.parametrize("s_kv,topk", [(16384, 4096), (16384, 128), (1024, 128), (4096, 2048), (8, 64), (16388, 512), (16384, 6000), (40000, 9000)])
def test_normal_scores(s_kv, topk):
    rng = np.random.default_rng(s_kv + topk)
    _check(rng.standard_normal((37, s_kv)).astype(np.float32), topk)


def test_agrees_with_torch_topk_on_distinct_scores():
    rng = np.random.default_rng(5)
    s = rng.permuted(np.tile(np.arange(16384, dtype=np.float32), (8, 1)), axis=1) * 0.37 - 900.0
    got_i, got_c = _run(s, 2048)
    want = torch.topk(torch.from_numpy(s), 2048, dim=1).indices.sort(dim=1).values.numpy().astype(np.int32)
    assert np.array_equal(got_i, want) and (got_c == 2048).all()


def test_ties_go_to_the_smaller_index():
    rng = np.random.default_rng(11)
    few = rng.integers(0, 5, size=(9, 16384)).astype(np.float32)          # five distinct values
    _check(few, 4096)
    _check(few, 5000)                                                      # beyond the staged row size
    _check(np.full((3, 2048), 1.5, np.float32), 512)                       # every key ties
    close = (1.0 + rng.integers(0, 7, size=(5, 8192)) * 2.0 ** -23).astype(np.float32)   # differ in the last bits only
    _check(close, 1000)


def test_special_values():
    rng = np.random.default_rng(13)
    s = rng.standard_normal((6, 4096)).astype(np.float32)
    s[0, ::3] = np.nan
    s[1, 100:] = -np.inf                       # 100 candidates < topk
    s[2, :] = -np.inf                          # none
    s[3, ::2] = 0.0
    s[3, 1::4] = -0.0                          # signed zeros tie
    s[4, 7] = np.inf
    s[4, 9] = -3.0e38
    s[5, :] = np.nan
    _check(s, 256)
    den = (rng.standard_normal((4, 2048)) * 1e-41).astype(np.float32)     # denormals order like any other float
    _check(den, 300)


def test_ragged_lengths_and_short_rows():
    rng = np.random.default_rng(17)
    s = rng.standard_normal((16, 8192)).astype(np.float32)
    lengths = np.array([0, 1, 3, 4, 5, 63, 64, 65, 511, 512, 2047, 4096, 8191, 8192, 9000, -5], np.int32)
    _check(s, 512, lengths=lengths)
    _check(s, 64, lengths=lengths)


def test_rows_longer_than_one_sweep():
    rng = np.random.default_rng(19)
    s = rng.standard_normal((5, 40000)).astype(np.float32)
    s[1] = np.round(s[1] * 4) / 4             # ties across sweeps
    _check(s, 4096, lengths=np.array([40000, 40000, 16385, 33000, 20], np.int32))


def test_pair_sharing_and_pool_offsets():
    rng = np.random.default_rng(23)
    s = rng.standard_normal((24, 16384)).astype(np.float32)
    s[0, ::5] = np.nan                         # ignored where the other token has a number
    s[1, ::10] = np.nan
    off = (np.arange(12) * 16384).astype(np.int32)
    _check(s, 2048, pair=True, row_offset=off, lengths=rng.integers(1, 16385, size=12).astype(np.int32))


def test_argument_rules():
    from mxdsa_b200.indexer import select_topk_indices
    dev = torch.device("cuda:0")
    with pytest.raises(RuntimeError):
        select_topk_indices(torch.zeros(4, 10, device=dev), 4)            # s_kv not a multiple of 4
    with pytest.raises(RuntimeError):
        select_topk_indices(torch.zeros(3, 16, device=dev), 4, pair=True)  # odd number of token rows
    with pytest.raises(RuntimeError):
        select_topk_indices(torch.zeros(4, 16), 4)                        # host tensor
    idx, cnt = select_topk_indices(torch.zeros(0, 16, device=dev), 4)
    assert idx.shape == (0, 4) and cnt.shape == (0,)


def test_selected_rows_drive_the_attention_operator():
    """Selection -> prefill: attending the selected keys of a length-limited, -1 padded row equals
    attending the same keys given as a full row plus topk_length (the -1 tail is never read)."""
    import mxdsa_b200
    from mxdsa_b200.indexer import select_topk_indices
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(29)
    s_q, s_kv, topk = 64, 1024, 128
    q = rng.standard_normal((s_q, 64, 512)).astype(np.float32)
    q_u8, _ = O.pack_q(q, paired_storage=True)
    kvf, w1, w2 = O.rank1_kv(rng, (s_kv, 1))
    kv_u8, _ = O.pack_prefill_kv(kvf)
    scores = rng.standard_normal((s_q, s_kv)).astype(np.float32)
    lengths = rng.integers(1, 200, size=s_q // 2).astype(np.int32)
    idx, cnt = select_topk_indices(torch.from_numpy(scores).to(dev), topk, torch.from_numpy(lengths).to(dev), pair=True)
    ref_i, ref_c = O.topk_select_ref(scores, topk, lengths, pair=True)
    assert np.array_equal(idx.cpu().numpy(), ref_i) and np.array_equal(cnt.cpu().numpy(), ref_c)
    tq, tkv = torch.from_numpy(q_u8).to(dev), torch.from_numpy(kv_u8).to(dev)
    out, mx, lse = mxdsa_b200.dual_mxfp8_head64_sparse_prefill_fwd(tq, tkv, idx.view(s_q // 2, 1, topk), 512 ** -0.5,
                                                                     w1, w2, None, None)
    full = idx.clone()
    full[full < 0] = 0
    out2, mx2, lse2 = mxdsa_b200.dual_mxfp8_head64_sparse_prefill_fwd(tq, tkv, full.view(s_q // 2, 1, topk), 512 ** -0.5,
                                                                        w1, w2, None, cnt)
    torch.cuda.synchronize()
    assert torch.equal(out, out2) and torch.equal(lse, lse2) and torch.equal(mx, mx2)
    ro, rm, rl = O.prefill_ref(q_u8, kv_u8, ref_i.reshape(s_q // 2, 1, topk), 512 ** -0.5, w1, w2, None, None)
    assert O.max_abs(out.float().cpu().numpy(), ro) <= 2e-2
    assert O.max_abs(lse.cpu().numpy(), rl) <= 1e-3
