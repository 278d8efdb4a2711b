"""Wire-format restatement checks that need no fixture: number formats and packers."""
import numpy as np

from oracle import mxdsa_oracle as O


def test_e4m3_roundtrip_all_codes():
    codes = np.arange(256, dtype=np.uint8)
    vals = O.e4m3_decode(codes)
    ok = ~np.isnan(vals)
    enc = O.e4m3_encode(vals[ok])
    # -0 encodes to 0x80, +0 to 0x00; every finite code is a fixed point
    assert np.array_equal(enc, codes[ok])
    assert vals[0x7E] == 448.0 and vals[0x38] == 1.0 and vals[0x01] == 2.0 ** -9


def test_e4m3_round_half_even_and_saturation():
    assert O.e4m3_encode(np.array([1.0625], np.float32))[0] == 0x38      # tie -> even (1.0)
    assert O.e4m3_encode(np.array([1.1875], np.float32))[0] == 0x3A      # tie -> even (1.25)
    assert O.e4m3_encode(np.array([1e9], np.float32))[0] == 0x7E
    assert O.e4m3_encode(np.array([-1e9], np.float32))[0] == 0xFE


def test_ue8m0_roundup():
    assert list(O.ue8m0_roundup(np.array([1.0, 1.0001, 0.5, 0.75]))) == [127, 128, 126, 127]


def test_q_pack_layout():
    rng = np.random.default_rng(1)
    q = rng.standard_normal((3, 64, 512)).astype(np.float32)
    packed, deq = O.pack_q(q)
    assert packed.shape == (3, 64, 528)
    assert np.array_equal(packed[..., 512:520], packed[..., 520:528])
    # scale g covers dims [32g,32g+32) and [256+32g, 256+32g+32)
    g = 3
    sc = O.ue8m0_decode(packed[0, 0, 512 + g])
    blk = np.concatenate([q[0, 0, 32 * g:32 * g + 32], q[0, 0, 256 + 32 * g:256 + 32 * g + 32]])
    assert sc >= np.abs(blk).max() / 448 > sc / 2
    assert np.abs(deq - q).max() < 0.3
    # paired storage is a pure byte permutation of the natural one
    paired, _ = O.pack_q(q, paired_storage=True)
    nat = packed[..., :512].reshape(3, 64, 2, 8, 32)
    assert np.array_equal(paired[..., :512].reshape(3, 64, 8, 2, 32), nat.swapaxes(-3, -2))


def test_kv_pack_layouts():
    rng = np.random.default_rng(2)
    kv, w1, w2 = O.rank1_kv(rng, (70, 1))
    packed, deq = O.pack_prefill_kv(kv)
    flat = packed.reshape(-1)
    slots = flat[70 * 512:].reshape(70, 16)
    assert np.array_equal(slots[:, :8], slots[:, 8:])
    # rank-1: scale byte g - scale byte 0 is the same for every token and equals log2 W[g]
    diff = slots[:, :8].astype(int) - slots[:, :1].astype(int)
    assert np.all(diff == diff[0])
    assert list(diff[0]) == list(O.w_words_to_log2(w1, w2))
    pages = rng.standard_normal((3, 64, 1, 512)).astype(np.float32)
    pp, _ = O.pack_decode_kv_pages(pages)
    assert pp.shape == (3, 64, 1, 528)
    one = pp.reshape(3, -1)
    d, s, _ = O.quantize_groups(pages, 64)
    assert np.array_equal(one[:, :64 * 512].reshape(3, 64, 512), d[:, :, 0])
    assert np.array_equal(one[:, 64 * 512:].reshape(3, 64, 16)[..., :8], s[:, :, 0])


def test_combine_matches_single_pass():
    rng = np.random.default_rng(3)
    # three splits of the same row must merge to the un-split softmax
    logits = rng.standard_normal((3, 64, 40)) * 3
    v = rng.standard_normal((3, 40, 512))
    m = logits.max(-1)
    p = np.exp(logits - m[..., None])
    l = p.sum(-1)
    o = np.einsum("srk,skd->srd", p, v) / l[..., None]
    lse2 = (m + np.log(l)) * O.LOG2E
    out, lse = O.combine_ref(lse2, o, None)
    allp = np.exp(logits.transpose(1, 0, 2).reshape(64, -1))
    ref = (allp @ v.reshape(-1, 512)) / allp.sum(-1, keepdims=True)
    assert np.allclose(out, ref, atol=1e-9)
    assert np.allclose(lse, np.log(allp.sum(-1)), atol=1e-9)
