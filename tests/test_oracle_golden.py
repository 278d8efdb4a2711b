"""Pins the CPU oracle against the reference's own kernels.

The fixtures under tests/golden/ are outputs of the unmodified reference extension on a B200
(tests/golden/gen_golden.py); the inputs are rebuilt here from their seeds and their hash is
checked, then the oracle must agree with the reference within the north-star tolerances (it
actually agrees to about one bf16 ulp)."""
import numpy as np
import pytest

import cases
from helpers import check_against_golden, load_golden
from oracle import mxdsa_oracle as O


@pytest.mark.parametrize("name", list(cases.PREFILL_CASES))
def test_prefill_oracle_matches_reference_kernel(name):
    g = load_golden(name)
    c = cases.build(name)
    assert str(g["input_hash"]) == cases.input_hash(c), "inputs rebuilt from the seed differ"
    out, mxl, lse = O.prefill_ref(c["q"], c["kv"], c["indices"], c["sm_scale"], c["w1"], c["w2"],
                                  c["attn_sink"], c["topk_length"], level=1)
    check_against_golden(g, out, lse, mxl, out_tol=5e-3)


@pytest.mark.parametrize("name", list(cases.DECODE_CASES))
def test_decode_oracle_matches_reference_kernel(name):
    g = load_golden(name)
    c = cases.build(name)
    cc = cases.DECODE_CASES[name]
    assert str(g["input_hash"]) == cases.input_hash(c)
    parts = int(g["num_sm_parts"])
    sm = O.sched_meta_ref(cc["b"], cc["topk"], cc.get("extra_topk", 0), parts, c["topk_length"],
                          c["extra_topk_length"])
    # integer work: bit exact (the 8th int of a record is uninitialised padding in the reference)
    assert np.array_equal(sm.meta[:, :7], g["sched_meta"][:, :7])
    assert np.array_equal(sm.num_splits, g["num_splits"])
    out, lse = O.decode_ref(c["q"], c["kv"], c["indices"], c["topk_length"], c["attn_sink"],
                            c["extra_kv"], c["extra_indices"], c["extra_topk_length"], c["sm_scale"],
                            c["w1"], c["w2"], level=1, sched=sm)
    assert tuple(g["lse_shape"]) == (cc["b"], 64, cc["s_q"])  # returned as a [b,64,s_q] view
    check_against_golden(g, out, lse, lse_is_b_h_s=True, out_tol=5e-3)


def test_scheduler_matches_reference_at_benchmark_shapes():
    s = load_golden("sched")
    for b in (64, 128):
        for extra in (0, 128, 1024, 4096):
            sm = O.sched_meta_ref(b, 128, extra, 24)
            assert np.array_equal(sm.meta[:, :7], s[f"meta_b{b}_e{extra}"][:, :7]), (b, extra)
            assert np.array_equal(sm.num_splits, s[f"splits_b{b}_e{extra}"]), (b, extra)


def test_semantic_probes():
    """Single-purpose runs of the reference kernel that fix how it reads its operands."""
    p = load_golden("probes")
    # Q memory block 2g+h is contracted with K block 8h+g
    assert list(p["pair_out"].argmax(1)) == [8 * (m % 2) + m // 2 for m in range(16)]
    # the Q scale byte used with K block k is k % 8, the K scale byte is k // 2
    assert list(np.log2(p["qscale_logit"] / 32)) == [1 + k % 8 for k in range(16)]
    assert list(np.log2(p["kscale_logit"] / 32)) == [1 + k // 2 for k in range(16)]
    # V uses the token's scale byte 0 only
    assert np.all(np.diag(p["kscale_out"]) == 2.0)
    # w1 word j scales dims [32j, 32j+32), w2 word j scales dims [256+32j, ...)
    assert list(np.log2(p["w_out"][::32])) == list(range(8)) + [j - 10 for j in range(8)]
    # byte (position // 32) % 4 of a w word applies to the key at that position of its tile
    assert list(p["w_byte_out"]) == [2.0, 1.0, 2.0, 1.0]
    # decode: queries 2p and 2p+1 follow index row p
    assert list(p["decode_row_out"]) == [0.25, 0.25, 0.5, 0.5, 1.0, 1.0]
    # the oracle's operand reading reproduces the pairing probe
    q = np.zeros((2, 64, 528), np.uint8)
    q[..., 32:64] = 0x38
    q[..., 512:] = 127
    qk = O.q_kernel_order(q)
    assert np.all(qk[0, 0, 256:288] == 1.0) and qk[0, 0].sum() == 32


def test_level0_is_the_ideal_the_kernel_approximates():
    """Level 0 (no probability quantisation) stays close to the reference in cosine but not in
    max-abs: the E4M3 probabilities are part of the contract."""
    name = "prefill_t64_peaked"
    g = load_golden(name)
    c = cases.build(name)
    out, _, lse = O.prefill_ref(c["q"], c["kv"], c["indices"], c["sm_scale"], c["w1"], c["w2"],
                                c["attn_sink"], c["topk_length"], level=0)
    from helpers import bf16_bits_to_f32
    kept = out.reshape(-1, 512)[g["out_kept"]]
    assert O.cosine(kept, bf16_bits_to_f32(g["out_rows"])) > 0.9999
    fin = np.isfinite(g["lse"])
    assert np.abs(lse[fin] - g["lse"][fin]).max() < 1e-3
