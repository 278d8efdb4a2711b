"""The wire format is pinned to the reference's own packers.

tests/golden/packers.npz holds the bytes that the reference's tests/mxfp8_test_utils.py (imported unmodified by
tests/golden/gen_packer_golden.py) produced for the seeded inputs of tests/golden/packer_cases.py, edge rows of
the scale rule included.  The numpy oracle and the torch packers of this repository must produce the same bytes.
"""
import os

import numpy as np
import torch

import packer_cases as PC
from helpers import GOLDEN_DIR
from oracle import mxdsa_oracle as O

G = np.load(os.path.join(GOLDEN_DIR, "packers.npz"))


def test_oracle_packers_equal_reference_bytes():
    assert np.array_equal(O.pack_q(PC.q_input())[0], G["q"])
    assert np.array_equal(O.pack_prefill_kv(PC.prefill_kv_input())[0], G["prefill_kv"])
    assert np.array_equal(O.pack_decode_kv_pages(PC.decode_kv_input())[0], G["decode_kv"])


def test_torch_packers_equal_reference_bytes():
    from mxdsa_b200 import packing as P
    for dtype in (torch.float32, torch.bfloat16):
        q = torch.from_numpy(PC.q_input()).to(dtype)
        assert np.array_equal(P.pack_dual_q64(q)[0].numpy(), G["q"])
        kv = torch.from_numpy(PC.prefill_kv_input()).to(dtype)
        assert np.array_equal(P.pack_dual_prefill_kv64(kv)[0].numpy(), G["prefill_kv"])
        pages = torch.from_numpy(PC.decode_kv_input()).to(dtype)
        assert np.array_equal(P.pack_dual_decode_kv_pages(pages)[0].numpy(), G["decode_kv"])


def test_paired_storage_is_a_permutation_of_the_reference_bytes():
    """paired_storage only reorders the 512 data bytes ([g][half][32] instead of natural order)."""
    want = G["q"]
    got = O.pack_q(PC.q_input(), paired_storage=True)[0]
    assert np.array_equal(got[..., 512:], want[..., 512:])
    nat = got[..., :512].reshape(*got.shape[:-1], 8, 2, 32).swapaxes(-3, -2).reshape(*got.shape[:-1], 512)
    assert np.array_equal(nat, want[..., :512])
