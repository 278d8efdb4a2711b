"""Argument rules of the two entry points (reference csrc/bindings/binding.cpp:36-71 and
dual_mxfp8_sparse_decode.h:43-107): violations raise RuntimeError before any device work, from
the C++ extension and from the ctypes implementation alike."""
import pytest
import torch

import mxdsa_b200
from mxdsa_b200 import api

W = [0x7F7F7F7F] * 8


def _impls():
    return [mxdsa_b200, api]


def _prefill_args(s_q=4, heads=64, row=528, s_kv=8, topk=64, idx_dtype=torch.int32):
    return (torch.zeros(s_q, heads, row, dtype=torch.uint8), torch.zeros(s_kv, 1, 528, dtype=torch.uint8),
            torch.zeros(s_q // 2, 1, topk, dtype=idx_dtype))


@pytest.mark.parametrize("impl", _impls(), ids=["extension", "ctypes"])
@pytest.mark.parametrize("kwargs,needle", [
    (dict(s_q=3), "even, positive"),
    (dict(heads=32), "[s_q, 64, 528]"),
    (dict(row=512), "512 E4M3 bytes"),
    (dict(topk=96), "multiple of 64"),
])
def test_prefill_shape_rules(impl, kwargs, needle):
    q, kv, idx = _prefill_args(**kwargs)
    with pytest.raises(RuntimeError, match="(?s).*" + needle.replace("[", r"\[").replace("]", r"\]")):
        impl.dual_mxfp8_head64_sparse_prefill_fwd(q, kv, idx, 1.0, W, W, None, None)


@pytest.mark.parametrize("impl", _impls(), ids=["extension", "ctypes"])
def test_extended_prefill_lifts_three_rules_and_keeps_the_rest(impl):
    """Odd s_q, any topk and float8_e4m3fn pass the extended operator's checks (it then stops at the first rule
    both operators share that a CPU tensor breaks); the drop-in operator still refuses float8 inputs."""
    q = torch.zeros(3, 64, 528, dtype=torch.uint8).view(torch.float8_e4m3fn)
    kv = torch.zeros(8, 1, 528, dtype=torch.uint8).view(torch.float8_e4m3fn)
    idx = torch.zeros(2, 1, 100, dtype=torch.int32)
    with pytest.raises(RuntimeError, match="must be on CUDA"):
        impl.dual_mxfp8_head64_sparse_prefill_fwd_ex(q, kv, idx, 1.0, W, W, None, None)
    with pytest.raises(RuntimeError, match="(?s).*512 E4M3 bytes"):
        impl.dual_mxfp8_head64_sparse_prefill_fwd_ex(q[:, :, :512], kv, idx, 1.0, W, W, None, None)
    with pytest.raises(RuntimeError, match="(?s).*even, positive"):
        impl.dual_mxfp8_head64_sparse_prefill_fwd(q.view(torch.uint8), kv.view(torch.uint8), idx, 1.0, W, W, None, None)


@pytest.mark.parametrize("impl", _impls(), ids=["extension", "ctypes"])
def test_prefill_w_words_and_device(impl):
    q, kv, idx = _prefill_args()
    with pytest.raises(RuntimeError, match="8 pre-expanded"):
        impl.dual_mxfp8_head64_sparse_prefill_fwd(q, kv, idx, 1.0, W[:7], W, None, None)
    with pytest.raises(RuntimeError, match="must be on CUDA"):
        impl.dual_mxfp8_head64_sparse_prefill_fwd(q, kv, idx, 1.0, W, W, None, None)


def _decode_args(b=2, s_q=2, heads=64, topk=64):
    return (torch.zeros(b, s_q, heads, 528, dtype=torch.uint8), torch.zeros(4, 64, 1, 528, dtype=torch.uint8),
            torch.zeros(b, s_q, topk, dtype=torch.int32))


@pytest.mark.parametrize("impl", _impls(), ids=["extension", "ctypes"])
def test_decode_rules(impl):
    q, kv, idx = _decode_args(heads=128)
    with pytest.raises(RuntimeError, match="head64 only"):
        impl.dual_mxfp8_sparse_decode_fwd(q, kv, idx, None, None, None, None, None, None, None, 512, 512, 1.0, W, W)
    q, kv, idx = _decode_args()
    with pytest.raises(RuntimeError, match="d_qk=d_v=512"):
        impl.dual_mxfp8_sparse_decode_fwd(q, kv, idx, None, None, None, None, None, None, None, 576, 512, 1.0, W, W)
    q, kv, idx = _decode_args(topk=100)
    with pytest.raises(RuntimeError, match="multiple of 64"):
        impl.dual_mxfp8_sparse_decode_fwd(q, kv, idx, None, None, None, None, None, None, None, 512, 512, 1.0, W, W)
    q, kv, idx = _decode_args()
    with pytest.raises(RuntimeError, match="extra_indices must be provided"):
        impl.dual_mxfp8_sparse_decode_fwd(q, kv, idx, None, None, None, None, kv, None, None, 512, 512, 1.0, W, W)
    with pytest.raises(RuntimeError, match="require extra_kv"):
        impl.dual_mxfp8_sparse_decode_fwd(q, kv, idx, None, None, None, None, None, idx, None, 512, 512, 1.0, W, W)


def test_packers_match_the_oracle_packers_bit_for_bit():
    import numpy as np
    from mxdsa_b200 import packing as P
    from oracle import mxdsa_oracle as O
    g = torch.Generator().manual_seed(5)
    q = torch.randn(5, 64, 512, generator=g) * torch.exp2(torch.randint(-12, 12, (5, 64, 1), generator=g).float())
    a, da = P.pack_dual_q64(q)
    b, db = O.pack_q(q.numpy())
    assert np.array_equal(a.numpy(), b) and np.array_equal(da.numpy(), db)
    a, _ = P.pack_dual_q64(q, paired_storage=True)
    b, _ = O.pack_q(q.numpy(), paired_storage=True)
    assert np.array_equal(a.numpy(), b)
    kv, w1, w2 = P.make_rank1_kv((40, 1), generator=g)
    a, da = P.pack_dual_prefill_kv64(kv)
    b, db = O.pack_prefill_kv(kv.numpy())
    assert np.array_equal(a.numpy(), b) and np.array_equal(da.numpy(), db)
    slots = a.reshape(-1)[40 * 512:].reshape(40, 16)[:, :8].numpy().astype(int)
    assert (slots - slots[:, :1] == O.w_words_to_log2(w1, w2)).all()      # rank-1 scales
    pages = torch.randn(3, 64, 1, 512, generator=g)
    a = P.pack_dual_decode_kv_pages(pages)
    b, db = O.pack_decode_kv_pages(pages.numpy())
    assert np.array_equal(a[0].numpy(), b) and np.array_equal(a[1].numpy(), db)
    assert a[0].stride() == (64 * 528, 528, 528, 1)
