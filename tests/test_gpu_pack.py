"""GPU: the fused quantise-and-pack kernels produce, byte for byte, what the CPU oracle's packers
(and the torch packers of mxdsa_b200.packing) produce for the same values -- seeded normal inputs,
ragged sizes and the edge values of the scale rule."""
import numpy as np
import pytest
import torch

from oracle import mxdsa_oracle as O

pytestmark = pytest.mark.gpu


def _bf16(x: np.ndarray) -> np.ndarray:
    return O.bf16_round(x.astype(np.float32))


def _edge_rows() -> np.ndarray:
    """512-wide rows that exercise the scale rule: all zero, amax/448 an exact power of two, just above
    one, huge, tiny, negative maxima, a single non-zero element, values beyond +-448 after scaling never
    occur by construction."""
    rng = np.random.default_rng(7)
    rows = [np.zeros(512, np.float32)]
    for amax in (448.0, 1.75, 3.5, 1.7578125, 0.875, 7e4, 3e-5, 2.0 ** -120):
        r = rng.standard_normal(512).astype(np.float32)
        r = r / np.abs(r).max() * amax
        rows.append(r)
        rows.append(-r)
    one = np.zeros(512, np.float32)
    one[300] = -5.0
    rows.append(one)
    grp = rng.standard_normal(512).astype(np.float32)
    grp[64:128] *= 1e-4      # one KV group (and parts of two Q groups) far smaller than the rest
    grp[256:288] *= 300.0
    rows.append(grp)
    return _bf16(np.stack(rows))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("paired", [False, True])
def test_pack_q_matches_oracle(dtype, paired):
    from mxdsa_b200 import quantize as Z
    rng = np.random.default_rng(11)
    x = _bf16(rng.standard_normal((37, 64, 512)) * rng.choice([0.01, 1.0, 40.0], size=(37, 64, 1)))
    x[0, :_edge_rows().shape[0]] = _edge_rows()
    want, _ = O.pack_q(x, paired_storage=paired)
    got = Z.pack_dual_q64(torch.from_numpy(x).to("cuda", dtype), paired_storage=paired).cpu().numpy()
    assert got.shape == want.shape and got.dtype == np.uint8
    assert np.array_equal(got, want)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_pack_prefill_kv_matches_oracle_and_torch_packer(dtype):
    from mxdsa_b200 import packing as P, quantize as Z
    rng = np.random.default_rng(12)
    x = _bf16(rng.standard_normal((1000 + _edge_rows().shape[0], 1, 512)) * 3.0)
    x[:_edge_rows().shape[0], 0] = _edge_rows()
    want, _ = O.pack_prefill_kv(x)
    t = torch.from_numpy(x).to("cuda", dtype)
    got = Z.pack_dual_prefill_kv64(t)
    assert np.array_equal(got.cpu().numpy(), want)
    assert torch.equal(got, P.pack_dual_prefill_kv64(t)[0])


def test_pack_decode_pages_matches_oracle():
    from mxdsa_b200 import quantize as Z
    rng = np.random.default_rng(13)
    x = _bf16(rng.standard_normal((5, 64, 1, 512)))
    want, _ = O.pack_decode_kv_pages(x)
    got = Z.pack_dual_decode_kv_pages(torch.from_numpy(x).to("cuda", torch.bfloat16))
    assert np.array_equal(got.cpu().numpy(), want)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_cuda_packers_equal_reference_bytes(dtype):
    """The fused kernels against the bytes of the reference's own Python packers (tests/golden/packers.npz)."""
    import os
    import packer_cases as PC
    from helpers import GOLDEN_DIR
    from mxdsa_b200 import quantize as Z
    g = np.load(os.path.join(GOLDEN_DIR, "packers.npz"))
    cuda = lambda a: torch.from_numpy(a).to("cuda", dtype)
    assert np.array_equal(Z.pack_dual_q64(cuda(PC.q_input())).cpu().numpy(), g["q"])
    assert np.array_equal(Z.pack_dual_prefill_kv64(cuda(PC.prefill_kv_input())).cpu().numpy(), g["prefill_kv"])
    assert np.array_equal(Z.pack_dual_decode_kv_pages(cuda(PC.decode_kv_input())).cpu().numpy(), g["decode_kv"])


def test_packed_tensors_feed_the_attention_entry_point():
    """End of the widened path: fused packers -> prefill attention equals torch packers -> prefill attention."""
    import mxdsa_b200 as M
    from mxdsa_b200 import packing as P, quantize as Z
    g = torch.Generator(device="cuda").manual_seed(5)
    q = torch.randn(64, 64, 512, device="cuda", generator=g).bfloat16()
    kvf, w1, w2 = P.make_rank1_kv((512, 1), device="cuda", generator=g)
    kvf = kvf.bfloat16()
    idx = torch.stack([torch.randperm(512, device="cuda", generator=g)[:128] for _ in range(32)]).int().view(32, 1, 128)
    a = M.dual_mxfp8_head64_sparse_prefill_fwd(Z.pack_dual_q64(q), Z.pack_dual_prefill_kv64(kvf), idx, 512 ** -0.5, w1, w2)
    b = M.dual_mxfp8_head64_sparse_prefill_fwd(P.pack_dual_q64(q)[0], P.pack_dual_prefill_kv64(kvf)[0], idx, 512 ** -0.5,
                                              w1, w2)
    for x, y in zip(a, b):
        assert torch.equal(x, y)


def test_argument_rules():
    import ctypes
    from mxdsa_b200 import capi
    L = capi.lib()
    assert L.mxdsa_pack_q(None) == 1
    buf = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    p = capi.PackQParams(rows=1, src=buf.data_ptr() + 8, src_dtype=0, dst=buf.data_ptr())
    assert L.mxdsa_pack_q(ctypes.byref(p)) == 3          # misaligned source
    p = capi.PackQParams(rows=1, src=buf.data_ptr(), src_dtype=5, dst=buf.data_ptr())
    assert L.mxdsa_pack_q(ctypes.byref(p)) == 2          # unknown dtype
    k = capi.PackKVParams(rows=10, src=buf.data_ptr(), src_dtype=0, dst=buf.data_ptr(), rows_per_page=4)
    assert L.mxdsa_pack_kv(ctypes.byref(k)) == 2         # rows not a multiple of the page size
