"""Seeded inputs of the packer pin (shared by the generator of packers.npz and by the tests).

Every array holds float32 values that are exactly representable in bf16, so the same values can be fed
to the torch packers (any dtype), the numpy oracle and the CUDA pack kernels.
"""
import numpy as np


def _bf16(x: np.ndarray) -> np.ndarray:
    u = np.asarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000          # round to nearest even at bit 16
    return u.astype(np.uint32).view(np.float32)


def edge_rows() -> np.ndarray:
    """512-wide rows that exercise the scale rule: all zero, amax/448 an exact power of two, just above one,
    huge, tiny, negative maxima, a single non-zero element, groups of very different magnitude."""
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
    grp[64:128] *= 1e-4
    grp[256:288] *= 300.0
    rows.append(grp)
    return _bf16(np.stack(rows))


def q_input() -> np.ndarray:
    """[6, 64, 512]: token 0 carries the edge rows in its first heads."""
    rng = np.random.default_rng(21)
    x = _bf16(rng.standard_normal((6, 64, 512)) * rng.choice([0.01, 1.0, 40.0], size=(6, 64, 1)))
    e = edge_rows()
    x[0, :e.shape[0]] = e
    return x


def prefill_kv_input() -> np.ndarray:
    """[96, 1, 512]: the first rows are the edge rows."""
    rng = np.random.default_rng(22)
    e = edge_rows()
    x = _bf16(rng.standard_normal((96, 1, 512)) * 3.0)
    x[:e.shape[0], 0] = e
    return x


def decode_kv_input() -> np.ndarray:
    """[3 pages, 32 keys, 1, 512]."""
    rng = np.random.default_rng(23)
    e = edge_rows()
    x = _bf16(rng.standard_normal((3, 32, 1, 512)) * rng.choice([0.1, 1.0, 25.0], size=(3, 32, 1, 1)))
    x[1, :e.shape[0], 0] = e
    return x
