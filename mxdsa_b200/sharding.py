"""Multi-GPU decomposition of the path: no exchange step, only a partition of independent units.

Prefill is sharded by query PAIR (both tokens of a pair share one index row, so a pair never
straddles ranks), decode by request.  Every rank holds a full copy of the KV it needs; nothing is
communicated on the timed path.  The only collective use is bookkeeping around a measurement:
a barrier before/after and a MAX reduction of the per-rank device time.
"""
from __future__ import annotations

from typing import Tuple


def shard_range(n_units: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous [begin, end) slice of n_units for `rank`; sizes differ by at most one unit and
    the larger shards come first."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank/world {rank}/{world}")
    base, rem = divmod(n_units, world)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


def shard_query_tokens(s_q: int, rank: int, world: int) -> Tuple[int, int]:
    """Token range of a prefill batch for `rank` (always an even number of tokens)."""
    if s_q % 2:
        raise ValueError("s_q must be even: query tokens are processed in pairs")
    b, e = shard_range(s_q // 2, rank, world)
    return 2 * b, 2 * e


def max_over_ranks(value: float, group=None) -> float:
    """MAX of a per-rank number (device milliseconds) over the process group; identity when
    torch.distributed is not initialised."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        return float(value)
    dev = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
    t = torch.tensor([float(value)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())
