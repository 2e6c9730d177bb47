"""Work partitioning over the GPUs of one box.  Every (sequence, KV-head group)
of a prefill and every sequence of a decode is independent (the reference grid
is (B*Hq, ...), flash_attn_triton.py:83-88), so ranks take disjoint slices and
no collective sits on the data path; only timings and, optionally, outputs are
gathered."""
from typing import List, Sequence, Tuple

import torch


def contiguous_shard(n_units: int, world: int, rank: int) -> Tuple[int, int]:
    """[begin, end) of the units rank owns when n_units are split as evenly as
    possible into contiguous slices (the first n_units % world ranks get one more)."""
    base, extra = divmod(n_units, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def balanced_shards(costs: Sequence[float], world: int) -> List[List[int]]:
    """Greedy longest-first assignment of units with unequal cost (ragged
    sequence lengths: cost = len for decoding, len**2 for causal prefill)."""
    order = sorted(range(len(costs)), key=lambda i: -costs[i])
    loads = [0.0] * world
    out: List[List[int]] = [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda j: loads[j])
        out[r].append(i)
        loads[r] += costs[i]
    return [sorted(s) for s in out]


def shard_prefill_heads(q, k, v, world: int, rank: int):
    """Slice packed [1,T,H,D] prefill inputs by KV head (a query-head group stays
    with its KV head).  Returns strided views; the kernels honour the strides."""
    hkv = k.shape[2]
    g = q.shape[2] // hkv
    b, e = contiguous_shard(hkv, world, rank)
    return q[:, :, b * g:e * g], k[:, :, b:e], v[:, :, b:e]


def max_over_ranks(value: float, device=None) -> float:
    """Max of a per-rank scalar (timings are reported as the slowest rank's)."""
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([value], dtype=torch.float64, device=device or "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(value: float, device=None) -> float:
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([value], dtype=torch.float64, device=device or "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())
