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


def prefill_unit_pieces(n_batch: int, n_kv_heads: int, world: int, rank: int) -> List[Tuple[int, int, int, int]]:
    """The (sequence, KV head) units of a prefill, numbered b * n_kv_heads + hk (the order of the
    reference grid's first axis, flash_attn_triton.py:83-91, taken per KV head so a query-head
    group stays with its KV head), split into `world` contiguous slices.  Returns rank's slice as
    rectangles (b0, b1, hk0, hk1): sequences b0..b1-1, KV heads hk0..hk1-1 -- at most three (the
    head tail of a first sequence, whole sequences, the head prefix of a last one)."""
    u0, u1 = contiguous_shard(n_batch * n_kv_heads, world, rank)
    pieces: List[Tuple[int, int, int, int]] = []
    while u0 < u1:
        b, hk = divmod(u0, n_kv_heads)
        if hk == 0 and u1 - u0 >= n_kv_heads:
            nb = (u1 - u0) // n_kv_heads
            pieces.append((b, b + nb, 0, n_kv_heads))
            u0 += nb * n_kv_heads
        else:
            hk1 = min(n_kv_heads, hk + (u1 - u0))
            pieces.append((b, b + 1, hk, hk1))
            u0 += hk1 - hk
    return pieces


def slice_prefill_piece(q, k, v, cu_seqlens: Sequence[int], piece: Tuple[int, int, int, int]):
    """Views of packed [1, T, H, D] prefill inputs for one rectangle of prefill_unit_pieces:
    (q, k, v, cu) with cu (host integers) rebased to the first sequence of the piece.  No copy:
    token rows are a contiguous range, heads a strided slice the kernels take as is."""
    b0, b1, hk0, hk1 = piece
    g = q.shape[2] // k.shape[2]
    t0, t1 = int(cu_seqlens[b0]), int(cu_seqlens[b1])
    cu = [int(cu_seqlens[b]) - t0 for b in range(b0, b1 + 1)]
    return q[:, t0:t1, hk0 * g:hk1 * g], k[:, t0:t1, hk0:hk1], v[:, t0:t1, hk0:hk1], cu


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
