"""Host-side partitioning logic and the max-over-ranks reduction on 2 gloo ranks."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tritonops_b200 import sharding, workloads


@pytest.mark.parametrize("n,world", [(128, 1), (128, 8), (32, 4), (7, 3), (3, 8)])
def test_contiguous_shard_partitions(n, world):
    spans = [sharding.contiguous_shard(n, world, r) for r in range(world)]
    assert spans[0][0] == 0 and spans[-1][1] == n
    for a, b in zip(spans, spans[1:]):
        assert a[1] == b[0]
    sizes = [e - b for b, e in spans]
    assert max(sizes) - min(sizes) <= 1


def test_balanced_shards_cover_and_balance():
    g = torch.Generator().manual_seed(2)
    lens = torch.randint(1024, 8193, (64,), generator=g).tolist()
    for world in (2, 4, 8):
        shards = sharding.balanced_shards(lens, world)
        assert sorted(i for s in shards for i in s) == list(range(64))
        loads = [sum(lens[i] for i in s) for s in shards]
        assert max(loads) <= 1.05 * (sum(lens) / world) + max(lens) / world


def test_head_sharding_keeps_gqa_groups():
    q = torch.zeros(1, 10, 8, 16)
    k = torch.zeros(1, 10, 4, 16)
    for r in range(2):
        qs, ks, vs = sharding.shard_prefill_heads(q, k, k, 2, r)
        assert qs.shape[2] == 4 and ks.shape[2] == 2


def test_workload_generators_are_seeded():
    a, b = workloads.cfg1(), workloads.cfg1()
    assert torch.equal(a.q, b.q) and a.flops == 4 * 2 * 128 * 128 * 64
    idx, cnt = workloads.block_sparse_lists(1, 2, 32, 8, 0.1, 3)
    assert idx.shape[:3] == (1, 2, 32) and int(cnt[0, 0, 0]) == 1
    for qb in range(32):
        row = idx[0, 0, qb, :int(cnt[0, 0, qb])].tolist()
        assert row == sorted(row) and row[-1] == qb and all(x in row for x in range(max(0, qb - 7), qb + 1))
    sel = workloads.topk_block_lists(2, 3, 512, 64, 4)
    assert sel.shape == (2, 3, 64) and bool((sel[..., -1] == 511).all())
    assert bool((sel[..., 1:] > sel[..., :-1]).all())
    f = workloads.block_sparse_flops(idx, cnt, 64, 128, 32 * 64)
    assert f == 4.0 * 128 * ((int(cnt.sum()) - 64) * 64 * 64 + 64 * (64 * 65 // 2))


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # each rank owns a slice of the (batch x head) units; timings reduce by max
        b, e = sharding.contiguous_shard(128, world, rank)
        mx = sharding.max_over_ranks(float(10 + rank))
        tot = sharding.sum_over_ranks(float(e - b))
        ret[rank] = (mx, tot)
    finally:
        dist.destroy_process_group()


def test_two_rank_reduction_gloo():
    world = 2
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, 29531, ret), nprocs=world, join=True)
        assert ret[0] == ret[1] == (11.0, 128.0)
