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


@pytest.mark.parametrize("B,Hkv,world", [(4, 32, 1), (4, 32, 2), (4, 32, 4), (4, 32, 8), (2, 16, 8), (3, 5, 4), (1, 2, 8)])
def test_prefill_unit_pieces_tile_the_units(B, Hkv, world):
    seen = []
    for r in range(world):
        for b0, b1, h0, h1 in sharding.prefill_unit_pieces(B, Hkv, world, r):
            assert 0 <= b0 < b1 <= B and 0 <= h0 < h1 <= Hkv
            assert (h0, h1) == (0, Hkv) or b1 == b0 + 1          # partial heads only inside one sequence
            seen += [b * Hkv + h for b in range(b0, b1) for h in range(h0, h1)]
    assert seen == list(range(B * Hkv))                           # disjoint, complete and in order


def _shard_worker(rank, world, port, ret):
    """Each rank attends over its own (sequence x KV head) rectangles (the CPU oracle stands in
    for the kernel here); gathered and put back in place they must equal the unsharded result
    bit for bit, because every (sequence, head) is computed independently."""
    from oracle import attention_oracle as orc
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)
        lens, Hq, Hkv, D = [70, 33, 128], 6, 3, 32
        cu = [0, 70, 103, 231]
        q = torch.randn(1, 231, Hq, D, generator=g).to(torch.bfloat16)
        k = torch.randn(1, 231, Hkv, D, generator=g).to(torch.bfloat16)
        v = torch.randn(1, 231, Hkv, D, generator=g).to(torch.bfloat16)
        mine = torch.zeros(1, 231, Hq, D, dtype=torch.bfloat16)
        for piece in sharding.prefill_unit_pieces(len(lens), Hkv, world, rank):
            qs, ks, vs, cus = sharding.slice_prefill_piece(q, k, v, cu, piece)
            o = orc.dense_prefill_refpath(qs, ks, vs, torch.tensor(cus, dtype=torch.int32))
            b0, b1, h0, h1 = piece
            mine[:, cu[b0]:cu[b1], h0 * 2:h1 * 2] = o
        bits = mine.view(torch.int16).to(torch.int32)       # disjoint pieces: a sum of bit patterns is a gather
        dist.all_reduce(bits, op=dist.ReduceOp.SUM)
        mine = bits.to(torch.int16).view(torch.bfloat16)
        full = orc.dense_prefill_refpath(q, k, v, torch.tensor(cu, dtype=torch.int32))
        ret[rank] = bool(torch.equal(mine, full))
    finally:
        dist.destroy_process_group()


def test_sharded_prefill_equals_unsharded_gloo():
    world = 2
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_shard_worker, args=(world, 29537, ret), nprocs=world, join=True)
        assert ret[0] is True and ret[1] is True


def test_host_pipeline_chunk_ranges():
    """The row ranges the host pipeline streams a sequence in: they tile [0, n), start on
    multiples of 256 and end on one or at n; a non-causal sequence is one range."""
    from tritonops_b200.host import chunk_ranges
    for n in (1, 255, 256, 257, 2048, 2049, 5000):
        for chunk in (256, 1024, 2048):
            r = chunk_ranges(n, chunk, True)
            assert r[0][0] == 0 and r[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(r, r[1:]))
            assert all(t0 % 256 == 0 and (t1 % 256 == 0 or t1 == n) and t1 > t0 for t0, t1 in r)
        assert chunk_ranges(n, 1024, False) == [(0, n)]
    assert chunk_ranges(0, 1024, True) == []
