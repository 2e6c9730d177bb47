"""GPU parity of the block-selection kernels (window covers, top-k) and of paged
decoding.  Index outputs are compared bit for bit with the CPU oracle; paged
decoding is compared bit for bit with dense decoding of the same keys laid out
as a padded cache, and with fp32 math within the bf16 / fp16 tolerance."""
import numpy as np
import pytest
import torch

from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu


def _ops():
    from tritonops_b200 import ops
    return ops


@pytest.mark.parametrize("L,G", [(64, 64), (200, 256), (1, 0), (0, 128), (2, 0), (65, 1), (128, 64),
                                 (4096, 0), (0, 0), (129, 100)])
@pytest.mark.parametrize("nqb", [1, 5, 40])
def test_window_cover_prefill_equals_brute_force(L, G, nqb):
    ops = _ops()
    block = 64
    idx, cnt = ops.window_blocks_prefill(2, 3, nqb, L, G, block_size=block)
    ref_idx, ref_cnt = orc.window_to_block_lists(nqb * block, block, L, G)
    assert idx.shape[:3] == (2, 3, nqb)
    for b in range(2):
        for h in range(3):
            assert torch.equal(cnt[b, h].cpu(), ref_cnt)
            w = min(idx.shape[-1], ref_idx.shape[-1])
            assert torch.equal(idx[b, h, :, :w].cpu(), ref_idx[:, :w])
            assert (idx[b, h, :, w:] == -1).all()
            assert (ref_idx[:, w:] == -1).all()


def test_window_cover_prefill_feeds_block_list_prefill():
    """Whole-block cover >= exact window, so with block-aligned windows the block-list
    kernel on the generated lists equals the block-list oracle on the oracle's lists."""
    ops = _ops()
    from tritonops_b200 import _lib
    B, H, S, D, L, G = 1, 2, 512, 64, 128, 64
    g = torch.Generator().manual_seed(11)
    q, k, v = [torch.randn(B, S, H, D, generator=g).to(torch.bfloat16) for _ in range(3)]
    idx, cnt = ops.window_blocks_prefill(B, H, S // 64, L, G)
    o, _ = ops.prefill(q.cuda(), k.cuda(), v.cuda(), causal=True, sparsity=_lib.BLOCK_LIST,
                       block_idx=idx, block_cnt=cnt)
    cu = torch.tensor([0, S], dtype=torch.int32)
    ref, _ = orc.block_sparse_prefill_exact(q.reshape(1, B * S, H, D), k.reshape(1, B * S, H, D),
                                            v.reshape(1, B * S, H, D), cu, idx.cpu(), cnt.cpu())
    assert (o.float().cpu().reshape(ref.shape) - ref.float()).abs().max().item() <= 2e-2


@pytest.mark.parametrize("L,G", [(64, 64), (200, 128), (1024, 256), (1, 64), (0, 64), (64, 0), (100, 30)])
def test_window_cover_decode_equals_brute_force(L, G):
    ops = _ops()
    lens = [0, 1, 63, 64, 65, 700, 137, 4096, 129, 5000]
    block = 64
    idx, cnt = ops.window_blocks_decode(torch.tensor(lens, dtype=torch.int32).cuda(), 2, L, G, block_size=block)
    ref_idx, ref_cnt = orc.window_decode_block_cover(lens, block, L, G, idx.shape[-1])
    for h in range(2):
        assert torch.equal(cnt[:, h].cpu(), ref_cnt)
        assert torch.equal(idx[:, h].cpu(), ref_idx)
    # a small max_sel keeps the first entries
    idx2, cnt2 = ops.window_blocks_decode(torch.tensor(lens, dtype=torch.int32).cuda(), 1, L, G,
                                          block_size=block, max_sel=2)
    r2, c2 = orc.window_decode_block_cover(lens, block, L, G, 2)
    assert torch.equal(idx2[:, 0].cpu(), r2) and torch.equal(cnt2[:, 0].cpu(), c2)


def test_window_cover_decode_matches_window_decoding():
    """Block-aligned windows: block-list decoding on the generated lists == window decoding."""
    ops = _ops()
    from tritonops_b200 import _lib
    lens = [1024, 777, 64, 300]
    g = torch.Generator().manual_seed(3)
    q = torch.randn(4, 8, 128, generator=g).to(torch.bfloat16).cuda()
    kc = torch.randn(4, 1024, 2, 128, generator=g).to(torch.bfloat16).cuda()
    vc = torch.randn(4, 1024, 2, 128, generator=g).to(torch.bfloat16).cuda()
    sl = torch.tensor(lens, dtype=torch.int32).cuda()
    idx, cnt = ops.window_blocks_decode(sl, 2, 128, 64)
    o_blocks = ops.decode(q, kc, vc, seqlens=sl, sparsity=_lib.BLOCK_LIST, block_idx=idx, block_cnt=cnt,
                          block_size=64)
    ref = orc.block_sparse_decoding_exact(q.cpu(), kc.cpu(), vc.cpu(), lens, idx[:, :, :].cpu(), cnt.cpu())
    assert (o_blocks.float().cpu() - ref.float()).abs().max().item() <= 2e-2


@pytest.mark.parametrize("n,k", [(512, 64), (256, 8), (37, 5), (1, 1), (8192, 100), (300, 300), (64, 128)])
def test_topk_blocks_equals_oracle(n, k):
    ops = _ops()
    g = torch.Generator().manual_seed(n * 1000 + k)
    rows = 6
    s = torch.randn(rows, n, generator=g)
    s[1] = torch.round(s[1] * 2) / 2                  # many exact ties
    s[2] = 0.0                                         # all equal: lowest blocks win
    if n > 4:
        s[3, ::3] = float("nan")
        s[3, 1] = float("inf")
        s[3, 2] = float("-inf")
        s[4, 0] = -0.0
        s[4, 1] = 0.0
    nv = torch.tensor([n, max(n // 2, 1), n, n, max(n - 1, 1), 0], dtype=torch.int32)
    for ff, fl, use_nv in [(0, 0, False), (1, 1, True), (2, 3, True), (0, 1, False)]:
        idx, cnt = ops.topk_blocks(s.cuda(), k, n_valid=nv.cuda() if use_nv else None, force_first=ff,
                                   force_last=fl)
        ridx, rcnt = orc.topk_blocks(s.numpy(), k, nv.numpy() if use_nv else None, ff, fl)
        assert torch.equal(cnt.cpu(), rcnt), (ff, fl, use_nv)
        assert torch.equal(idx.cpu(), ridx), (ff, fl, use_nv)


def test_topk_blocks_strided_rows_and_leading_shape():
    ops = _ops()
    g = torch.Generator().manual_seed(5)
    big = torch.randn(2, 3, 700, generator=g).cuda()
    s = big[:, :, :512]                                # row stride 700
    idx, cnt = ops.topk_blocks(s, 64, force_last=1)
    ridx, rcnt = orc.topk_blocks(s.cpu().reshape(6, 512).numpy(), 64, None, 0, 1)
    assert idx.shape == (2, 3, 64) and cnt.shape == (2, 3)
    assert torch.equal(idx.cpu().reshape(6, 64), ridx) and torch.equal(cnt.cpu().reshape(6), rcnt)
    assert (idx[..., -1] == 511).all()


def test_topk_feeds_block_list_decoding():
    ops = _ops()
    from tritonops_b200 import _lib
    B, Hq, Hkv, D, T, block, k = 3, 8, 2, 128, 2048, 64, 8
    lens = [2048, 1000, 130]
    g = torch.Generator().manual_seed(9)
    q = torch.randn(B, Hq, D, generator=g).to(torch.bfloat16)
    kc = torch.randn(B, T, Hkv, D, generator=g).to(torch.bfloat16)
    vc = torch.randn(B, T, Hkv, D, generator=g).to(torch.bfloat16)
    scores = torch.randn(B, Hkv, T // block, generator=g)
    nv = torch.tensor([[(n + block - 1) // block] * Hkv for n in lens], dtype=torch.int32)
    idx, cnt = ops.topk_blocks(scores.cuda(), k, n_valid=nv.cuda().reshape(-1), force_first=1, force_last=1)
    o = ops.decode(q.cuda(), kc.cuda(), vc.cuda(), seqlens=torch.tensor(lens, dtype=torch.int32).cuda(),
                   sparsity=_lib.BLOCK_LIST, block_idx=idx, block_cnt=cnt, block_size=block)
    ref = orc.block_sparse_decoding_exact(q, kc, vc, lens, idx.cpu(), cnt.cpu())
    assert (o.float().cpu() - ref.float()).abs().max().item() <= 2e-2


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("page,D,Hq,Hkv", [(16, 128, 8, 2), (64, 128, 32, 8), (128, 64, 4, 4), (48, 96, 6, 1)])
def test_paged_decode_equals_padded_decode(dtype, page, D, Hq, Hkv):
    ops = _ops()
    lens = [1500, 1, 0, 777, page, page + 1, 2048]
    B = len(lens)
    max_pages = (2048 + page - 1) // page
    need = sum((n + page - 1) // page for n in lens)
    P = need + 7
    g = torch.Generator().manual_seed(page + D)
    perm = torch.randperm(P, generator=g)
    table = torch.full((B, max_pages), -1, dtype=torch.int32)
    it = 0
    for b, n in enumerate(lens):
        for i in range((n + page - 1) // page):
            table[b, i] = perm[it]
            it += 1
    q = torch.randn(B, Hq, D, generator=g).to(dtype)
    kp = torch.randn(P, page, Hkv, D, generator=g).to(dtype)
    vp = torch.randn(P, page, Hkv, D, generator=g).to(dtype)
    sl = torch.tensor(lens, dtype=torch.int32)
    o = ops.paged_decode(q.cuda(), kp.cuda(), vp.cuda(), table.cuda(), sl.cuda(), max_seqlen=2048)
    kc = orc.paged_to_padded(kp, table, lens, capacity=max_pages * page)
    vc = orc.paged_to_padded(vp, table, lens, capacity=max_pages * page)
    o_pad = ops.decode(q.cuda(), kc.cuda(), vc.cuda(), seqlens=sl.cuda(), max_seqlen=2048)
    assert torch.equal(o.cpu(), o_pad.cpu())             # same keys, same order, same arithmetic
    ref = orc.decoding_exact(q, kc, vc, lens)
    tol = 5e-3 if dtype == torch.float16 else 2e-2
    assert (o.float().cpu() - ref.float()).abs().max().item() <= tol
    assert o[2].abs().max().item() == 0.0


def test_paged_decode_rejects_bad_arguments():
    ops = _ops()
    q = torch.zeros(1, 4, 128, dtype=torch.bfloat16).cuda()
    pool = torch.zeros(4, 24, 1, 128, dtype=torch.bfloat16).cuda()      # page size not a multiple of 16
    table = torch.zeros(1, 2, dtype=torch.int32).cuda()
    sl = torch.tensor([10], dtype=torch.int32).cuda()
    with pytest.raises(ValueError):
        ops.paged_decode(q, pool, pool, table, sl)
    pool = torch.zeros(4, 32, 1, 128, dtype=torch.bfloat16).cuda()
    with pytest.raises(ValueError):
        ops.paged_decode(q, pool[:, :16], pool[:, :16], table, sl)       # pages not back to back
