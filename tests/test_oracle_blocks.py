"""CPU checks of the oracle's block-selection helpers against independent
formulations (they pin the GPU kernels' integer outputs bit for bit)."""
import numpy as np
import torch

from oracle import attention_oracle as orc


def test_topk_oracle_matches_stable_argsort():
    rng = np.random.default_rng(0)
    s = rng.standard_normal((5, 97)).astype(np.float32)
    s[1] = np.round(s[1])                                  # ties
    idx, cnt = orc.topk_blocks(s, 10)
    for r in range(5):
        order = np.argsort(-s[r], kind="stable")[:10]      # ties -> lower block first
        assert idx[r].tolist() == sorted(order.tolist())
        assert int(cnt[r]) == 10


def test_topk_oracle_forced_nan_and_short_rows():
    s = np.array([[0.5, float("nan"), 3.0, -1.0, 2.0, float("-inf")]], dtype=np.float32)
    idx, cnt = orc.topk_blocks(s, 3, None, 1, 1)
    assert idx[0].tolist() == [0, 2, 5] and int(cnt[0]) == 3   # first and last forced, then the best
    idx, cnt = orc.topk_blocks(s, 4, np.array([2]), 0, 0)
    assert idx[0].tolist() == [0, 1, -1, -1] and int(cnt[0]) == 2
    idx, cnt = orc.topk_blocks(s, 5)
    assert idx[0].tolist() == [0, 2, 3, 4, 5]                  # NaN ranks below -inf


def test_decode_block_cover_matches_ranges():
    for L, G in [(64, 64), (200, 128), (1, 64), (0, 64), (64, 0), (100, 30)]:
        lens = [0, 1, 63, 64, 65, 700, 137, 4096]
        idx, cnt = orc.window_decode_block_cover(lens, 64, L, G, 64)
        for b, n in enumerate(lens):
            g = min(G, n)
            s2 = max(n - L, g)
            want = sorted(set(range((g + 63) // 64)) | (set(range(s2 // 64, (n + 63) // 64)) if s2 < n else set()))
            assert idx[b, :int(cnt[b])].tolist() == want


def test_paged_to_padded_round_trip():
    g = torch.Generator().manual_seed(0)
    pages = torch.randn(9, 16, 2, 8, generator=g)
    table = torch.tensor([[3, 7, 1], [8, 0, -1]], dtype=torch.int32)
    lens = [40, 17]
    pad = orc.paged_to_padded(pages, table, lens)
    assert pad.shape == (2, 48, 2, 8)
    assert torch.equal(pad[0, 16:32], pages[7]) and torch.equal(pad[0, 32:40], pages[1, :8])
    assert torch.equal(pad[1, 16:17], pages[0, :1]) and pad[1, 17:].abs().sum() == 0 and pad[0, 40:].abs().sum() == 0


def test_block_list_cpu_baseline_forms_agree_with_fp32_math():
    """The low-precision loops bench.py times as the CPU baseline of the block-list configs
    compute the same attention as the fp32 oracle, to bf16 accuracy."""
    from tritonops_b200 import workloads
    g = torch.Generator().manual_seed(0)
    n, H, D = 256, 2, 64
    q, k, v = (torch.randn(1, n, H, D, generator=g).to(torch.bfloat16) for _ in range(3))
    cu = torch.tensor([0, n], dtype=torch.int32)
    idx, cnt = workloads.block_sparse_lists(1, H, n // 64, 2, 0.5, 1)
    ref, _ = orc.block_sparse_prefill_exact(q, k, v, cu, idx, cnt)
    low = orc.block_sparse_prefill_refpath(q, k, v, cu, idx, cnt)
    assert (low.float() - ref).abs().max().item() <= 4e-2
    only = orc.block_sparse_prefill_refpath(q, k, v, cu, idx, cnt, heads={(0, 1)})
    assert torch.equal(only[0, :, 1], low[0, :, 1]) and only[0, :, 0].abs().max().item() == 0.0
    qd = torch.randn(2, 4, D, generator=g).to(torch.bfloat16)
    kc, vc = (torch.randn(2, 512, 2, D, generator=g).to(torch.bfloat16) for _ in range(2))
    sel = workloads.topk_block_lists(2, 2, 8, 3, 4)
    ref = orc.block_sparse_decoding_exact(qd, kc, vc, [512, 512], sel)
    low = orc.block_sparse_decoding_refpath(qd, kc, vc, sel)
    assert (low.float() - ref).abs().max().item() <= 4e-2
