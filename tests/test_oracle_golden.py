"""Pin the CPU oracle against outputs recorded from the reference itself
(tests/golden/make_golden.py): its naive torch paths and its Triton kernels
run by the Triton CPU interpreter."""
import math

import pytest
import torch

from cases import build, checksum, load_golden
from oracle import attention_oracle as orc

LOG2E = orc.LOG2E
GT = load_golden("golden_torch.npz")
GK = load_golden("golden_triton.npz")


def maxabs(a, b):
    return (a.float() - b.float()).abs().max().item()


def lens_of(i):
    return (i["cu"][1:] - i["cu"][:-1]).tolist()


@pytest.mark.parametrize("name", sorted(set(GT) | set(GK)))
def test_inputs_reproduce(name):
    i = build(name)
    for g in (GT, GK):
        if name in g:
            assert checksum(i) == g[name]["insum"]


# ---- restatements of the reference torch paths must match them bit for bit
@pytest.mark.parametrize("name", ["dense_a", "dense_b", "dense_c"])
def test_dense_refpath_bitexact(name):
    i = build(name)
    o = orc.dense_prefill_refpath(i["q"], i["k"], i["v"], i["cu"])
    assert torch.equal(o, GT[name]["o"])


def test_decoding_refpath_bitexact():
    i = build("decode_mha")
    o = orc.decoding_refpath(i["q"], i["k"], i["v"], i["cu"])
    assert torch.equal(o, GT["decode_mha"]["o"])


@pytest.mark.parametrize("G,L", [(64, 64), (128, 200), (256, 1024)])
def test_window_decoding_refpath_bitexact(G, L):
    i = build("sparse_decode_mha")
    o = orc.window_decoding_refpath(i["q"], i["k"], i["v"], i["cu"], G, L)
    assert torch.equal(o, GT["sparse_decode_mha"][f"o_G{G}_L{L}"])


@pytest.mark.parametrize("L,G", [(128, 0), (64, 100), (200, 256), (1, 0), (64, 128)])
def test_window_prefill_refpath_bitexact(L, G):
    i = build("window_bf16")
    o = orc.window_prefill_refpath(i["q"], i["k"], i["v"], i["cu"], None, L, G)
    assert torch.equal(o, GT["window_bf16"][f"o_L{L}_G{G}"])


# ---- the exact fp32 oracle agrees with the reference within the stated tolerance
@pytest.mark.parametrize("name", ["dense_a", "dense_b", "dense_c"])
def test_dense_exact_vs_reference_torch(name):
    i = build(name)
    o, _ = orc.dense_prefill_exact(i["q"], i["k"], i["v"], i["cu"])
    assert maxabs(o, GT[name]["o"]) <= 2e-2


def test_cfg1_exact_vs_reference():
    i = build("cfg1")
    o_c, lse_c = orc.dense_prefill_exact(i["q"], i["k"], i["v"], i["cu"], causal=True)
    o_n, _ = orc.dense_prefill_exact(i["q"], i["k"], i["v"], i["cu"], causal=False)
    assert maxabs(o_c, GT["cfg1"]["o_causal"]) <= 5e-3
    assert maxabs(o_n, GT["cfg1"]["o_noncausal"]) <= 5e-3
    # the Triton kernel itself (interpreter): O and base-2 LSE of prescaled scores
    assert maxabs(o_c, GK["cfg1"]["o"]) <= 5e-3
    assert maxabs(lse_c * LOG2E, GK["cfg1"]["lse2"]) <= 5e-3


def test_dense_ragged_exact_vs_reference_kernel():
    i = build("dense_ragged_f16")
    o, lse = orc.dense_prefill_exact(i["q"], i["k"], i["v"], i["cu"])
    assert maxabs(o, GK["dense_ragged_f16"]["o"]) <= 5e-3
    assert maxabs(lse * LOG2E, GK["dense_ragged_f16"]["lse2"]) <= 5e-3


@pytest.mark.parametrize("L,G", [(64, 100), (256, 256), (128, 64)])
def test_window_prefill_exact_vs_reference_kernel(L, G):
    i = build("dense_ragged_f16")
    o, lse = orc.window_prefill_exact(i["q"], i["k"], i["v"], i["cu"], local=L, glob=G)
    assert maxabs(o, GK["dense_ragged_f16"][f"win_o_L{L}_G{G}"]) <= 5e-3
    assert maxabs(lse * LOG2E, GK["dense_ragged_f16"][f"win_lse2_L{L}_G{G}"]) <= 5e-3


@pytest.mark.parametrize("L,G", [(128, 0), (64, 100), (200, 256), (1, 0), (64, 128)])
def test_window_prefill_exact_vs_reference_torch(L, G):
    i = build("window_bf16")
    o, _ = orc.window_prefill_exact(i["q"], i["k"], i["v"], i["cu"], local=L, glob=G)
    assert maxabs(o, GT["window_bf16"][f"o_L{L}_G{G}"]) <= 2e-2


def test_decoding_exact_vs_reference():
    i = build("decode_mha")
    o = orc.decoding_exact(i["q"], i["kc"], i["vc"], lens_of(i))
    assert maxabs(o, GT["decode_mha"]["o"]) <= 5e-3
    i = build("decode_gqa")
    o = orc.decoding_exact(i["q"], i["kc"], i["vc"], lens_of(i))
    assert maxabs(o, GK["decode_gqa"]["o"]) <= 5e-3


@pytest.mark.parametrize("chunk", [128, 512, 64])
def test_split_combine_equals_unsplit(chunk):
    i = build("decode_gqa")
    a = orc.decoding_exact(i["q"], i["kc"], i["vc"], lens_of(i))
    b = orc.decoding_split_combine(i["q"], i["kc"], i["vc"], lens_of(i), chunk=chunk)
    assert maxabs(a, b) <= 1e-5


@pytest.mark.parametrize("G,L", [(64, 64), (128, 200), (256, 1024)])
def test_window_decoding_exact_vs_reference(G, L):
    i = build("sparse_decode_mha")
    o = orc.window_decoding_exact(i["q"], i["kc"], i["vc"], lens_of(i), glob=G, local=L)
    assert maxabs(o, GT["sparse_decode_mha"][f"o_G{G}_L{L}"]) <= 5e-3
    i = build("sparse_decode_gqa")
    o = orc.window_decoding_exact(i["q"], i["kc"], i["vc"], lens_of(i), glob=G, local=L)
    assert maxabs(o, GK["sparse_decode_gqa"][f"o_G{G}_L{L}"]) <= 5e-3
    assert o[2].abs().max().item() == 0.0          # the length-0 sequence


# ---- block-index layouts tie back to the window semantics
@pytest.mark.parametrize("L,G", [(64, 0), (100, 70), (1, 0)])
def test_block_lists_cover_window_mask(L, G):
    i = build("dense_ragged_f16")
    lens = lens_of(i)
    # a block list built from the window, refined by the element mask, must
    # reproduce the window result when the window is block aligned
    B, Hq = len(lens), i["q"].shape[2]
    nqb = max((n + 63) // 64 for n in lens)
    per = [orc.window_to_block_lists(n, 64, L, G) for n in lens]
    mx = max(p[0].shape[1] for p in per)
    idx = torch.full((B, Hq, nqb, mx), -1, dtype=torch.int32)
    cnt = torch.zeros(B, Hq, nqb, dtype=torch.int32)
    for b, (ix, ct) in enumerate(per):
        idx[b, :, :ix.shape[0], :ix.shape[1]] = ix
        cnt[b, :, :ct.shape[0]] = ct
    o_blk, _ = orc.block_sparse_prefill_exact(i["q"], i["k"], i["v"], i["cu"], idx, cnt)
    # block lists are a superset of the window mask: equality holds for the
    # block-aligned window (L multiple of 64 covering whole blocks is not
    # guaranteed), so compare against the dense mask built from the lists
    for b, n in enumerate(lens):
        m = orc.block_list_mask(n, 64, idx[b, 0], cnt[b, 0])
        assert bool((m | ~orc.window_mask(n, L, G)).all())
    assert torch.isfinite(o_blk).all()


def test_block_sparse_decoding_full_list_equals_dense():
    i = build("decode_gqa")
    lens = lens_of(i)
    B, Hkv = len(lens), i["kc"].shape[2]
    nb = (max(lens) + 63) // 64
    idx = torch.arange(nb, dtype=torch.int32).expand(B, Hkv, nb).contiguous()
    a = orc.decoding_exact(i["q"], i["kc"], i["vc"], lens)
    b = orc.block_sparse_decoding_exact(i["q"], i["kc"], i["vc"], lens, idx)
    assert maxabs(a, b) <= 1e-5


@pytest.mark.parametrize("name", ["dense_a", "dense_b", "dense_c"])
def test_grads_exact_vs_reference_autograd(name):
    """fp32 gradients of the oracle against the reference torch path's autograd
    gradients (bf16 arithmetic): the reference test's tolerances
    (flash_attn_triton.py:1086-1089)."""
    i = build(name)
    g = GT[name]
    dq, dk, dv = orc.dense_prefill_grads_exact(i["q"], i["k"], i["v"], i["cu"], g["do"])
    torch.testing.assert_close(dq, g["dq"].float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(dk, g["dk"].float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(dv, g["dv"].float(), rtol=1e-1, atol=1e-1)
