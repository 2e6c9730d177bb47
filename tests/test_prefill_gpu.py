"""GPU parity of the prefill path (dense causal / non-causal, window-sparse)
against the CPU oracle and the reference's recorded outputs.  Tolerances:
max-abs <= 5e-3 (fp16), <= 2e-2 (bf16) against fp32 math on the same rounded
inputs; LSE compared in natural log after converting the base-2 form."""
import math

import pytest
import torch

from cases import build, load_golden
from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu
TOL = {torch.float16: 5e-3, torch.bfloat16: 2e-2}
LOG2E = orc.LOG2E


def _mods():
    from tritonops_b200 import ops, workloads
    from tritonops_b200.flash_attn_triton import flash_attn_triton as fa
    from tritonops_b200.flash_attn_triton import flash_attn_sparse_attn_triton as sp
    return ops, workloads, fa, sp


def maxabs(a, b):
    return (a.float().cpu() - b.float().cpu()).abs().max().item()


def make(lens, hq, hkv, d, dtype, seed=0, dist="randn", scale=1.0):
    g = torch.Generator().manual_seed(seed)
    T = sum(lens)
    draw = torch.randn if dist == "randn" else torch.rand
    q = (draw(1, T, hq, d, generator=g) * scale).to(dtype)
    k = (draw(1, T, hkv, d, generator=g) * scale).to(dtype)
    v = draw(1, T, hkv, d, generator=g).to(dtype)
    cu = torch.zeros(len(lens) + 1, dtype=torch.int32)
    cu[1:] = torch.cumsum(torch.tensor(lens), 0)
    return q, k, v, cu


def test_golden_reference_outputs():
    """The inputs the reference itself was run on (torch path and Triton kernels)."""
    _, _, fa, sp = _mods()
    gt, gk = load_golden("golden_torch.npz"), load_golden("golden_triton.npz")
    for name in ("dense_a", "dense_b", "dense_c"):
        i = build(name)
        o = fa.flash_attn_triton.apply(i["q"].cuda(), i["k"].cuda(), i["v"].cuda(), i["cu"].cuda())
        assert maxabs(o, gt[name]["o"]) <= 2e-2
    for name in ("cfg1", "dense_ragged_f16"):
        i = build(name)
        d = i["q"].shape[-1]
        o, lse2 = fa.flash_attn_triton_fwd(i["q"].cuda(), i["k"].cuda(), i["v"].cuda(),
                                           i["cu"].cuda(), d ** -0.5 * LOG2E)
        assert maxabs(o, gk[name]["o"]) <= 5e-3
        assert maxabs(lse2, gk[name]["lse2"]) <= 5e-3
    i = build("cfg1")
    o = fa.flash_attention(i["q"].cuda(), i["k"].cuda(), i["v"].cuda(), i["cu"].cuda(), causal=False)
    assert maxabs(o, gt["cfg1"]["o_noncausal"]) <= 5e-3
    i = build("dense_ragged_f16")
    for L, G in [(64, 100), (256, 256), (128, 64)]:
        o, lse2 = sp.flash_attn_sparse_triton(i["q"].cuda(), i["k"].cuda(), i["v"].cuda(),
                                              i["cu"].cuda(), L, G)
        assert maxabs(o, gk["dense_ragged_f16"][f"win_o_L{L}_G{G}"]) <= 5e-3
        assert maxabs(lse2, gk["dense_ragged_f16"][f"win_lse2_L{L}_G{G}"]) <= 5e-3
    i = build("window_bf16")
    for L, G in [(128, 0), (64, 100), (200, 256), (1, 0), (64, 128)]:
        o, _ = sp.flash_attn_sparse_triton(i["q"].cuda(), i["k"].cuda(), i["v"].cuda(),
                                           i["cu"].cuda(), L, G)
        assert maxabs(o, gt["window_bf16"][f"o_L{L}_G{G}"]) <= 2e-2


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("B,maxlen,hq,hkv,d", [(3, 128, 2, 2, 96), (2, 256, 8, 4, 128), (4, 512, 4, 1, 64)])
def test_reference_test_configs(dtype, B, maxlen, hq, hkv, d):
    """flash_attn_triton.py:1001-1009: random lengths in [1, maxlen], U[0,1) inputs."""
    _, _, fa, _ = _mods()
    g = torch.Generator().manual_seed(42 + d)
    lens = torch.randint(1, maxlen + 1, (B,), generator=g).tolist()
    q, k, v, cu = make(lens, hq, hkv, d, dtype, seed=d, dist="rand")
    o = fa.flash_attn_triton.apply(q.cuda(), k.cuda(), v.cuda(), cu.cuda())
    ref, _ = orc.dense_prefill_exact(q, k, v, cu)
    assert maxabs(o, ref) <= TOL[dtype]


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("d", [32, 64, 96, 128])
def test_ragged_lengths_sweep(causal, d):
    """Every tile-boundary case: lengths around 1, 128, 256, 384 and beyond."""
    _, _, fa, _ = _mods()
    lens = [1, 2, 127, 128, 129, 255, 256, 257, 383, 385, 640, 5]
    q, k, v, cu = make(lens, 4, 2, d, torch.bfloat16, seed=d)
    o, lse = fa.flash_attention(q.cuda(), k.cuda(), v.cuda(), cu.cuda(), causal=causal, return_lse=True)
    ref, rl = orc.dense_prefill_exact(q, k, v, cu, causal=causal)
    assert maxabs(o, ref) <= 2e-2
    assert maxabs(lse, rl) <= 1e-3


def test_zero_length_sequences_and_fixed_length_form():
    ops, _, fa, _ = _mods()
    q, k, v, cu = make([0, 200, 0, 130], 2, 2, 64, torch.float16, seed=2)
    o = fa.flash_attn_triton.apply(q.cuda(), k.cuda(), v.cuda(), cu.cuda())
    ref, _ = orc.dense_prefill_exact(q, k, v, cu)
    assert maxabs(o, ref) <= 5e-3
    # [B,S,H,D] fixed-length form, with and without cu_seqlens, must agree
    g = torch.Generator().manual_seed(3)
    B, S = 3, 300
    q = torch.randn(B, S, 4, 128, generator=g).to(torch.bfloat16).cuda()
    k = torch.randn(B, S, 2, 128, generator=g).to(torch.bfloat16).cuda()
    v = torch.randn(B, S, 2, 128, generator=g).to(torch.bfloat16).cuda()
    o1 = fa.flash_attention(q, k, v, None, causal=True)
    cu = (torch.arange(B + 1, dtype=torch.int32) * S).cuda()
    o2 = fa.flash_attention(q.view(1, B * S, 4, 128), k.view(1, B * S, 2, 128),
                            v.view(1, B * S, 2, 128), cu, causal=True)
    assert torch.equal(o1.view(1, B * S, 4, 128), o2)
    ref, _ = orc.dense_prefill_exact(q.view(1, B * S, 4, 128).cpu(), k.view(1, B * S, 2, 128).cpu(),
                                     v.view(1, B * S, 2, 128).cpu(), cu.cpu())
    assert maxabs(o2, ref) <= 2e-2


def test_strided_heads_layout():
    """[B,H,S,D] storage seen through permuted [B,S,H,D] views (arbitrary strides)."""
    _, _, fa, _ = _mods()
    g = torch.Generator().manual_seed(4)
    B, H, S, D = 2, 4, 333, 128
    qs = torch.randn(B, H, S, D, generator=g).to(torch.bfloat16).cuda()
    ks = torch.randn(B, H, S, D, generator=g).to(torch.bfloat16).cuda()
    vs = torch.randn(B, H, S, D, generator=g).to(torch.bfloat16).cuda()
    o = fa.flash_attention(qs.permute(0, 2, 1, 3), ks.permute(0, 2, 1, 3), vs.permute(0, 2, 1, 3),
                           None, causal=True)
    cu = torch.arange(B + 1, dtype=torch.int32) * S
    pk = lambda t: t.permute(0, 2, 1, 3).reshape(1, B * S, H, D).cpu()
    ref, _ = orc.dense_prefill_exact(pk(qs), pk(ks), pk(vs), cu)
    assert maxabs(o.reshape(1, B * S, H, D), ref) <= 2e-2


@pytest.mark.parametrize("scale", [10.0, 30.0])
def test_large_magnitude_scores(scale):
    """Sharp softmax (scores up to hundreds): the lazy rescale must stay exact."""
    _, _, fa, _ = _mods()
    q, k, v, cu = make([700, 300], 2, 1, 64, torch.float16, seed=5, scale=scale)
    o = fa.flash_attn_triton.apply(q.cuda(), k.cuda(), v.cuda(), cu.cuda())
    ref, _ = orc.dense_prefill_exact(q, k, v, cu)
    assert torch.isfinite(o).all()
    assert maxabs(o, ref) <= 5e-3


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("L,G", [(128, 0), (64, 100), (64, 128), (200, 256), (1, 0), (100, 30),
                                 (256, 256), (300, 700), (1000, 1), (0, 64), (5000, 0)])
def test_window_prefill(dtype, L, G):
    """Oracle semantics of the module's torch function for every (L, G), including
    those where the reference Triton kernel deviates from it (guard at
    flash_attn_sparse_attn_triton.py:179)."""
    _, _, _, sp = _mods()
    lens = [1500, 129, 700, 1]
    q, k, v, cu = make(lens, 4, 2, 96, dtype, seed=L + G)
    o, lse2 = sp.flash_attn_sparse_triton(q.cuda(), k.cuda(), v.cuda(), cu.cuda(), L, G)
    ref, rl = orc.window_prefill_exact(q, k, v, cu, local=L, glob=G)
    assert maxabs(o, ref) <= TOL[dtype]
    fin = torch.isfinite(rl)
    assert maxabs(lse2.cpu()[fin], rl[fin] * LOG2E) <= 2e-3
    assert bool((lse2.cpu()[~fin] == -math.inf).all())


def test_cfg2_shape_properties():
    """Full config 2 (B=4,H=32,S=4096,D=128 causal bf16): sampled heads against
    fp32 math on the device, determinism, and prefix invariance (causal rows do
    not depend on later tokens)."""
    ops, wl, fa, _ = _mods()
    w = wl.cfg2("cuda")
    o, lse = ops.prefill(w.q, w.k, w.v, cu_seqlens=w.cu_seqlens, max_seqlen=w.max_seqlen)
    o_again, _ = ops.prefill(w.q, w.k, w.v, cu_seqlens=w.cu_seqlens, max_seqlen=w.max_seqlen)
    assert torch.equal(o, o_again)
    S = 4096
    tril = torch.ones(S, S, dtype=torch.bool, device="cuda").tril()
    for b, h in [(0, 0), (1, 13), (3, 31)]:
        sl = slice(b * S, (b + 1) * S)
        s = (w.q[0, sl, h].float() @ w.k[0, sl, h].float().T) * w.scale
        s = s.masked_fill(~tril, -math.inf)
        ref = torch.softmax(s, -1) @ w.v[0, sl, h].float()
        assert (o[0, sl, h].float() - ref).abs().max().item() <= 2e-2
        assert (lse[0, sl, h] - torch.logsumexp(s, -1)).abs().max().item() <= 1e-3
    # prefix invariance: the first 1000 tokens of sequence 2 alone give the same rows
    sl = slice(2 * S, 2 * S + 1000)
    cu1 = torch.tensor([0, 1000], dtype=torch.int32, device="cuda")
    o_pre, _ = ops.prefill(w.q[:, sl].contiguous(), w.k[:, sl].contiguous(), w.v[:, sl].contiguous(),
                           cu_seqlens=cu1, max_seqlen=1000)
    assert (o_pre.float() - o[:, sl].float()).abs().max().item() <= 2e-2


def test_status_word_stays_clear_and_errors():
    ops, _, fa, _ = _mods()
    q, k, v, cu = make([100], 4, 3, 64, torch.float16)
    with pytest.raises(ValueError):
        fa.flash_attn_triton.apply(q.cuda(), k.cuda(), v.cuda(), cu.cuda())      # 4 % 3
    q, k, v, cu = make([100], 2, 2, 48, torch.float16)
    with pytest.raises(ValueError):
        fa.flash_attn_triton.apply(q.cuda(), k.cuda(), v.cuda(), cu.cuda())      # head_dim 48


# ---------------------------------------------------------------- block-list sparsity
def _random_lists(lens, hq, p_keep, seed, local=2, empty_rows=()):
    """Per (b, h, q block): the `local` nearest causal blocks plus Bernoulli(p_keep)
    earlier ones, ascending, -1 padded; `empty_rows` q blocks get an empty list."""
    g = torch.Generator().manual_seed(seed)
    B = len(lens)
    nqb = max((n + 63) // 64 for n in lens)
    keep = torch.rand(B, hq, nqb, nqb, generator=g) < p_keep
    i = torch.arange(nqb)[:, None]
    j = torch.arange(nqb)[None, :]
    mask = ((keep & (j < i)) | ((j <= i) & (j > i - local)))
    for qb in empty_rows:
        mask[:, :, qb, :] = False
    cnt = mask.sum(-1).to(torch.int32)
    mx = max(int(cnt.max()), 1)
    key = torch.where(mask, j.expand_as(mask), torch.full_like(mask, nqb, dtype=torch.long))
    idx = key.sort(-1).values[..., :mx]
    idx = torch.where(idx >= nqb, torch.full_like(idx, -1), idx).to(torch.int32)
    return idx.contiguous(), cnt.contiguous()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("d,hq,hkv", [(128, 4, 2), (64, 2, 2), (96, 4, 1)])
def test_block_sparse_prefill(dtype, d, hq, hkv):
    _, _, _, sp = _mods()
    lens = [300, 1000, 129, 64, 1]
    q, k, v, cu = make(lens, hq, hkv, d, dtype, seed=d + hq)
    idx, cnt = _random_lists(lens, hq, 0.3, seed=d, empty_rows=(3,))
    o, lse = sp.flash_attn_block_sparse(q.cuda(), k.cuda(), v.cuda(), cu.cuda(), idx.cuda(), cnt.cuda())
    ref, rl = orc.block_sparse_prefill_exact(q, k, v, cu, idx, cnt)
    assert maxabs(o, ref) <= TOL[dtype]
    fin = torch.isfinite(rl)
    assert maxabs(lse.cpu()[fin], rl[fin]) <= 2e-3
    assert bool((lse.cpu()[~fin] == -math.inf).all())
    assert o.cpu()[~fin].abs().max().item() == 0.0 if (~fin).any() else True


def test_block_sparse_full_lists_equal_dense_and_bad_entries_are_ignored():
    """All causal blocks listed == dense causal attention; out-of-range, negative
    and above-diagonal entries are dropped instead of being dereferenced."""
    _, _, fa, sp = _mods()
    lens = [500, 257]
    q, k, v, cu = make(lens, 2, 2, 128, torch.bfloat16, seed=9)
    nqb = 8
    idx = torch.arange(nqb, dtype=torch.int32).expand(2, 2, nqb, nqb).contiguous()
    cnt = (torch.arange(nqb, dtype=torch.int32) + 1).expand(2, 2, nqb).contiguous()
    o_dense = fa.flash_attention(q.cuda(), k.cuda(), v.cuda(), cu.cuda(), causal=True)
    o_blk, _ = sp.flash_attn_block_sparse(q.cuda(), k.cuda(), v.cuda(), cu.cuda(), idx.cuda(), cnt.cuda())
    assert maxabs(o_blk, o_dense) <= 2e-2
    # same lists plus garbage entries appended
    idx2 = torch.full((2, 2, nqb, nqb + 3), -1, dtype=torch.int32)
    idx2[..., :nqb] = idx
    for qb in range(nqb):
        idx2[:, :, qb, qb + 1:qb + 4] = torch.tensor([qb + 1, 100000, -7], dtype=torch.int32)
    cnt2 = cnt + 3
    o_blk2, _ = sp.flash_attn_block_sparse(q.cuda(), k.cuda(), v.cuda(), cu.cuda(), idx2.cuda(), cnt2.cuda())
    assert torch.equal(o_blk2, o_blk)


def test_block_sparse_window_equivalence():
    """A block-aligned window written as block lists gives the window result."""
    _, _, _, sp = _mods()
    lens = [640, 384]
    q, k, v, cu = make(lens, 4, 2, 128, torch.bfloat16, seed=21)
    nqb = 10
    # keys of the query's own block and the previous one: block lists {qb-1, qb}
    idx = torch.full((2, 4, nqb, 2), -1, dtype=torch.int32)
    cnt = torch.zeros(2, 4, nqb, dtype=torch.int32)
    for qb in range(nqb):
        row = [x for x in (qb - 1, qb) if x >= 0]
        idx[:, :, qb, :len(row)] = torch.tensor(row, dtype=torch.int32)
        cnt[:, :, qb] = len(row)
    o, _ = sp.flash_attn_block_sparse(q.cuda(), k.cuda(), v.cuda(), cu.cuda(), idx.cuda(), cnt.cuda())
    ref, _ = orc.block_sparse_prefill_exact(q, k, v, cu, idx, cnt)
    assert maxabs(o, ref) <= 2e-2


def test_cfg4_shape_properties():
    """Config 4 at full size (B=2,H=16,S=16384,D=128, 64x64 blocks): sampled
    (b, h) against fp32 dense-masked math on the device, and determinism."""
    ops, wl, _, sp = _mods()
    w = wl.cfg4("cuda")
    f = lambda: sp.flash_attn_block_sparse(w.q, w.k, w.v, w.cu_seqlens, w.block_idx, w.block_cnt,
                                           max_seqlen=w.max_seqlen)
    o, lse = f()
    o2, _ = f()
    assert torch.equal(o, o2)
    S, nqb = 16384, 256
    for b, h in [(0, 0), (1, 11)]:
        sl = slice(b * S, (b + 1) * S)
        bm = torch.zeros(nqb, nqb, dtype=torch.bool, device="cuda")
        row = w.block_idx[b, h]                                   # [nqb, max_nnz]
        valid = row >= 0
        qq = torch.arange(nqb, device="cuda")[:, None].expand_as(row)
        bm[qq[valid], row[valid].long()] = True
        mask = bm.repeat_interleave(64, 0).repeat_interleave(64, 1)
        mask &= torch.ones(S, S, dtype=torch.bool, device="cuda").tril()
        # row chunks keep the fp32 score matrix small
        for r0 in (0, 8192 - 512, S - 1024):
            rs = slice(r0, r0 + 1024)
            s = (w.q[0, sl, h][rs].float() @ w.k[0, sl, h].float().T) * w.scale
            s = s.masked_fill(~mask[rs], -math.inf)
            ref = torch.softmax(s, -1) @ w.v[0, sl, h].float()
            assert (o[0, sl, h][rs].float() - ref).abs().max().item() <= 2e-2
            assert (lse[0, sl, h][rs] - torch.logsumexp(s, -1)).abs().max().item() <= 1e-3


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("mode", ["dense", "noncausal", "window", "blocks"])
def test_rows_after_a_sequence_never_reach_its_output(dtype, mode):
    """The reference loads every tile with zero padding past the sequence end
    (flash_attn_triton.py:155-165), so whatever follows a sequence in the packed arrays cannot
    reach its output.  Here the second sequence is first real data, then NaN / Inf: the first
    sequence's O and LSE must not change by a bit and must stay finite."""
    ops, _, _, sp = _mods()
    lens = [300, 200]                      # 300 = 2 * 128 + 44: the last KV tile holds 84 foreign rows
    q, k, v, cu = make(lens, 4, 2, 128, dtype, seed=21)

    def run(q, k, v):
        kw = dict(cu_seqlens=cu.cuda(), max_seqlen=300)
        if mode == "window":
            kw.update(sparsity=ops.WINDOW, window_local=100, window_global=64)
        elif mode == "blocks":
            idx, cnt = _random_lists(lens, 4, 0.5, seed=2)
            kw.update(sparsity=ops.BLOCK_LIST, block_idx=idx.cuda(), block_cnt=cnt.cuda())
        elif mode == "noncausal":
            kw.update(causal=False)
        return ops.prefill(q.cuda(), k.cuda(), v.cuda(), **kw)

    o_a, lse_a = run(q, k, v)
    q2, k2, v2 = q.clone(), k.clone(), v.clone()
    q2[0, 300:] = float("nan")
    k2[0, 300:] = float("inf")
    v2[0, 300:] = float("nan")
    o_b, lse_b = run(q2, k2, v2)
    assert torch.isfinite(o_b[0, :300].float()).all() and torch.isfinite(lse_b[0, :300]).all()
    assert torch.equal(o_a[0, :300], o_b[0, :300]) and torch.equal(lse_a[0, :300], lse_b[0, :300])


def test_sequence_longer_than_max_seqlen_is_cut_there():
    """max_seqlen sizes the grid; a longer sequence is attended over its first
    ceil(max_seqlen / 256) * 256 tokens only, and nothing outside is read as a key."""
    ops, _, _, _ = _mods()
    q, k, v, cu = make([700], 2, 2, 64, torch.float16, seed=6)
    o, lse = ops.prefill(q.cuda(), k.cuda(), v.cuda(), cu_seqlens=cu.cuda(), max_seqlen=500, causal=False)
    cu_cut = torch.tensor([0, 512], dtype=torch.int32)
    ref, rl = orc.dense_prefill_exact(q[:, :512], k[:, :512], v[:, :512], cu_cut, causal=False)
    assert maxabs(o[:, :512], ref) <= 5e-3
    assert maxabs(lse[:, :512], rl) <= 2e-3


def test_row_ranges_gqa_half_precision_narrow_heads():
    """The row-range call on a GQA shape with 64-wide heads in fp16, ranges of different sizes."""
    from tritonops_b200 import ops
    B, T, Hq, Hkv, D = 1, 1300, 8, 2, 64
    g = torch.Generator().manual_seed(11)
    q = torch.randn(B, T, Hq, D, generator=g).to(torch.float16).cuda()
    k = torch.randn(B, T, Hkv, D, generator=g).to(torch.float16).cuda()
    v = torch.randn(B, T, Hkv, D, generator=g).to(torch.float16).cuda()
    o_full, lse_full = ops.prefill(q, k, v, causal=True)
    o, lse = torch.zeros_like(o_full), torch.zeros_like(lse_full)
    for r0, r1 in ((0, 1024), (1024, 1280), (1280, 1300)):
        ops.prefill_rows(q, k, v, o, lse, r0, r1, causal=True)
    assert torch.equal(o, o_full) and torch.equal(lse, lse_full)


@pytest.mark.parametrize("causal", [True, False])
def test_row_ranges_equal_the_full_call(causal):
    """b200attn_prefill_fwd_rows: query rows computed range by range equal the full call bit for
    bit, rows outside the range are left alone, and a causal range reads no key at or beyond its
    end (those rows hold NaN until their own range is computed)."""
    from tritonops_b200 import ops
    B, T, Hq, Hkv, D = 2, 1100, 4, 2, 128
    g = torch.Generator().manual_seed(3)
    q = torch.randn(B, T, Hq, D, generator=g).to(torch.bfloat16).cuda()
    k = torch.randn(B, T, Hkv, D, generator=g).to(torch.bfloat16).cuda()
    v = torch.randn(B, T, Hkv, D, generator=g).to(torch.bfloat16).cuda()
    o_full, lse_full = ops.prefill(q, k, v, causal=causal)
    o = torch.full_like(o_full, 7.0)
    lse = torch.full_like(lse_full, 7.0)
    kk, vv = (k.clone(), v.clone()) if causal else (k, v)
    for r0, r1 in ((0, 256), (256, 768), (768, 1100)):
        if causal:                         # keys that have "not arrived yet" are NaN
            kk[:, r1:], vv[:, r1:] = float("nan"), float("nan")
            kk[:, :r1], vv[:, :r1] = k[:, :r1], v[:, :r1]
        ops.prefill_rows(q, kk, vv, o, lse, r0, r1, causal=causal)
        assert torch.equal(o[:, r0:r1], o_full[:, r0:r1]) and torch.equal(lse[:, r0:r1], lse_full[:, r0:r1])
        assert bool((o[:, r1:] == 7.0).all()) and bool((lse[:, r1:] == 7.0).all())
    assert torch.equal(o, o_full) and torch.equal(lse, lse_full)
    with pytest.raises(ValueError):
        ops.prefill_rows(q, k, v, o, lse, 100, 512, causal=causal)
