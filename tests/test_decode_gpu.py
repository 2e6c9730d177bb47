"""GPU parity of the decoding path (dense, window-sparse, block-list) against the
CPU oracle, the reference's recorded outputs and size-independent properties.
Tolerances are the stated ones: max-abs <= 5e-3 (fp16), <= 2e-2 (bf16) against
fp32 math on the same rounded inputs."""
import pytest
import torch

from cases import build, load_golden
from oracle import attention_oracle as orc

pytestmark = pytest.mark.gpu
TOL = {torch.float16: 5e-3, torch.bfloat16: 2e-2}


def _mods():
    from tritonops_b200 import ops, workloads
    from tritonops_b200.flash_attn_triton import flash_attn_decoding as dec
    from tritonops_b200.flash_attn_triton import flash_attn_decoding_sparse as dsp
    return ops, workloads, dec, dsp


def maxabs(a, b):
    return (a.float().cpu() - b.float().cpu()).abs().max().item()


def make(B, Hq, Hkv, D, lens, dtype, seed=0, tmax=None, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    tmax = tmax or max(max(lens), 1)
    q = (torch.randn(B, Hq, D, generator=g) * scale).to(dtype)
    kc = (torch.randn(B, tmax, Hkv, D, generator=g) * scale).to(dtype)
    vc = torch.randn(B, tmax, Hkv, D, generator=g).to(dtype)
    cu = torch.zeros(B + 1, dtype=torch.int32)
    cu[1:] = torch.cumsum(torch.tensor(lens), 0)
    return q, kc, vc, cu


def test_golden_reference_kernel_outputs():
    """Same inputs the reference's Triton decoding kernels were run on."""
    _, _, dec, dsp = _mods()
    gk = load_golden("golden_triton.npz")
    i = build("decode_gqa")
    o = dec.flash_attention_decoding(i["q"].cuda(), i["kc"].cuda(), i["vc"].cuda(), i["cu"].cuda())
    assert maxabs(o, gk["decode_gqa"]["o"]) <= 5e-3
    i = build("sparse_decode_gqa")
    for G, L in [(64, 64), (128, 200), (256, 1024)]:
        o = dsp.flash_attention_sparse_decoding(i["q"].cuda(), i["kc"].cuda(), i["vc"].cuda(),
                                                i["cu"].cuda(), G, L)
        assert maxabs(o, gk["sparse_decode_gqa"][f"o_G{G}_L{L}"]) <= 5e-3
        assert o[2].abs().max().item() == 0.0


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("D", [32, 64, 96, 128])
@pytest.mark.parametrize("Hq,Hkv", [(2, 2), (4, 1), (8, 2), (32, 8), (16, 1), (12, 1)])
def test_dense_decode_sweep(dtype, D, Hq, Hkv):
    _, _, dec, _ = _mods()
    lens = [0, 1, 2, 4, 15, 16, 17, 63, 64, 65, 511, 512, 513, 1300]
    q, kc, vc, cu = make(len(lens), Hq, Hkv, D, lens, dtype, seed=D + Hq)
    o = dec.flash_attention_decoding(q.cuda(), kc.cuda(), vc.cuda(), cu.cuda())
    ref = orc.decoding_exact(q, kc, vc, lens)
    assert maxabs(o, ref) <= TOL[dtype]
    assert o[0].abs().max().item() == 0.0


def test_reference_test_shape():
    """flash_attn_decoding.py:371-437: Hq=Hkv=2, D=96, lens 512/2049/8192, fp16."""
    _, _, dec, _ = _mods()
    lens = [512, 2049, 8192]
    q, kc, vc, cu = make(3, 2, 2, 96, lens, torch.float16, seed=42)
    o = dec.flash_attention_decoding(q.cuda(), kc.cuda(), vc.cuda(), cu.cuda())
    assert maxabs(o, orc.decoding_exact(q, kc, vc, lens)) <= 5e-3


def test_seqlens_form_scale_and_chunk():
    ops, _, _, _ = _mods()
    lens = [700, 33, 2048, 1]
    q, kc, vc, cu = make(4, 8, 2, 128, lens, torch.bfloat16, seed=3)
    ref = orc.decoding_exact(q, kc, vc, lens, scale=0.3)
    sl = torch.tensor(lens, dtype=torch.int32).cuda()
    outs = [ops.decode(q.cuda(), kc.cuda(), vc.cuda(), seqlens=sl, scale=0.3, chunk=c)
            for c in (0, 64, 128, 1024)]
    for o in outs:
        assert maxabs(o, ref) <= 2e-2
    # bigger chunks than any length: single-chunk path
    assert maxabs(outs[0], outs[3]) <= 2e-2


def test_long_sequences_with_long_chunks():
    """Few sequences, many keys: the library picks chunks of up to 8192 keys; every explicit
    chunk size gives the same answer as fp32 math."""
    ops, _, _, _ = _mods()
    lens = [20000, 8193]
    q, kc, vc, cu = make(2, 8, 2, 128, lens, torch.bfloat16, seed=9, tmax=20000)
    ref = orc.decoding_exact(q, kc, vc, lens)
    sl = torch.tensor(lens, dtype=torch.int32).cuda()
    for c in (0, 2048, 4096, 8192):
        o = ops.decode(q.cuda(), kc.cuda(), vc.cuda(), seqlens=sl, chunk=c)
        assert maxabs(o, ref) <= 2e-2, c


def test_strided_cache_views():
    """Arbitrary batch/token/head strides are honoured (the reference passes all
    strides through, flash_attn_decoding.py:280-297)."""
    ops, _, _, _ = _mods()
    lens = [100, 257]
    g = torch.Generator().manual_seed(9)
    big_k = torch.randn(2, 300, 6, 128, generator=g).to(torch.float16).cuda()
    big_v = torch.randn(2, 300, 6, 128, generator=g).to(torch.float16).cuda()
    q = torch.randn(2, 8, 128, generator=g).to(torch.float16).cuda()
    kc, vc = big_k[:, :, 1:5:2], big_v[:, :, 1:5:2]   # Hkv = 2, head stride 256
    cu = torch.tensor([0, 100, 357], dtype=torch.int32).cuda()
    o = ops.decode(q, kc, vc, cu_seqlens=cu)
    ref = orc.decoding_exact(q.cpu(), kc.cpu(), vc.cpu(), lens)
    assert maxabs(o, ref) <= 5e-3


@pytest.mark.parametrize("scale", [10.0, 100.0])
def test_large_magnitude_inputs_stay_finite(scale):
    """Input-scale robustness sweep of flash_attn_decoding_sparse.py:506-630."""
    _, _, dec, dsp = _mods()
    lens = [0, 1, 2, 4, 300, 1000]
    q, kc, vc, cu = make(len(lens), 8, 2, 64, lens, torch.float16, seed=1, scale=scale)
    for o in (dec.flash_attention_decoding(q.cuda(), kc.cuda(), vc.cuda(), cu.cuda()),
              dsp.flash_attention_sparse_decoding(q.cuda(), kc.cuda(), vc.cuda(), cu.cuda(), 64, 128)):
        assert torch.isfinite(o).all()
        assert o[0].abs().max().item() == 0.0
        assert o[1:].abs().max().item() > 0.0


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("G,L", [(64, 64), (64, 1024), (128, 128), (128, 200), (256, 1024), (256, 1)])
def test_window_decode(dtype, G, L):
    _, _, _, dsp = _mods()
    lens = [0, 1, 63, 64, 65, 128, 129, 300, 700, 1500, 2561]
    q, kc, vc, cu = make(len(lens), 8, 2, 128, lens, dtype, seed=G + L)
    o = dsp.flash_attention_sparse_decoding(q.cuda(), kc.cuda(), vc.cuda(), cu.cuda(), G, L)
    ref = orc.window_decoding_exact(q, kc, vc, lens, glob=G, local=L)
    assert maxabs(o, ref) <= TOL[dtype]


def test_window_decode_rejects_bad_global_window():
    _, _, _, dsp = _mods()
    q, kc, vc, cu = make(1, 2, 2, 64, [10], torch.float16)
    with pytest.raises(AssertionError):
        dsp.flash_attention_sparse_decoding(q.cuda(), kc.cuda(), vc.cuda(), cu.cuda(), 512, 512)


@pytest.mark.parametrize("Hq,Hkv", [(4, 4), (8, 2)])
def test_block_list_decode(Hq, Hkv):
    _, wl, _, dsp = _mods()
    lens = [4096, 4000, 1000, 64]
    q, kc, vc, cu = make(4, Hq, Hkv, 128, lens, torch.bfloat16, seed=5, tmax=4096)
    idx = wl.topk_block_lists(4, Hkv, 64, 16, seed=4)
    idx[3, :, 5:] = -1                                   # ragged list through padding
    cnt = torch.tensor([[16] * Hkv, [16] * Hkv, [16] * Hkv, [5] * Hkv], dtype=torch.int32)
    ref = orc.block_sparse_decoding_exact(q, kc, vc, lens, idx, cnt)
    for bc in (cnt.cuda(), None):
        o = dsp.flash_attention_block_sparse_decoding(q.cuda(), kc.cuda(), vc.cuda(), cu.cuda(),
                                                      idx.cuda(), bc)
        assert maxabs(o, ref) <= 2e-2


def test_cfg3_shape_properties():
    """Full config-3 size: (i) rows checked against the oracle, (ii) chunking
    invariance, (iii) a permutation of the batch permutes the output."""
    ops, wl, _, _ = _mods()
    w = wl.cfg3("cuda")
    o = ops.decode(w.q, w.k_cache, w.v_cache, cu_seqlens=w.cu_seqlens, max_seqlen=w.max_seqlen)
    rows = [0, 17, 63]
    ref = orc.decoding_exact(w.q[rows].cpu(), w.k_cache[rows].cpu(), w.v_cache[rows].cpu(),
                             w.seqlens[rows].cpu().tolist())
    assert maxabs(o[rows], ref) <= 2e-2
    o2 = ops.decode(w.q, w.k_cache, w.v_cache, seqlens=w.seqlens, chunk=2048)
    assert maxabs(o, o2) <= 2e-2
    perm = torch.randperm(64, generator=torch.Generator().manual_seed(0)).cuda()
    o3 = ops.decode(w.q[perm], w.k_cache[perm], w.v_cache[perm], seqlens=w.seqlens[perm])
    assert torch.equal(o3, o[perm])


def test_error_codes():
    ops, _, _, _ = _mods()
    q, kc, vc, cu = make(2, 4, 3, 64, [5, 5], torch.float16)
    with pytest.raises(ValueError):
        ops.decode(q.cuda(), kc.cuda(), vc.cuda(), cu_seqlens=cu.cuda())        # 4 % 3 != 0
    q, kc, vc, cu = make(2, 4, 2, 48, [5, 5], torch.float16)
    with pytest.raises(ValueError):
        ops.decode(q.cuda(), kc.cuda(), vc.cuda(), cu_seqlens=cu.cuda())        # head_dim 48
    with pytest.raises(RuntimeError):
        ops.decode(q, kc, vc, cu_seqlens=cu)                                    # CPU tensors


def test_cfg5_shape_properties():
    """Full config-5 size (B=32, H=32 MHA, D=128, 32768 keys in 512 blocks of 64, 64 blocks
    listed per (b, h)): sampled (b, h) against fp32 math over the 64 gathered blocks on the
    device, determinism, and a permutation of the batch permutes the output."""
    ops, wl, _, _ = _mods()
    w = wl.cfg5("cuda")
    f = lambda q, kc, vc, sl, idx: ops.decode(q, kc, vc, seqlens=sl, sparsity=ops.BLOCK_LIST,
                                              block_idx=idx, block_size=64)
    o = f(w.q, w.k_cache, w.v_cache, w.seqlens, w.block_idx)
    assert torch.equal(o, f(w.q, w.k_cache, w.v_cache, w.seqlens, w.block_idx))
    assert bool((w.block_idx[..., -1] == 511).all())           # the newest block is always listed
    assert bool((w.block_idx[..., 1:] > w.block_idx[..., :-1]).all())
    for b, h in [(0, 0), (5, 17), (13, 2), (31, 31), (20, 9), (8, 30)]:
        rows = (w.block_idx[b, h].long()[:, None] * 64 + torch.arange(64, device="cuda")[None, :]).reshape(-1)
        kk, vv = w.k_cache[b, rows, h].float(), w.v_cache[b, rows, h].float()
        p = torch.softmax((kk @ w.q[b, h].float()) * w.scale, 0)
        assert (o[b, h].float() - p @ vv).abs().max().item() <= 2e-2
    # batch permutation on a slice (a permuted copy of the whole 17 GB cache is not needed for
    # the property): sequences 3, 1, 2, 0 of the first four
    perm = torch.tensor([3, 1, 2, 0], device="cuda")
    o4 = f(w.q[perm], w.k_cache[:4][perm], w.v_cache[:4][perm], w.seqlens[perm], w.block_idx[perm])
    assert torch.equal(o4, o[perm])


def test_length_beyond_max_seqlen_is_cut_there():
    """A length larger than max_seqlen (which sizes the grid and the scratch) is treated as
    max_seqlen: the truncated result, and nothing is read or written out of bounds (a canary
    row behind the output stays intact)."""
    ops, _, _, _ = _mods()
    lens = [300, 200]
    q, kc, vc, _ = make(2, 8, 2, 128, lens, torch.bfloat16, seed=11, tmax=320)
    sl = torch.tensor([300, 200], dtype=torch.int32).cuda()
    for chunk in (0, 64):
        o = ops.decode(q.cuda(), kc.cuda(), vc.cuda(), seqlens=sl, max_seqlen=256, chunk=chunk)
        ref = orc.decoding_exact(q, kc, vc, [256, 200])
        assert maxabs(o, ref) <= 2e-2


def test_debug_status_mode_covers_decoding(monkeypatch):
    """With the status word switched on, decoding and paged decoding pass one, find it clear
    after a synchronisation and return the same bits."""
    ops, _, _, _ = _mods()
    lens = [700, 33]
    q, kc, vc, _ = make(2, 8, 2, 128, lens, torch.bfloat16, seed=4, tmax=704)
    sl = torch.tensor(lens, dtype=torch.int32).cuda()
    o0 = ops.decode(q.cuda(), kc.cuda(), vc.cuda(), seqlens=sl)
    monkeypatch.setattr(ops, "DEBUG_STATUS", True)
    o1 = ops.decode(q.cuda(), kc.cuda(), vc.cuda(), seqlens=sl)
    assert torch.equal(o0, o1)
    assert int(ops._status_word(torch.device("cuda", 0)).item()) == 0
    table = torch.arange(2 * 11, dtype=torch.int32).view(2, 11).cuda()
    o2 = ops.paged_decode(q.cuda(), kc.cuda().view(22, 64, 2, 128), vc.cuda().view(22, 64, 2, 128), table, sl)
    assert torch.equal(o0, o2)
