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
