"""KV-cache glue kernels: bit-exact against the Python copy loops of the
reference's decoding tests (flash_attn_decoding.py:404-425), restated in
tests/golden/cases.py:packed_to_cache."""
import pytest
import torch

from cases import packed_to_cache

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("lens,H,D", [([200, 515, 70], 2, 96), ([0, 1, 33], 4, 128), ([1000], 8, 64)])
def test_pack_to_cache_bit_exact(dtype, lens, H, D):
    from tritonops_b200 import ops
    g = torch.Generator().manual_seed(1)
    T = sum(lens)
    k = torch.randn(1, max(T, 1), H, D, generator=g).to(dtype)[:, :T]
    cu = torch.zeros(len(lens) + 1, dtype=torch.int32)
    cu[1:] = torch.cumsum(torch.tensor(lens), 0)
    ref = packed_to_cache(k, cu)
    cap = ref.shape[1]
    out = ops.pack_kv_cache(k.cuda(), cu.cuda(), cap)
    assert torch.equal(out.cpu(), ref)
    # larger capacity, no zero fill: the valid rows still match, the rest is untouched
    pre = torch.full((len(lens), cap + 7, H, D), 3.0, dtype=dtype).cuda()
    out2 = ops.pack_kv_cache(k.cuda(), cu.cuda(), cap + 7, out=pre.clone(), zero_pad=False)
    for b, n in enumerate(lens):
        assert torch.equal(out2[b, :n].cpu(), ref[b, :n])
        assert torch.equal(out2[b, n:], pre[b, n:])


def test_append_then_decode_equals_rebuilt_cache():
    """Append one token per sequence, then decoding over the grown cache equals
    decoding over a cache rebuilt from scratch."""
    from tritonops_b200 import ops
    g = torch.Generator().manual_seed(2)
    lens = [300, 17, 511, 0]
    B, H, D, cap = len(lens), 2, 128, 512
    kc = torch.randn(B, cap, H, D, generator=g).to(torch.bfloat16).cuda()
    vc = torch.randn(B, cap, H, D, generator=g).to(torch.bfloat16).cuda()
    nk = torch.randn(B, H, D, generator=g).to(torch.bfloat16).cuda()
    nv = torch.randn(B, H, D, generator=g).to(torch.bfloat16).cuda()
    q = torch.randn(B, 4, D, generator=g).to(torch.bfloat16).cuda()
    sl = torch.tensor(lens, dtype=torch.int32).cuda()
    kc2, vc2 = kc.clone(), vc.clone()
    for b, n in enumerate(lens):
        kc2[b, n], vc2[b, n] = nk[b], nv[b]
    ops.append_kv(kc, vc, nk, nv, sl)
    assert torch.equal(kc, kc2) and torch.equal(vc, vc2)
    o1 = ops.decode(q, kc, vc, seqlens=sl + 1)
    o2 = ops.decode(q, kc2, vc2, seqlens=sl + 1)
    assert torch.equal(o1, o2)
    # a sequence already at capacity is skipped
    full = torch.tensor([cap, 1, 2, 3], dtype=torch.int32).cuda()
    before = kc.clone()
    ops.append_kv(kc, vc, nk, nv, full)
    assert torch.equal(kc[0], before[0])
