"""This library against the reference's own Triton kernels, both on the GPU, on identical
seeded inputs: flash_attn_triton_fwd (flash_attn_triton.py:595-658), flash_attention_decoding
(flash_attn_decoding.py:213-336), flash_attention_sparse_decoding
(flash_attn_decoding_sparse.py:222-365) and the window-sparse kernel launched as its shadowed
launcher body does (flash_attn_sparse_attn_triton.py:237-326), the last only for (local, global)
where that kernel equals its own torch oracle.  Tolerance: max-abs <= 2e-2 (bf16), <= 5e-3
(fp16), the same bound the library is held to against fp32 math.

The reference modules are staged under oracle/_ref/ by oracle/make_ref.py; a kernel that the
installed Triton cannot compile or run for this GPU is skipped with the exception text.
Collected after the other parity tests (file name) so a problem in the reference's code cannot
mask them."""
import pytest
import torch

from oracle import ref_triton

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not ref_triton.staged(), reason="reference modules not staged (python -m oracle.make_ref)")]
TOL = {torch.float16: 5e-3, torch.bfloat16: 2e-2}
LOG2E = ref_triton.LOG2E


def maxabs(a, b):
    return (a.float() - b.float()).abs().max().item()


def reference(fn, *args):
    """Run a reference entry point; a compile / launch exception of its Triton code skips the test."""
    try:
        out = fn(*args)
        torch.cuda.synchronize()
        return out
    except Exception as e:  # noqa: BLE001 - whatever Triton raises for this GPU is the skip reason
        pytest.skip(f"reference Triton path did not run here: {type(e).__name__}: {str(e)[:300]}")


def packed(lens, hq, hkv, d, dtype, seed, dist="randn"):
    g = torch.Generator().manual_seed(seed)
    T = sum(lens)
    draw = torch.randn if dist == "randn" else torch.rand
    q, k, v = (draw(1, T, h, d, generator=g).to(dtype).cuda() for h in (hq, hkv, hkv))
    cu = torch.zeros(len(lens) + 1, dtype=torch.int32)
    cu[1:] = torch.cumsum(torch.tensor(lens), 0)
    return q, k, v, cu.cuda()


def cache(lens, hq, hkv, d, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    B, tmax = len(lens), max(lens)
    q = torch.randn(B, hq, d, generator=g).to(dtype).cuda()
    kc = torch.randn(B, tmax, hkv, d, generator=g).to(dtype).cuda()
    vc = torch.randn(B, tmax, hkv, d, generator=g).to(dtype).cuda()
    cu = torch.zeros(B + 1, dtype=torch.int32)
    cu[1:] = torch.cumsum(torch.tensor(lens), 0)
    return q, kc, vc, cu.cuda()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("lens,hq,hkv,d,dist", [
    ([128], 2, 2, 64, "randn"),                 # config 1's shape (the kernel is causal)
    ([77, 128, 300], 2, 2, 96, "rand"),         # the reference test's configs, flash_attn_triton.py:1005-1009
    ([256, 131], 8, 4, 128, "rand"),
    ([512, 33, 400, 1], 4, 1, 64, "rand"),
    ([1000, 2048], 8, 2, 128, "randn")])
def test_dense_prefill_vs_reference_kernel(dtype, lens, hq, hkv, d, dist):
    from tritonops_b200.flash_attn_triton.flash_attn_triton import flash_attn_triton_fwd
    q, k, v, cu = packed(lens, hq, hkv, d, dtype, seed=d + hq, dist=dist)
    ro, rl = reference(ref_triton.dense_prefill, q, k, v, cu)
    o, lse2 = flash_attn_triton_fwd(q, k, v, cu, d ** -0.5 * LOG2E)
    assert maxabs(o, ro) <= TOL[dtype]
    assert maxabs(lse2, rl) <= 5e-3            # base-2 LSE of the prescaled scores, both sides fp32


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("local,glob", [(128, 0), (64, 100), (256, 256), (128, 64), (1, 0), (300, 127)])
def test_window_prefill_vs_reference_kernel(dtype, local, glob):
    from tritonops_b200.flash_attn_triton.flash_attn_sparse_attn_triton import flash_attn_sparse_triton
    assert ref_triton.window_kernel_matches_its_oracle(local, glob)
    q, k, v, cu = packed([700, 129, 2048], 4, 2, 96, dtype, seed=local + glob, dist="rand")
    ro, rl = reference(ref_triton.window_prefill, q, k, v, cu, local, glob)
    o, lse2 = flash_attn_sparse_triton(q, k, v, cu, local, glob)
    assert maxabs(o, ro) <= TOL[dtype]
    assert maxabs(lse2, rl) <= 5e-3


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("lens,hq,hkv,d", [
    ([512, 2049, 8192], 2, 2, 96),              # the reference test's shape, flash_attn_decoding.py:371-437
    ([1, 130, 4000, 0], 32, 8, 128),            # config 3's head layout, with an empty sequence
    ([700, 64], 8, 1, 64)])
def test_decoding_vs_reference_kernels(dtype, lens, hq, hkv, d):
    from tritonops_b200.flash_attn_triton.flash_attn_decoding import flash_attention_decoding
    q, kc, vc, cu = cache(lens, hq, hkv, d, dtype, seed=hq + d)
    ro = reference(ref_triton.decoding, q, kc, vc, cu)
    o = flash_attention_decoding(q, kc, vc, cu)
    # the reference rounds its chunk partials to the input dtype before combining them
    # (flash_attn_decoding.py:121), ours stay fp32: same bound as against fp32 math
    assert maxabs(o, ro) <= TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("glob,local", [(64, 64), (128, 200), (256, 1024), (256, 4096)])
def test_sparse_decoding_vs_reference_kernels(dtype, glob, local):
    from tritonops_b200.flash_attn_triton.flash_attn_decoding_sparse import flash_attention_sparse_decoding
    q, kc, vc, cu = cache([512, 2561, 8192, 137], 24, 4, 128, dtype, seed=glob + local)   # :409-503's shape
    ro = reference(ref_triton.sparse_decoding, q, kc, vc, cu, glob, local)
    o = flash_attention_sparse_decoding(q, kc, vc, cu, glob, local)
    assert maxabs(o, ro) <= TOL[dtype]


@pytest.mark.parametrize("lens,hq,hkv,d", [
    ([256, 131, 77], 8, 4, 128)])                # the reference test's GQA config, flash_attn_triton.py:1005-1009 (the
                                                 # reference autotunes its backward kernels for about a minute per head dim)
def test_backward_vs_reference_kernels(lens, hq, hkv, d):
    """dQ, dK, dV of this library against the reference's three backward kernels and host-side
    GQA sum (flash_attn_triton.py:184-592, :661-813), both under autograd on the GPU, with the
    reference test's own inputs (bf16 U[0,1)) and tolerances (1e-2 on dq / dk widened to 2e-2 for
    bf16 operands, 1e-1 on dv; :1086-1089)."""
    from tritonops_b200.flash_attn_triton.flash_attn_triton import flash_attn_triton
    q, k, v, cu = packed(lens, hq, hkv, d, torch.bfloat16, seed=d, dist="rand")
    do = torch.randn(q.shape, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16).cuda()
    ro, rdq, rdk, rdv = reference(ref_triton.dense_prefill_grads, q, k, v, cu, do)
    qq, kk, vv = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
    o = flash_attn_triton.apply(qq, kk, vv, cu)
    o.backward(do)
    assert maxabs(o, ro) <= 2e-2
    for ours, ref, tol in ((qq.grad, rdq, 2e-2), (kk.grad, rdk, 2e-2), (vv.grad, rdv, 1e-1)):
        bad = (ours.float() - ref.float()).abs() > tol + tol * ref.float().abs()
        assert not bool(bad.any()), f"max err {maxabs(ours, ref):.4g}, {int(bad.sum())} elements off"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("rows,dim", [(64, 128), (300, 1024), (2048, 4096), (37, 4104)])
def test_rmsnorm_forward_vs_reference_kernel(dtype, rows, dim):
    """RMSNorm forward against the reference's Triton kernel (common/rms.py:9-88) through its
    module; the 2048 x 4096 case takes this library's streaming kernel.  (The reference's Triton
    backward multiplies dy of one 128-wide block with the weights of another when dim > 128,
    :197-199, so only dim <= 128 gradients are compared.)"""
    from tritonops_b200.common.rms import RMSNormTriton
    g = torch.Generator().manual_seed(rows + dim)
    x = torch.randn(rows, dim, generator=g).to(dtype).cuda()
    w = (1 + 0.1 * torch.randn(dim, generator=g)).to(dtype).cuda()
    dy = torch.randn(rows, dim, generator=g).to(dtype).cuda()
    ref_mod = reference(ref_triton.rmsnorm_module, dim, 1e-6, w)
    xr = x.clone().requires_grad_(True)
    ry = reference(ref_mod.to(dtype), xr)
    ours = RMSNormTriton(dim, 1e-6).to("cuda").to(dtype)
    with torch.no_grad():
        ours.weight.copy_(w)
    xo = x.clone().requires_grad_(True)
    y = ours(xo)
    rel = {torch.float32: 1e-5, torch.float16: 2e-3, torch.bfloat16: 1.6e-2}[dtype]
    assert maxabs(y, ry) <= rel * max(1.0, ry.float().abs().max().item())
    if dim <= 128:
        reference(lambda: ry.backward(dy))
        y.backward(dy)
        assert maxabs(xo.grad, xr.grad) <= rel * max(1.0, xr.grad.float().abs().max().item())
