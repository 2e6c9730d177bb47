"""GPU parity of RMSNorm forward / backward against the CPU oracle (fp64 math on the same
rounded inputs), the reference's recorded outputs, and the reference's own test recipe
(common/rms.py:430-484: dim 255, eps 0.1, rtol = atol = 1e-2)."""
import os
import sys

import numpy as np
import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
from rms_cases import EPS, SHAPES, build  # noqa: E402
from oracle import rmsnorm_oracle as orc  # noqa: E402

pytestmark = pytest.mark.gpu
G = dict(np.load(os.path.join(HERE, "golden", "golden_rms.npz")))


def test_golden_reference_outputs_and_gradients():
    from tritonops_b200.common.rms import RMSNormTritonFunction
    for name in SHAPES:
        x, w, dy = build(name)
        xc = x.cuda().requires_grad_(True)
        wc = w.cuda().requires_grad_(True)
        y = RMSNormTritonFunction.apply(xc, wc, EPS)
        y.backward(dy.cuda())
        assert np.abs(y.detach().cpu().numpy() - G[f"{name}/y"]).max() <= 1e-5, name
        assert np.abs(y.detach().cpu().numpy() - G[f"{name}/y_triton"]).max() <= 1e-5, name
        assert np.abs(xc.grad.cpu().numpy() - G[f"{name}/dx"]).max() <= 1e-5, name
        assert np.abs(wc.grad.cpu().numpy() - G[f"{name}/dw"]).max() <= 1e-4, name


def test_reference_test_recipe():
    from tritonops_b200.common.rms import RMSNormTriton
    torch.manual_seed(42)
    dim, eps = 255, 1e-1
    m = RMSNormTriton(dim=dim, eps=eps).to("cuda")
    for shape in [(1, dim), (16, 128, dim), (8, 3, 28, dim)]:
        x = torch.randn(*shape, device="cuda", requires_grad=True)
        y = m(x)
        g = torch.randn_like(y)
        m.zero_grad()
        y.backward(g)
        ry, _, rdx, rdw = orc.rmsnorm_exact(x.detach().cpu(), m.weight.detach().cpu(), eps, g.cpu())
        torch.testing.assert_close(y.detach().cpu().double(), ry, rtol=1e-2, atol=1e-2)
        torch.testing.assert_close(x.grad.cpu().double(), rdx, rtol=1e-2, atol=1e-2)
        torch.testing.assert_close(m.weight.grad.cpu().double(), rdw, rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("dtype,wdtype", [(torch.bfloat16, torch.bfloat16), (torch.bfloat16, torch.float32),
                                          (torch.float16, torch.float16), (torch.float32, torch.float32)])
@pytest.mark.parametrize("rows,dim", [(1, 8), (37, 255), (300, 1024), (64, 4096), (700, 4104), (5, 16384), (9, 5000),
                                      # 1024 rows and more of 2 .. 16 KB: the streaming kernels (bulk-copy ring)
                                      (1024, 1024), (3000, 4096), (1100, 4104), (2500, 2048), (1029, 8192)])
def test_forward_backward_against_fp64_math(dtype, wdtype, rows, dim):
    from tritonops_b200 import ops
    g = torch.Generator().manual_seed(rows * 31 + dim)
    x = torch.randn(rows, dim, generator=g).to(dtype)
    w = (1 + 0.1 * torch.randn(dim, generator=g)).to(wdtype)
    dy = torch.randn(rows, dim, generator=g).to(dtype)
    y, rstd = ops.rmsnorm_fwd(x.cuda(), w.cuda(), 1e-6)
    dx, dw = ops.rmsnorm_bwd(dy.cuda(), x.cuda(), w.cuda(), rstd)
    ry, rr, rdx, rdw = orc.rmsnorm_exact(x, w, 1e-6, dy)
    rel = {torch.float32: 2e-6, torch.float16: 1e-3, torch.bfloat16: 8e-3}[dtype]
    assert (y.cpu().double() - ry).abs().max().item() <= rel * max(1.0, ry.abs().max().item())
    assert (rstd.cpu().double() - rr).abs().max().item() <= 2e-6 * rr.abs().max().item()
    assert (dx.cpu().double() - rdx).abs().max().item() <= rel * max(1.0, rdx.abs().max().item())
    wrel = {torch.float32: 2e-5, torch.float16: 1e-3, torch.bfloat16: 8e-3}[wdtype]
    assert (dw.cpu().double() - rdw).abs().max().item() <= wrel * max(1.0, rdw.abs().max().item())
    # deterministic (fixed summation order for dweight)
    dx2, dw2 = ops.rmsnorm_bwd(dy.cuda(), x.cuda(), w.cuda(), rstd)
    assert torch.equal(dw, dw2) and torch.equal(dx, dx2)


def test_streaming_kernels_repeat_and_take_strided_rows():
    """Many back-to-back calls of the streaming kernels on a shape that keeps every SM's ring full
    (bulk copies landing out of order must not confuse the slot barriers), with rows that are a
    strided view; every call must give the first call's bits."""
    from tritonops_b200 import ops
    g = torch.Generator().manual_seed(1)
    big = torch.randn(20000, 2 * 4096, generator=g).to(torch.bfloat16).cuda()
    x, dy = big[:, :4096], big[:, 4096:]                  # row stride 8192 elements
    w = (1 + 0.1 * torch.randn(4096, generator=g)).to(torch.bfloat16).cuda()
    y0, r0 = ops.rmsnorm_fwd(x, w, 1e-6)
    dx0, dw0 = ops.rmsnorm_bwd(dy, x, w, r0)
    ry, rr, rdx, rdw = orc.rmsnorm_exact(x[:64].cpu(), w.cpu(), 1e-6, dy[:64].cpu())
    assert (y0[:64].cpu().double() - ry).abs().max().item() <= 8e-3 * ry.abs().max().item()
    assert (dx0[:64].cpu().double() - rdx).abs().max().item() <= 8e-3 * max(1.0, rdx.abs().max().item())
    outs = [(ops.rmsnorm_fwd(x, w, 1e-6), ops.rmsnorm_bwd(dy, x, w, r0)) for _ in range(40)]
    torch.cuda.synchronize()
    for (y, r), (dx, dw) in outs:
        assert torch.equal(y, y0) and torch.equal(r, r0) and torch.equal(dx, dx0) and torch.equal(dw, dw0)


def test_strided_rows_empty_and_errors():
    from tritonops_b200 import ops
    big = torch.randn(10, 3, 300, device="cuda", dtype=torch.bfloat16)
    x = big[:, 1, :256]                                   # row stride 900, not contiguous
    w = torch.ones(256, device="cuda", dtype=torch.bfloat16)
    y, _ = ops.rmsnorm_fwd(x, w, 1e-6)
    ry, _ = orc.rmsnorm_exact(x.cpu(), w.cpu(), 1e-6)
    assert (y.cpu().double() - ry).abs().max().item() <= 2e-2
    y0, r0 = ops.rmsnorm_fwd(torch.empty(0, 64, device="cuda"), torch.ones(64, device="cuda"), 1e-6)
    assert y0.shape == (0, 64) and r0.numel() == 0
    with pytest.raises(ValueError):
        ops.rmsnorm_fwd(torch.zeros(2, 8, device="cuda", dtype=torch.float64), torch.ones(8, device="cuda"), 1e-6)
    with pytest.raises(ValueError):
        ops.rmsnorm_fwd(torch.zeros(2, 8, device="cuda"), torch.ones(9, device="cuda"), 1e-6)
    with pytest.raises(RuntimeError):
        ops.rmsnorm_fwd(torch.zeros(2, 8), torch.ones(8), 1e-6)
