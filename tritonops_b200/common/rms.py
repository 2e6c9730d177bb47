"""Drop-in for the reference's common/rms.py: same class names and call signatures
(RMSNormTritonFunction.apply(x, weight, eps), RMSNormTriton(dim, eps)), with the
arithmetic in libb200attn.so (b200attn_rmsnorm_fwd / _bwd).  CUDA tensors only."""
import torch
import torch.nn as nn
from torch.autograd import Function

from .. import ops


class RMSNormTritonFunction(Function):
    """Mirrors RMSNormTritonFunction of the reference (common/rms.py:221-355)."""

    @staticmethod
    def forward(ctx, x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
        assert x.shape[-1] == weight.shape[0], f"Expected weight dim {x.shape[-1]}, got {weight.shape[0]}"
        y, rstd = ops.rmsnorm_fwd(x, weight, eps)
        ctx.save_for_backward(x, weight, rstd)
        return y

    @staticmethod
    def backward(ctx, grad_output: torch.Tensor):
        x, weight, rstd = ctx.saved_tensors
        dx, dw = ops.rmsnorm_bwd(grad_output, x, weight, rstd)
        return dx, dw, None


class RMSNormTriton(nn.Module):
    """Mirrors RMSNormTriton of the reference (common/rms.py:358-382)."""

    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return RMSNormTritonFunction.apply(x, self.weight, self.eps)
