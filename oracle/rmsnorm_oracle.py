"""CPU oracle for RMSNorm.  TEST INFRASTRUCTURE ONLY (imported by tests/ and smoke checks,
never by the package).

Parity pin: tests/test_oracle_golden_rms.py checks both functions against
tests/golden/golden_rms.npz, which tests/golden/make_golden_rms.py recorded from the
reference itself (its torch module's outputs and gradients, and its Triton forward
kernel run by the Triton interpreter)."""
import torch


def rmsnorm_refpath(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """The reference's torch module restated (common/rms.py:408-427): mean of squares,
    sqrt(mean + eps), divide, scale -- all in the input dtype."""
    mean_square = torch.mean(x ** 2, dim=-1, keepdim=True)
    rms = torch.sqrt(mean_square + eps)
    return weight * (x / rms)


def rmsnorm_exact(x, weight, eps, dy=None):
    """fp64 math from the given (already rounded) inputs: y, rstd and, with dy, (dx, dw).
    y = x r w with r = (mean(x^2) + eps)^-1/2 (common/rms.py:68,80);
    dx = r (w dy - x r^2 mean_d(dy w x)), dw = sum_rows dy x r (:197-217 with the block bug removed)."""
    x64, w64 = x.double(), weight.double()
    D = x.shape[-1]
    r = torch.rsqrt((x64 * x64).mean(dim=-1, keepdim=True) + eps)
    y = x64 * r * w64
    if dy is None:
        return y, r.squeeze(-1)
    g = dy.double()
    c = (g * w64 * x64).sum(dim=-1, keepdim=True)
    dx = r * (w64 * g - x64 * (r * r) * c / D)
    dw = (g * x64 * r).reshape(-1, D).sum(dim=0)
    return y, r.squeeze(-1), dx, dw
