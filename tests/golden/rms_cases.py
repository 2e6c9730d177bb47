"""Seeded inputs of the RMSNorm fixtures (shared by make_golden_rms.py and the tests)."""
import torch

EPS = 1e-1   # the reference's own test value (common/rms.py:436)
SHAPES = {"rows1": (1, 255), "seq": (2, 16, 255), "image": (2, 3, 5, 255), "even": (3, 7, 512)}


def build(name):
    shape = SHAPES[name]
    g = torch.Generator().manual_seed(42 + len(shape) + shape[-1])
    x = torch.randn(*shape, generator=g)
    w = 1.0 + 0.1 * torch.randn(shape[-1], generator=g)
    dy = torch.randn(*shape, generator=g)
    return x, w, dy
