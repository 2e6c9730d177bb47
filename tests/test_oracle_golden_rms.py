"""The RMSNorm oracle against outputs recorded from the reference (torch module and its
Triton forward kernel under the interpreter)."""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
from rms_cases import EPS, SHAPES, build  # noqa: E402
from oracle import rmsnorm_oracle as orc  # noqa: E402

G = dict(np.load(os.path.join(HERE, "golden", "golden_rms.npz")))


def test_refpath_is_bit_exact_against_the_reference_module():
    for name in SHAPES:
        x, w, _ = build(name)
        assert np.array_equal(orc.rmsnorm_refpath(x, w, EPS).numpy(), G[f"{name}/y"]), name


def test_exact_math_matches_reference_outputs_and_gradients():
    for name in SHAPES:
        x, w, dy = build(name)
        y, _, dx, dw = orc.rmsnorm_exact(x, w, EPS, dy)
        assert np.abs(y.numpy() - G[f"{name}/y"]).max() <= 1e-5, name
        assert np.abs(y.numpy() - G[f"{name}/y_triton"]).max() <= 1e-5, name
        assert np.abs(dx.numpy() - G[f"{name}/dx"]).max() <= 1e-5, name
        assert np.abs(dw.numpy() - G[f"{name}/dw"]).max() <= 1e-4, name
