"""Generate tests/golden/golden_rms.npz by running the REFERENCE's RMSNorm.

    REFERENCE_ROOT=<checkout of rookie-joe/TritonOps> python tests/golden/make_golden_rms.py

Recorded per case of rms_cases.py: the output and the gradients of the reference's
torch module (common/rms.py:385-427) on CPU fp32 tensors, and the output of its
Triton forward kernel (:9-88) executed by Triton's CPU interpreter.  The Triton
backward kernel is not recorded: for dim > 128 it multiplies dy of one 128-wide
block with the weights of another (:197-199 use the x-block's b_w inside the loop
over dy blocks), so it does not equal the torch module there.
"""
import os
import subprocess
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from rms_cases import EPS, SHAPES, build  # noqa: E402

REF = os.environ.get("REFERENCE_ROOT")
if not REF or not os.path.isdir(REF):
    raise SystemExit("set REFERENCE_ROOT to a checkout of the reference (rookie-joe/TritonOps)")


def torch_part():
    sys.path.insert(0, REF)
    from common.rms import RMSNormTorch
    out = {}
    for name in SHAPES:
        x, w, dy = build(name)
        m = RMSNormTorch(x.shape[-1], EPS)
        with torch.no_grad():
            m.weight.copy_(w)
        xr = x.clone().requires_grad_(True)
        y = m(xr)
        y.backward(dy)
        out[f"{name}/y"] = y.detach().numpy()
        out[f"{name}/dx"] = xr.grad.numpy()
        out[f"{name}/dw"] = m.weight.grad.numpy()
    return out


def triton_part():
    os.environ["TRITON_INTERPRET"] = "1"
    sys.path.insert(0, REF)
    from common.rms import RMSNormTritonFunction
    out = {}
    for name in SHAPES:
        x, w, _ = build(name)
        y = RMSNormTritonFunction.apply(x, w, EPS)
        out[f"{name}/y_triton"] = y.numpy()
    return out


if __name__ == "__main__":
    if len(sys.argv) > 1 and sys.argv[1] == "--triton":
        np.savez_compressed(os.path.join(HERE, "_rms_triton_tmp.npz"), **triton_part())
        sys.exit(0)
    store = torch_part()
    # the interpreter has to be switched on before triton is imported: own process
    subprocess.check_call([sys.executable, os.path.abspath(__file__), "--triton"])
    tmp = os.path.join(HERE, "_rms_triton_tmp.npz")
    store.update(dict(np.load(tmp)))
    os.remove(tmp)
    np.savez_compressed(os.path.join(HERE, "golden_rms.npz"), **store)
    print("wrote golden_rms.npz", os.path.getsize(os.path.join(HERE, "golden_rms.npz")), "bytes", sorted(store)[:6])
