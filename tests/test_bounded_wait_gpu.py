"""Failure detection without a GPU fault: a device-side wait on a barrier that nothing ever
completes runs out of its cycle budget, the kernel returns normally with the status word set,
and the context stays usable.  Also the debug mode that checks the prefill kernels' status word."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_wait_gives_up_and_context_survives():
    from tritonops_b200 import ops
    status, waited = ops.selftest_bounded_wait(budget_cycles=2_000_000)      # about 1 ms
    assert status == 3            # bit 0: the waiter gave up; bit 1: a later wait returned at once
    assert 2_000_000 <= waited <= 40_000_000
    # the GPU context is intact: real work still runs and is correct
    q = torch.randn(1, 256, 2, 64, device="cuda", dtype=torch.bfloat16)
    o, _ = ops.prefill(q, q, q, causal=True)
    torch.cuda.synchronize()
    assert torch.isfinite(o.float()).all()
    status2, _ = ops.selftest_bounded_wait(budget_cycles=500_000)
    assert status2 == 3


def test_probe_refuses_long_budgets():
    from tritonops_b200 import ops
    with pytest.raises(ValueError):
        ops.selftest_bounded_wait(budget_cycles=10**10)


def test_debug_status_mode_checks_the_status_word():
    """With B200ATTN_DEBUG_STATUS=1 every prefill call hands the kernels a status word and checks
    it after a synchronisation; a healthy run leaves it zero."""
    code = (
        "import torch\n"
        "from tritonops_b200 import ops\n"
        "assert ops.DEBUG_STATUS\n"
        "q = torch.randn(1, 300, 4, 128, device='cuda', dtype=torch.bfloat16)\n"
        "o, lse = ops.prefill(q, q, q, causal=True)\n"
        "dq, dk, dv = ops.prefill_bwd(q, q, q, o, torch.ones_like(o), lse, causal=True)\n"
        "assert int(ops._status_word(q.device).item()) == 0\n"
        "print('ok')\n")
    env = dict(os.environ, B200ATTN_DEBUG_STATUS="1", PYTHONPATH=ROOT)
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0 and "ok" in out.stdout, out.stderr[-2000:]
