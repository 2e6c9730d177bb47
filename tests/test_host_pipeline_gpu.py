"""The host-buffer pipeline (copy in / attend / copy out on three streams) returns exactly what
the packed varlen call returns on the same inputs."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_host_pipeline_equals_packed_call():
    from tritonops_b200 import ops
    from tritonops_b200.host import HostPrefill
    lens = [300, 1, 0, 517, 128, 1000]
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    T, Hq, Hkv, D = cu[-1], 8, 2, 128
    g = torch.Generator().manual_seed(0)
    hq = torch.randn(1, T, Hq, D, generator=g).to(torch.bfloat16).pin_memory()
    hk = torch.randn(1, T, Hkv, D, generator=g).to(torch.bfloat16).pin_memory()
    hv = torch.randn(1, T, Hkv, D, generator=g).to(torch.bfloat16).pin_memory()
    ho = torch.zeros(1, T, Hq, D, dtype=torch.bfloat16).pin_memory()
    hl = torch.zeros(1, T, Hq, dtype=torch.float32).pin_memory()
    pipe = HostPrefill("cuda:0")
    scale = D ** -0.5
    for _ in range(3):                      # slots are reused across calls
        pipe.run(hq, hk, hv, cu, ho, hl, scale=scale)
        torch.cuda.synchronize()
    cu_dev = torch.tensor(cu, dtype=torch.int32, device="cuda")
    o, lse = ops.prefill(hq.cuda(), hk.cuda(), hv.cuda(), cu_seqlens=cu_dev, max_seqlen=max(lens), scale=scale)
    assert torch.equal(ho, o.cpu())
    assert torch.equal(hl, lse.cpu())


def test_host_pipeline_rejects_pageable_and_device_tensors():
    from tritonops_b200.host import HostPrefill
    pipe = HostPrefill("cuda:0")
    t = torch.zeros(1, 8, 2, 64, dtype=torch.bfloat16)
    l = torch.zeros(1, 8, 2)
    with pytest.raises(ValueError):
        pipe.run(t, t, t, [0, 8], t, l, scale=1.0)
