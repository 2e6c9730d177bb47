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


def test_host_pipeline_growing_lengths_over_several_calls():
    """Each run() brings longer sequences than the one before, without a synchronisation between
    the calls, so staging buffers are replaced while kernels of the previous call may still be
    reading the old ones; every call must still equal the packed call on its own inputs."""
    from tritonops_b200 import ops
    from tritonops_b200.host import HostPrefill
    Hq, Hkv, D = 4, 2, 64
    pipe = HostPrefill("cuda:0")
    g = torch.Generator().manual_seed(5)
    runs = []
    for lens in ([40, 90], [130, 260, 300], [520, 700, 900, 1100], [1500, 2100]):
        cu = [0]
        for n in lens:
            cu.append(cu[-1] + n)
        T = cu[-1]
        hq = torch.randn(1, T, Hq, D, generator=g).to(torch.float16).pin_memory()
        hk = torch.randn(1, T, Hkv, D, generator=g).to(torch.float16).pin_memory()
        hv = torch.randn(1, T, Hkv, D, generator=g).to(torch.float16).pin_memory()
        ho = torch.zeros(1, T, Hq, D, dtype=torch.float16).pin_memory()
        hl = torch.zeros(1, T, Hq, dtype=torch.float32).pin_memory()
        pipe.run(hq, hk, hv, cu, ho, hl, scale=D ** -0.5)
        runs.append((lens, cu, hq, hk, hv, ho, hl))
    torch.cuda.synchronize()
    for lens, cu, hq, hk, hv, ho, hl in runs:
        cu_dev = torch.tensor(cu, dtype=torch.int32, device="cuda")
        o, lse = ops.prefill(hq.cuda(), hk.cuda(), hv.cuda(), cu_seqlens=cu_dev, max_seqlen=max(lens), scale=D ** -0.5)
        assert torch.equal(ho, o.cpu()) and torch.equal(hl, lse.cpu())


def test_host_pipeline_small_chunks_and_non_causal():
    """256-row chunks (the smallest the row-range call takes) and the non-causal path, which
    cannot be chunked, against the packed call."""
    from tritonops_b200 import ops
    from tritonops_b200.host import HostPrefill
    lens = [700, 256, 1030]
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    T, Hq, Hkv, D = cu[-1], 4, 4, 64
    g = torch.Generator().manual_seed(9)
    hq = torch.randn(1, T, Hq, D, generator=g).to(torch.bfloat16).pin_memory()
    hk = torch.randn(1, T, Hkv, D, generator=g).to(torch.bfloat16).pin_memory()
    hv = torch.randn(1, T, Hkv, D, generator=g).to(torch.bfloat16).pin_memory()
    cu_dev = torch.tensor(cu, dtype=torch.int32, device="cuda")
    pipe = HostPrefill("cuda:0", chunk_tokens=256)
    for causal in (True, False):
        ho = torch.zeros(1, T, Hq, D, dtype=torch.bfloat16).pin_memory()
        hl = torch.zeros(1, T, Hq, dtype=torch.float32).pin_memory()
        pipe.run(hq, hk, hv, cu, ho, hl, scale=D ** -0.5, causal=causal)
        torch.cuda.synchronize()
        o, lse = ops.prefill(hq.cuda(), hk.cuda(), hv.cuda(), cu_seqlens=cu_dev, max_seqlen=max(lens),
                             scale=D ** -0.5, causal=causal)
        assert torch.equal(ho, o.cpu()) and torch.equal(hl, lse.cpu())
    with pytest.raises(ValueError):
        HostPrefill("cuda:0", chunk_tokens=100)
