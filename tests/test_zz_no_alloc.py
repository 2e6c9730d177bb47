"""The allocation-free decoding entry point (b200attn_decode_fwd_noalloc) must
give exactly what b200attn_decode_fwd gives.  It serves hosts that cannot
allocate device memory at request time (all HBM already owned by a KV-cache
pool, latency-critical loops, plugins inside a fixed arena): its split-KV
partials live in a fixed array inside the library instead of a workspace.
Called straight through the C ABI, twice in a row, because consecutive calls
share that array.  Collected last (file name) so a failure here cannot mask
the other tests."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _args(q, kc, vc, o, seqlens, max_seqlen):
    from tritonops_b200._lib import BF16, DecodeArgs
    a = DecodeArgs()
    a.q, a.k_cache, a.v_cache, a.o = q.data_ptr(), kc.data_ptr(), vc.data_ptr(), o.data_ptr()
    a.dtype, a.batch, a.heads_q, a.heads_kv, a.head_dim = BF16, q.shape[0], q.shape[1], kc.shape[2], q.shape[2]
    a.max_seqlen, a.seqlens = max_seqlen, seqlens.data_ptr()
    a.q_stride_b, a.q_stride_h = q.stride(0), q.stride(1)
    a.k_stride_b, a.k_stride_t, a.k_stride_h = kc.stride(0), kc.stride(1), kc.stride(2)
    a.v_stride_b, a.v_stride_t, a.v_stride_h = vc.stride(0), vc.stride(1), vc.stride(2)
    a.o_stride_b, a.o_stride_h = o.stride(0), o.stride(1)
    a.softmax_scale = q.shape[2] ** -0.5
    return a


def _case(B, Hq, Hkv, D, tmax, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, Hq, D, generator=g).to(torch.bfloat16).cuda()
    kc = torch.randn(B, tmax, Hkv, D, generator=g).to(torch.bfloat16).cuda()
    vc = torch.randn(B, tmax, Hkv, D, generator=g).to(torch.bfloat16).cuda()
    lens = torch.randint(1, tmax + 1, (B,), generator=g).to(torch.int32)
    lens[0] = tmax
    return q, kc, vc, lens.cuda()


def test_noalloc_matches_workspace_entry_point_twice():
    from tritonops_b200 import _lib
    L = _lib.lib()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    # two different problems back to back: the second reuses the array the first dirtied
    for B, Hq, Hkv, D, tmax, seed in [(6, 16, 4, 128, 3000, 1), (3, 8, 8, 64, 700, 2)]:
        q, kc, vc, lens = _case(B, Hq, Hkv, D, tmax, seed)
        o_ws, o_na = torch.empty_like(q), torch.full_like(q, float("nan"))
        a = _args(q, kc, vc, o_ws, lens, tmax)
        need = L.b200attn_decode_workspace_bytes(C.byref(a))
        ws = torch.empty(need, dtype=torch.uint8, device="cuda")
        a.workspace, a.workspace_bytes = ws.data_ptr(), need
        assert L.b200attn_decode_fwd(C.byref(a), stream) == 0
        b = _args(q, kc, vc, o_na, lens, tmax)                      # no workspace given
        before = torch.cuda.memory_allocated()
        assert L.b200attn_decode_fwd_noalloc(C.byref(b), stream) == 0
        assert L.b200attn_decode_fwd_noalloc(C.byref(b), stream) == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        # same kernels on the same inputs: identical bits, well inside the bf16 tolerance of 2e-2
        assert torch.equal(o_na, o_ws)
        # ... and both are the right answer: fp32 softmax(q K^T scale) V on the same rounded inputs
        from oracle import attention_oracle as orc
        ref = orc.decoding_exact(q.cpu(), kc.cpu(), vc.cpu(), lens.cpu().tolist())
        assert (o_na.float().cpu() - ref).abs().max().item() <= 2e-2


def test_noalloc_rejects_oversized_problem():
    from tritonops_b200 import _lib
    L = _lib.lib()
    q, kc, vc, lens = _case(2, 8, 2, 128, 64, 3)
    a = _args(q, kc, vc, torch.empty_like(q), lens, 64)
    a.batch, a.max_seqlen = 4096, 1 << 20                            # sizes only; rejected before any launch
    assert L.b200attn_decode_workspace_bytes(C.byref(a)) > _lib.NOALLOC_SCRATCH_BYTES
    st = L.b200attn_decode_fwd_noalloc(C.byref(a), None)
    assert st == -11 and b"limit" in L.b200attn_strerror(st)
