"""The reference's Triton attention path (rookie-joe/TritonOps, flash_attn_triton/*.py), loaded
unmodified from oracle/_ref/ (staged by oracle/make_ref.py) and driven through its own entry
points on a CUDA device.  Test infrastructure: used by the GPU parity tests and by bench.py's
reference-on-GPU baseline, never by tritonops_b200/.

The window-sparse prefill has no callable launcher in the reference: its body
(flash_attn_sparse_attn_triton.py:237-326) is defined under a name that the torch oracle of
the same name (:391) then overwrites, and the only call site names a function that does not
exist (:480).  `window_prefill` below therefore launches the reference's kernel object with
the argument list of that body."""
import importlib
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
LOG2E = 1.4426950408889634
_mods = None


def staged() -> bool:
    return os.path.exists(os.path.join(REF_DIR, "flash_attn_triton", "flash_attn_triton.py"))


def load():
    """(dense, decoding, sparse_decoding, sparse_prefill) reference modules; raises when they are
    not staged or cannot be imported (the dense module imports the flash_attn package at its top)."""
    global _mods
    if _mods is None:
        if not staged():
            raise FileNotFoundError("reference modules are not staged under oracle/_ref (python -m oracle.make_ref)")
        if REF_DIR not in sys.path:
            sys.path.insert(0, REF_DIR)
        names = ("flash_attn_triton", "flash_attn_decoding", "flash_attn_decoding_sparse", "flash_attn_sparse_attn_triton")
        _mods = tuple(importlib.import_module("flash_attn_triton." + n) for n in names)
    return _mods


def dense_prefill(q, k, v, cu, scale=None):
    """flash_attn_triton_fwd (flash_attn_triton.py:595-658): (o, lse2); causal, sm_scale carries log2(e)."""
    dense = load()[0]
    return dense.flash_attn_triton_fwd(q, k, v, cu, (scale or q.shape[-1] ** -0.5) * LOG2E)


def dense_prefill_kernel_only(q, k, v, cu, o, lse, max_len, scale=None):
    """The same launch with outputs and the grid size supplied: no allocation, memset or host sync."""
    import triton
    dense = load()[0]
    _, T, hq, d = q.shape
    hkv, dv = v.shape[2], v.shape[3]
    grid = (cu.numel() - 1) * hq, triton.cdiv(max_len, 128), triton.cdiv(dv, 128)
    dense.flash_attn_fwd_kernel[grid](
        q, k, v, o, cu, lse, q.stride(1), q.stride(2), q.stride(3), k.stride(1), k.stride(2), k.stride(3),
        v.stride(1), v.stride(2), v.stride(3), o.stride(1), o.stride(2), o.stride(3), lse.stride(1), lse.stride(2),
        BLOCK_SIZE_QD=triton.next_power_of_2(d), HEAD_DIM_Q=d, HEAD_DIM_V=dv, BLOCK_SIZE_N=128, BLOCK_SIZE_KN=128,
        BLOCK_SIZE_D=128, NUM_HEADS=hq, GQA_RATIO=hq // hkv, sm_scale=(scale or d ** -0.5) * LOG2E)


def window_prefill(q, k, v, cu, local, glob, scale=None):
    """The window-sparse kernel (flash_attn_sparse_attn_triton.py:47-234) launched as its shadowed
    launcher body does (:237-326): (o, lse2).  The kernel equals its own torch oracle only when
    glob < 128 or local >= 128 * (glob // 128) (its second loop is skipped for query tiles that
    end inside the global window, :179)."""
    import torch
    import triton
    sp = load()[3]
    _, T, hq, d = q.shape
    hkv, dv = v.shape[2], v.shape[3]
    o = torch.zeros(1, T, hq, d, device=q.device, dtype=q.dtype)
    lse = torch.zeros(1, T, hq, device=q.device, dtype=torch.float32)
    grid = (cu.numel() - 1) * hq, triton.cdiv(int((cu[1:] - cu[:-1]).max().item()), 128), triton.cdiv(dv, 128)
    sp.flash_attn_fwd_kernel[grid](
        q, k, v, o, cu, lse, q.stride(1), q.stride(2), q.stride(3), k.stride(1), k.stride(2), k.stride(3),
        v.stride(1), v.stride(2), v.stride(3), o.stride(1), o.stride(2), o.stride(3), lse.stride(1), lse.stride(2),
        BLOCK_SIZE_QD=triton.next_power_of_2(d), HEAD_DIM_Q=d, HEAD_DIM_V=dv, BLOCK_SIZE_N=128, BLOCK_SIZE_KN=128,
        BLOCK_SIZE_D=128, NUM_HEADS=hq, GQA_RATIO=hq // hkv, sm_scale=(scale or d ** -0.5) * LOG2E,
        GLOBAL_WINDOW_SIZE=glob, LOCAL_WINDOW_SIZE=local)
    return o, lse


def dense_prefill_grads(q, k, v, cu, d_o):
    """Forward and backward through the reference's autograd function (flash_attn_triton.py:816-874):
    its three backward kernels (:184-592) and the host-side GQA sum (:813).  Returns (o, dq, dk, dv)."""
    dense = load()[0]
    q, k, v = (t.detach().clone().requires_grad_(True) for t in (q, k, v))
    o = dense.flash_attn_triton.apply(q, k, v, cu)
    o.backward(d_o)
    return o.detach(), q.grad, k.grad, v.grad


def rmsnorm_module(dim, eps, weight):
    """The reference's RMSNormTriton module (common/rms.py:358-382) with the given weight."""
    import torch
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    rms = importlib.import_module("common.rms")
    m = rms.RMSNormTriton(dim, eps).to(weight.device)
    with torch.no_grad():
        m.weight.copy_(weight)
    return m


def window_kernel_matches_its_oracle(local, glob) -> bool:
    return glob < 128 or local >= 128 * (glob // 128)


def decoding(q, kc, vc, cu):
    """flash_attention_decoding (flash_attn_decoding.py:213-336)."""
    return load()[1].flash_attention_decoding(q, kc, vc, cu)


def sparse_decoding(q, kc, vc, cu, glob, local):
    """flash_attention_sparse_decoding (flash_attn_decoding_sparse.py:222-365)."""
    return load()[2].flash_attention_sparse_decoding(q, kc, vc, cu, global_window_size=glob, local_window_size=local)


# --------------------------------------------------------------------------
# timing of the reference's kernels (bench.py runs this file as a child process)
# --------------------------------------------------------------------------
def _events_ms(fn, steps, warmup):
    import torch
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def bench_on_gpu():
    """Config 2 (kernel alone after its autotune, and through the reference's wrapper with its
    allocations, memsets and .item() synchronisation), config 3 through its wrapper, and the
    window kernel on the reference test's shape (flash_attn_sparse_attn_triton.py:445-503).  One
    JSON line; a kernel that does not run here is reported by its exception text."""
    import json
    import sys
    import torch
    sys.path.insert(0, os.path.dirname(HERE))
    from tritonops_b200 import workloads
    dev = torch.device("cuda", 0)
    out = {"what": "the reference's Triton kernels (triton %s) on this GPU, CUDA events" % __import__("triton").__version__}
    try:
        w = workloads.dense_causal(4, 32, 4096, 128, 1, dev, name="cfg2")
        o = torch.zeros_like(w.q)
        lse = torch.zeros(w.q.shape[:3], device=dev, dtype=torch.float32)
        dense_prefill_kernel_only(w.q, w.k, w.v, w.cu_seqlens, o, lse, 4096)      # compiles and autotunes
        out["cfg2_kernel_ms"] = _events_ms(lambda: dense_prefill_kernel_only(w.q, w.k, w.v, w.cu_seqlens, o, lse, 4096), 20, 3)
        out["cfg2_kernel_tflops"] = w.flops / out["cfg2_kernel_ms"] / 1e9
        out["cfg2_wrapper_ms"] = _events_ms(lambda: dense_prefill(w.q, w.k, w.v, w.cu_seqlens), 10, 3)
        try:
            out["cfg2_autotune_choice"] = str(load()[0].flash_attn_fwd_kernel.best_config)
        except Exception:
            pass
        del w, o, lse
    except Exception as e:  # noqa: BLE001
        out["cfg2_error"] = f"{type(e).__name__}: {str(e)[:300]}"
    if os.environ.get("B200ATTN_BENCH_REF_BACKWARD"):
        # forward + backward through the reference's autograd function (its backward kernels
        # autotune for about a minute at this size, so only on request)
        try:
            w = workloads.dense_causal(4, 32, 4096, 128, 1, dev, name="cfg2")
            do = torch.randn(w.q.shape, device=dev, dtype=torch.float32).to(w.q.dtype)
            dense = load()[0]
            o, lse = dense.flash_attn_triton_fwd(w.q, w.k, w.v, w.cu_seqlens, 128 ** -0.5 * LOG2E)
            fb = lambda: dense.flash_attn_triton_bwd(w.q, w.k, w.v, o, do, lse, w.cu_seqlens, 128 ** -0.5 * LOG2E)
            fb()
            out["cfg2_backward_wrapper_ms"] = _events_ms(fb, 5, 2)
            out["cfg2_backward_tflops"] = 2.5 * w.flops / out["cfg2_backward_wrapper_ms"] / 1e9
            del w, do, o, lse
        except Exception as e:  # noqa: BLE001
            out["cfg2_backward_error"] = f"{type(e).__name__}: {str(e)[:300]}"
    try:
        w3 = workloads.cfg3(dev)
        decoding(w3.q, w3.k_cache, w3.v_cache, w3.cu_seqlens)
        out["cfg3_wrapper_ms"] = _events_ms(lambda: decoding(w3.q, w3.k_cache, w3.v_cache, w3.cu_seqlens), 10, 3)
        out["cfg3_wrapper_GBs"] = w3.kv_bytes / out["cfg3_wrapper_ms"] / 1e6
        del w3
    except Exception as e:  # noqa: BLE001
        out["cfg3_error"] = f"{type(e).__name__}: {str(e)[:300]}"
    try:
        g = torch.Generator().manual_seed(42)
        q, k, v = (torch.rand(1, 4 * 2048, 4, 96, generator=g).to(torch.bfloat16).to(dev) for _ in range(3))
        cu = (torch.arange(5, dtype=torch.int32) * 2048).to(dev)
        window_prefill(q, k, v, cu, 128, 0)
        out["window_test_shape_ms"] = _events_ms(lambda: window_prefill(q, k, v, cu, 128, 0), 20, 3)
    except Exception as e:  # noqa: BLE001
        out["window_error"] = f"{type(e).__name__}: {str(e)[:300]}"
    print(json.dumps(out))


def interpret_cfg1():
    """Config 1's inputs through the reference's dense kernel executed by Triton's CPU
    interpreter (TRITON_INTERPRET=1 must be set before this process imports triton); the
    autotuner needs a GPU driver, so the kernel is entered through its `.fn`."""
    import json
    import sys
    import time
    import torch
    import triton
    sys.path.insert(0, os.path.dirname(HERE))
    from tritonops_b200 import workloads
    assert os.environ.get("TRITON_INTERPRET") == "1"
    dense = load()[0]
    w = workloads.cfg1("cpu")
    q, k, v, cu = w.q, w.k, w.v, w.cu_seqlens
    _, T, hq, d = q.shape
    o = torch.zeros_like(q)
    lse = torch.zeros(1, T, hq, dtype=torch.float32)

    def run():
        dense.flash_attn_fwd_kernel.fn[(hq, 1, 1)](
            q, k, v, o, cu, lse, q.stride(1), q.stride(2), q.stride(3), k.stride(1), k.stride(2), k.stride(3),
            v.stride(1), v.stride(2), v.stride(3), o.stride(1), o.stride(2), o.stride(3), lse.stride(1), lse.stride(2),
            BLOCK_SIZE_QD=triton.next_power_of_2(d), HEAD_DIM_Q=d, HEAD_DIM_V=d, BLOCK_SIZE_N=128, BLOCK_SIZE_KN=128,
            BLOCK_SIZE_D=128, NUM_HEADS=hq, GQA_RATIO=1, sm_scale=d ** -0.5 * LOG2E)

    run()
    n, t0 = 0, time.perf_counter()
    while time.perf_counter() - t0 < 2.0 and n < 50:
        run()
        n += 1
    dt = time.perf_counter() - t0
    print(json.dumps({"value": dt / n * 1e6, "unit": "us per call", "cores": 1, "kind": "reference",
                      "sample": f"{n} calls of the reference's flash_attn_fwd_kernel (causal) under TRITON_INTERPRET=1 "
                                f"on cfg1's inputs (fp16, B=1 H=2 S=128 D=64)"}))


if __name__ == "__main__":
    import sys as _sys
    if "--bench" in _sys.argv:
        bench_on_gpu()
    elif "--interpret-cfg1" in _sys.argv:
        interpret_cfg1()
