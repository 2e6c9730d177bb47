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


def window_kernel_matches_its_oracle(local, glob) -> bool:
    return glob < 128 or local >= 128 * (glob // 128)


def decoding(q, kc, vc, cu):
    """flash_attention_decoding (flash_attn_decoding.py:213-336)."""
    return load()[1].flash_attention_decoding(q, kc, vc, cu)


def sparse_decoding(q, kc, vc, cu, glob, local):
    """flash_attention_sparse_decoding (flash_attn_decoding_sparse.py:222-365)."""
    return load()[2].flash_attention_sparse_decoding(q, kc, vc, cu, global_window_size=glob, local_window_size=local)
