"""Generate the golden fixtures under tests/golden/ by running the REFERENCE.

Run where a checkout of the reference exists, named by REFERENCE_ROOT:

    REFERENCE_ROOT=<checkout of rookie-joe/TritonOps> python tests/golden/make_golden.py

Inputs are the seeded recipes of cases.py; the fixtures hold the reference's
outputs plus an input checksum.  Two files are written:

* ``golden_torch.npz``  : the reference's naive torch paths (flash_attn_torch,
  flash_attn_decoding_torch, the sparse decoding oracle, flash_attn_sparse_torch
  and the tutorial's torch_full_attention) on CPU tensors.
* ``golden_triton.npz`` : the reference's Triton kernels executed by Triton's
  CPU interpreter (TRITON_INTERPRET=1, fp16 only -- the interpreter mishandles
  bf16).  Autotuned kernels are entered through ``kernel.fn`` because the
  autotuner itself needs a GPU driver.

Half-precision outputs are stored as raw 16-bit patterns (int16) with a dtype
tag; ``load_golden`` in cases.py reads them back.
"""
import ast
import math
import os
import subprocess
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from cases import build, checksum  # noqa: E402

REF = os.environ.get("REFERENCE_ROOT")
if not REF or not os.path.isdir(REF):
    raise SystemExit("set REFERENCE_ROOT to a checkout of the reference (rookie-joe/TritonOps)")
STORE = {}


def put(case, **tensors):
    for name, t in tensors.items():
        key = f"{case}/{name}"
        if isinstance(t, torch.Tensor) and t.dtype in (torch.float16, torch.bfloat16):
            STORE[key] = t.contiguous().view(torch.int16).numpy()
            STORE[key + "__dtype"] = np.array("f16" if t.dtype == torch.float16 else "bf16")
        elif isinstance(t, torch.Tensor):
            STORE[key] = t.contiguous().numpy()
        else:
            STORE[key] = np.array(t)
    print("recorded", case, list(tensors))


def flush(fname):
    np.savez_compressed(os.path.join(HERE, fname), **STORE)
    print("wrote", fname, os.path.getsize(os.path.join(HERE, fname)), "bytes")
    STORE.clear()


def import_reference():
    sys.path.insert(0, REF)
    from flash_attn_triton import flash_attn_triton as dense
    from flash_attn_triton import flash_attn_decoding as dec
    from flash_attn_triton import flash_attn_decoding_sparse as dec_sp
    from flash_attn_triton import flash_attn_sparse_attn_triton as sp
    return dense, dec, dec_sp, sp


# ---------------------------------------------------------------- torch paths
def gen_torch():
    dense, dec, dec_sp, sp = import_reference()

    for name in ("dense_a", "dense_b", "dense_c"):
        i = build(name)
        put(name, o=dense.flash_attn_torch(i["q"], i["k"], i["v"], i["cu"]), insum=checksum(i))
        # gradients of the reference's torch path by autograd, as its own test does
        # (flash_attn_triton.py:1053-1063), with a seeded dO
        q, k, v = (i[n].clone().requires_grad_(True) for n in "qkv")
        o = dense.flash_attn_torch(q, k, v, i["cu"])
        do = torch.randn(o.shape, generator=torch.Generator().manual_seed(1234)).to(o.dtype)
        (o * do).sum().backward()
        put(name, do=do, dq=q.grad, dk=k.grad, dv=v.grad)

    # config 1: causal via flash_attn_torch; non-causal via the tutorial's
    # torch_full_attention, whose module runs CUDA code at import, so only
    # that function's source is compiled.  Tutorial layout is [B,H,N,D].
    i = build("cfg1")
    src = open(os.path.join(REF, "tutorial", "4.3.multi_head_attention.py")).read()
    fn = [n for n in ast.parse(src).body
          if isinstance(n, ast.FunctionDef) and n.name == "torch_full_attention"][0]
    ns = {"torch": torch, "math": math}
    exec(compile(ast.Module([fn], []), "tutorial_4_3", "exec"), ns)
    o_full = ns["torch_full_attention"](*(i[n].permute(0, 2, 1, 3) for n in "qkv"))
    put("cfg1", o_causal=dense.flash_attn_torch(i["q"], i["k"], i["v"], i["cu"]),
        o_noncausal=o_full.permute(0, 2, 1, 3).contiguous(), insum=checksum(i))

    i = build("decode_mha")
    put("decode_mha", o=dec.flash_attn_decoding_torch(i["q"], i["k"], i["v"], i["cu"]),
        insum=checksum(i))

    i = build("sparse_decode_mha")
    for G, L in [(64, 64), (128, 200), (256, 1024)]:
        o = dec_sp.flash_attn_decoding_torch(i["q"], i["k"], i["v"], i["cu"],
                                             global_window_size=G, local_window_size=L)
        put("sparse_decode_mha", **{f"o_G{G}_L{L}": o})
    put("sparse_decode_mha", insum=checksum(i))

    i = build("window_bf16")
    for L, G in [(128, 0), (64, 100), (200, 256), (1, 0), (64, 128)]:
        o = sp.flash_attn_sparse_torch(i["q"], i["k"], i["v"], i["cu"], None, L, G)
        put("window_bf16", **{f"o_L{L}_G{G}": o})
    put("window_bf16", insum=checksum(i))
    flush("golden_torch.npz")


# ------------------------------------------------------- Triton interpreter
def gen_triton():
    assert os.environ.get("TRITON_INTERPRET") == "1"
    import triton
    dense, dec, dec_sp, sp = import_reference()
    LOG2E = 1.4426950408889634

    def run_prefill(kernel, i, extra):
        q, k, v, cu = i["q"], i["k"], i["v"], i["cu"]
        _, T, hq, d = q.shape
        hkv, dv = v.shape[2], v.shape[3]
        o = torch.zeros(1, T, hq, d, dtype=q.dtype)
        lse = torch.zeros(1, T, hq, dtype=torch.float32)
        B = len(cu) - 1
        grid = (B * hq, triton.cdiv(int((cu[1:] - cu[:-1]).max()), 128), triton.cdiv(dv, 128))
        kernel.fn[grid](q, k, v, o, cu, lse,
                        q.stride(1), q.stride(2), q.stride(3),
                        k.stride(1), k.stride(2), k.stride(3),
                        v.stride(1), v.stride(2), v.stride(3),
                        o.stride(1), o.stride(2), o.stride(3),
                        lse.stride(1), lse.stride(2),
                        BLOCK_SIZE_QD=triton.next_power_of_2(d), HEAD_DIM_Q=d, HEAD_DIM_V=dv,
                        BLOCK_SIZE_N=128, BLOCK_SIZE_KN=128, BLOCK_SIZE_D=128,
                        NUM_HEADS=hq, GQA_RATIO=hq // hkv, sm_scale=d ** -0.5 * LOG2E, **extra)
        return o, lse

    # dense kernel (always causal): config 1 and a ragged GQA case with D=96
    for name in ("cfg1", "dense_ragged_f16"):
        i = build(name)
        o, lse = run_prefill(dense.flash_attn_fwd_kernel, i, {})
        put(name, o=o, lse2=lse, insum=checksum(i))

    # window-sparse kernel, only where it agrees with its own oracle
    # (G < 128 or L >= 128 * floor(G / 128))
    i = build("dense_ragged_f16")
    for L, G in [(64, 100), (256, 256), (128, 64)]:
        o, lse = run_prefill(sp.flash_attn_fwd_kernel, i,
                             dict(LOCAL_WINDOW_SIZE=L, GLOBAL_WINDOW_SIZE=G))
        put("dense_ragged_f16", **{f"win_o_L{L}_G{G}": o, f"win_lse2_L{L}_G{G}": lse})

    i = build("decode_gqa")
    put("decode_gqa", o=dec.flash_attention_decoding(i["q"], i["kc"], i["vc"], i["cu"]),
        insum=checksum(i))

    i = build("sparse_decode_gqa")
    for G, L in [(64, 64), (128, 200), (256, 1024)]:
        o = dec_sp.flash_attention_sparse_decoding(i["q"], i["kc"], i["vc"], i["cu"],
                                                   global_window_size=G, local_window_size=L)
        put("sparse_decode_gqa", **{f"o_G{G}_L{L}": o})
    put("sparse_decode_gqa", insum=checksum(i))
    flush("golden_triton.npz")


if __name__ == "__main__":
    if len(sys.argv) > 1 and sys.argv[1] == "--triton":
        gen_triton()
    else:
        gen_torch()
        env = dict(os.environ, TRITON_INTERPRET="1")
        subprocess.check_call([sys.executable, os.path.abspath(__file__), "--triton"], env=env)
