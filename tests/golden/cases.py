"""Seeded input recipes shared by make_golden.py (which runs the reference on
them) and by the tests (which rebuild the same inputs and compare with the
recorded reference outputs).  Inputs come from a seeded CPU generator, so they
are reproducible bit for bit; each fixture also records an input checksum so
that generator drift is detected rather than silently compared."""
import torch

DT = {"f16": torch.float16, "bf16": torch.bfloat16}


def cu_from(lens):
    cu = torch.zeros(len(lens) + 1, dtype=torch.int32)
    if lens:
        cu[1:] = torch.cumsum(torch.tensor(lens), 0)
    return cu


def packed_to_cache(k, cu):
    """[1, sum(len), H, D] packed rows -> zero-padded cache [B, Tmax, H, D], the
    hand copy the reference's tests do (flash_attn_decoding.py:404-425)."""
    B = len(cu) - 1
    tmax = int((cu[1:] - cu[:-1]).max())
    cache = torch.zeros(B, max(tmax, 1), k.shape[2], k.shape[3], dtype=k.dtype)
    for b in range(B):
        n = int(cu[b + 1] - cu[b])
        cache[b, :n] = k[0, int(cu[b]):int(cu[b + 1])]
    return cache


# name -> recipe.  kind "prefill": q [1,T,hq,d], k/v [1,T,hkv,d];
# kind "decode": q [B,hq,d], packed k/v [1,T,hkv,d] (+ padded caches).
CASES = {
    # reference's own dense test distribution: U[0,1) bf16 (flash_attn_triton.py:930-936)
    "dense_a": dict(kind="prefill", seed=42, lens=[97, 40, 5], hq=2, hkv=2, d=96, dtype="bf16", dist="rand"),
    "dense_b": dict(kind="prefill", seed=43, lens=[130, 61], hq=4, hkv=2, d=128, dtype="bf16", dist="rand"),
    "dense_c": dict(kind="prefill", seed=44, lens=[135, 1, 77], hq=4, hkv=1, d=64, dtype="bf16", dist="rand"),
    # benchmark config 1
    "cfg1": dict(kind="prefill", seed=0, lens=[128], hq=2, hkv=2, d=64, dtype="f16", dist="randn"),
    "dense_ragged_f16": dict(kind="prefill", seed=5, lens=[150, 37, 130], hq=4, hkv=2, d=96, dtype="f16", dist="randn"),
    "window_bf16": dict(kind="prefill", seed=11, lens=[300, 129], hq=4, hkv=2, d=96, dtype="bf16", dist="rand"),
    # decoding (flash_attn_decoding.py:371-437 scaled down); *_mha for the torch
    # oracles that need heads pre-expanded, *_gqa for the Triton wrappers
    "decode_mha": dict(kind="decode", seed=42, lens=[200, 515, 70], hq=2, hkv=2, d=96, dtype="f16", dist="randn"),
    "decode_gqa": dict(kind="decode", seed=42, lens=[200, 515, 70], hq=4, hkv=2, d=96, dtype="f16", dist="randn"),
    "sparse_decode_mha": dict(kind="decode", seed=7, lens=[700, 137, 64, 300], hq=4, hkv=4, d=128, dtype="f16", dist="randn"),
    "sparse_decode_gqa": dict(kind="decode", seed=7, lens=[700, 137, 0, 300], hq=4, hkv=2, d=128, dtype="f16", dist="randn"),
}


def build(name):
    c = CASES[name]
    g = torch.Generator().manual_seed(c["seed"])
    draw = (lambda *s: torch.rand(*s, generator=g)) if c["dist"] == "rand" else \
           (lambda *s: torch.randn(*s, generator=g))
    dt = DT[c["dtype"]]
    cu = cu_from(c["lens"])
    T = int(cu[-1])
    out = dict(cu=cu, lens=list(c["lens"]))
    if c["kind"] == "prefill":
        out["q"] = draw(1, T, c["hq"], c["d"]).to(dt)
    else:
        out["q"] = draw(len(c["lens"]), c["hq"], c["d"]).to(dt)
    out["k"] = draw(1, T, c["hkv"], c["d"]).to(dt)
    out["v"] = draw(1, T, c["hkv"], c["d"]).to(dt)
    if c["kind"] == "decode":
        out["kc"] = packed_to_cache(out["k"], cu)
        out["vc"] = packed_to_cache(out["v"], cu)
    return out


def checksum(inp):
    """Order-sensitive integer checksum of the 16-bit patterns of q, k, v."""
    tot = 0
    for i, n in enumerate(("q", "k", "v")):
        bits = inp[n].contiguous().view(torch.int16).to(torch.int64).flatten()
        w = torch.arange(1, bits.numel() + 1, dtype=torch.int64) % 65521
        tot = (tot * 31 + int((bits * w).sum())) % (1 << 61)
    return tot


def load_golden(fname):
    """Read a fixture written by make_golden.py -> {case: {name: tensor}}."""
    import os

    import numpy as np
    z = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), fname))
    out = {}
    for key in z.files:
        if key.endswith("__dtype"):
            continue
        case, name = key.split("/", 1)
        a = z[key]
        if key + "__dtype" in z.files:
            t = torch.from_numpy(a.copy()).view(DT[str(z[key + "__dtype"])])
        elif a.ndim == 0:
            t = a.item()
        else:
            t = torch.from_numpy(a.copy())
        out.setdefault(case, {})[name] = t
    return out
