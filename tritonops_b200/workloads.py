"""Seeded synthetic inputs for the five benchmark configurations and their
algorithmic work (FLOPs / bytes), plus scaled-down variants for tests.

The reference publishes no dataset; inputs are i.i.d. N(0,1) from the seeds the
configurations name.  Small configurations draw on the CPU generator so CPU
and GPU see identical bits; the large KV caches are drawn on the device."""
import math
from dataclasses import dataclass
from typing import Optional

import torch


@dataclass
class PrefillWork:
    q: torch.Tensor            # [1, B*S, Hq, D] packed
    k: torch.Tensor
    v: torch.Tensor
    cu_seqlens: torch.Tensor   # int32 [B+1]
    max_seqlen: int
    causal: bool
    scale: float
    flops: float               # 4*D per unmasked (query, key) pair
    block_idx: Optional[torch.Tensor] = None
    block_cnt: Optional[torch.Tensor] = None
    block_size: int = 64
    name: str = ""


@dataclass
class DecodeWork:
    q: torch.Tensor            # [B, Hq, D]
    k_cache: torch.Tensor      # [B, Tmax, Hkv, D]
    v_cache: torch.Tensor
    seqlens: torch.Tensor      # int32 [B]
    cu_seqlens: torch.Tensor   # int32 [B+1]
    max_seqlen: int
    scale: float
    kv_bytes: float            # K and V bytes of the visible keys + Q + O
    block_idx: Optional[torch.Tensor] = None
    block_size: int = 64
    name: str = ""


def _randn(shape, seed, dtype, device):
    """CPU-seeded normal draw moved to `device` (bit-identical everywhere)."""
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g).to(dtype).to(device)


def _randn_dev(shape, seed, dtype, device):
    g = torch.Generator(device=device).manual_seed(seed)
    return torch.randn(*shape, generator=g, device=device, dtype=torch.float32).to(dtype) \
        if math.prod(shape) < (1 << 28) else \
        torch.randn(*shape, generator=g, device=device, dtype=dtype)


def causal_flops(lens, heads, d):
    return float(sum(4 * heads * d * n * (n + 1) // 2 for n in lens))


def cfg1(device="cpu"):
    """Config 1: dense non-causal fp16, B=1,H=2,S=128,D=64, seed 0."""
    B, H, S, D = 1, 2, 128, 64
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(1, S, H, D, generator=g).to(torch.float16).to(device) for _ in range(3))
    cu = torch.tensor([0, S], dtype=torch.int32, device=device)
    return PrefillWork(q, k, v, cu, S, False, D ** -0.5, 4.0 * B * H * S * S * D, name="cfg1")


def dense_causal(B, H, S, D, seed, device, dtype=torch.bfloat16, hkv=None, name=""):
    hkv = hkv or H
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(1, B * S, H, D, generator=g).to(dtype).to(device)
    k = torch.randn(1, B * S, hkv, D, generator=g).to(dtype).to(device)
    v = torch.randn(1, B * S, hkv, D, generator=g).to(dtype).to(device)
    cu = (torch.arange(B + 1, dtype=torch.int32) * S).to(device)
    return PrefillWork(q, k, v, cu, S, True, D ** -0.5, causal_flops([S] * B, H, D), name=name)


def cfg2(device="cuda", batch=4):
    """Config 2: dense causal bf16, B=4,H=32,S=4096,D=128, seed 1."""
    return dense_causal(batch, 32, 4096, 128, 1, device, name="cfg2")


def decode_work(B, Hq, Hkv, D, tmax, lo, hi, seed, device, dtype=torch.bfloat16, on_device=False,
                name=""):
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(lo, hi + 1, (B,), generator=g).to(torch.int32)
    draw = _randn_dev if on_device else _randn
    q = draw((B, Hq, D), seed + 101, dtype, device)
    kc = draw((B, tmax, Hkv, D), seed + 102, dtype, device)
    vc = draw((B, tmax, Hkv, D), seed + 103, dtype, device)
    cu = torch.zeros(B + 1, dtype=torch.int32)
    cu[1:] = torch.cumsum(lens, 0)
    es = q.element_size()
    kv_bytes = float(int(lens.sum()) * Hkv * D * 2 * es + 2 * B * Hq * D * es)
    return DecodeWork(q, kc, vc, lens.to(device), cu.to(device), int(lens.max()), D ** -0.5,
                      kv_bytes, name=name)


def cfg3(device="cuda", batch=64):
    """Config 3: GQA decoding bf16, B=64,Hq=32,Hkv=8,D=128, cache padded to
    8192, lengths uniform in [1024, 8192] from seed 2."""
    return decode_work(batch, 32, 8, 128, 8192, 1024, 8192, 2, device, on_device=True, name="cfg3")


def block_sparse_lists(B, H, nqb, local_blocks, p, seed):
    """Config-4 pattern: q block i attends blocks max(0,i-local+1)..i plus each
    earlier block with probability p (Bernoulli per (b,h,i,j))."""
    g = torch.Generator().manual_seed(seed)
    keep = torch.rand(B, H, nqb, nqb, generator=g) < p
    i = torch.arange(nqb)[:, None]
    j = torch.arange(nqb)[None, :]
    local = (j <= i) & (j > i - local_blocks)
    mask = (keep & (j < i)) | local
    mask &= j <= i
    cnt = mask.sum(-1).to(torch.int32)
    max_nnz = int(cnt.max())
    # ascending indices of the set bits, -1 padded
    key = torch.where(mask, j.expand_as(mask), torch.full_like(mask, nqb, dtype=torch.long))
    idx = key.sort(-1).values[..., :max_nnz]
    idx = torch.where(idx >= nqb, torch.full_like(idx, -1), idx).to(torch.int32)
    return idx.contiguous(), cnt.contiguous()


def block_sparse_flops(idx, cnt, block, d, seqlen):
    """4*D per visible (query, key) pair: full blocks count block^2 pairs, the
    diagonal block block*(block+1)/2."""
    B, H, nqb, _ = idx.shape
    qb = torch.arange(nqb)[None, None, :, None]
    valid = idx >= 0
    diag = (valid & (idx == qb)).sum().item()
    full = valid.sum().item() - diag
    return 4.0 * d * (full * block * block + diag * block * (block + 1) // 2)


def cfg4(device="cuda", B=2, H=16, S=16384):
    """Config 4: block-sparse causal prefill bf16, D=128, 64x64 blocks, window of
    8 blocks + Bernoulli(0.1) earlier blocks, seed 3."""
    D, blk = 128, 64
    w = dense_causal(B, H, S, D, 3, device, name="cfg4")
    idx, cnt = block_sparse_lists(B, H, S // blk, 8, 0.1, 3)
    w.flops = block_sparse_flops(idx, cnt, blk, D, S)
    w.block_idx, w.block_cnt, w.block_size = idx.to(device), cnt.to(device), blk
    return w


def topk_block_lists(B, H, nblocks, nsel, seed):
    """Config-5 pattern: nsel distinct blocks uniformly without replacement,
    last block always included, ascending."""
    g = torch.Generator().manual_seed(seed)
    r = torch.rand(B, H, nblocks, generator=g)
    r[..., nblocks - 1] = -1.0
    return r.argsort(-1)[..., :nsel].sort(-1).values.to(torch.int32).contiguous()


def cfg5(device="cuda", B=32, H=32, T=32768):
    """Config 5: top-k block decoding bf16, MHA H=32, D=128, KV length 32768 in
    512 blocks of 64, 64 blocks selected per (b,h), seed 4."""
    D, blk, nsel = 128, 64, 64
    w = decode_work(B, H, H, D, T, T, T, 4, device, on_device=True, name="cfg5")
    w.block_idx = topk_block_lists(B, H, T // blk, nsel, 4).to(device)
    w.block_size = blk
    es = w.q.element_size()
    w.kv_bytes = float(B * H * nsel * blk * D * 2 * es + 2 * B * H * D * es + w.block_idx.numel() * 4)
    return w
