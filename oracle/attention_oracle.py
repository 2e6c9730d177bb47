"""CPU oracle for the flash_attn_triton hot path.  TEST INFRASTRUCTURE ONLY.

This module is the checker, never the product: only the test-suite, the smoke
check and the benchmark's CPU-baseline leg may import it.  The CUDA library
never routes through it and has no CPU fallback.

Parity pin: every function here is checked (tests/test_oracle_golden.py)
against fixtures under tests/golden/ that were produced by importing the
reference implementation itself -- its naive torch paths and, for fp16, its
Triton kernels run under TRITON_INTERPRET=1 -- by tests/golden/make_golden.py.
The block-index sparse layouts do not exist in the reference; for those the
oracle is pinned only through its equivalence with the dense masked math
(window masks expressed as block lists).

Two families of functions:

* ``*_exact``  : fp32/fp64 ``softmax(Q K^T * scale + mask) V`` and the natural
  log-sum-exp, computed from the fp16/bf16-rounded inputs.  This is what the
  CUDA kernels are compared with.
* ``*_refpath``: restatements of the reference's own naive torch code with its
  mixed precision (scores in the input dtype, fp32 softmax, probabilities cast
  back), used to pin the oracle against the reference and as the timed CPU
  baseline.

All layouts follow the reference:
  prefill   q [1, T, Hq, D], k/v [1, T, Hkv, D], cu_seq_lens int32 [B+1]
  decoding  q [B, Hq, D], k/v cache [B, Tmax, Hkv, D], lengths from cu_seq_lens
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import torch

LOG2E = 1.4426950408889634


# --------------------------------------------------------------------------
# helpers
# --------------------------------------------------------------------------
def _lens(cu_seq_lens) -> list:
    cu = [int(x) for x in cu_seq_lens]
    return [(cu[i], cu[i + 1]) for i in range(len(cu) - 1)]


def _masked_softmax_v(s: torch.Tensor, v: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """s [H, Q, K] with -inf at masked positions, v [H, K, D].

    Returns (o [H,Q,D], natural lse [H,Q]).  Rows with no visible key give
    o = 0 and lse = -inf (the reference's kernels leave their zero-initialised
    output untouched for such rows)."""
    m = s.max(dim=-1, keepdim=True).values
    m = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    p = torch.exp(s - m)
    l = p.sum(dim=-1, keepdim=True)
    o = torch.matmul(p, v) / torch.where(l == 0, torch.ones_like(l), l)
    lse = (m + torch.log(l)).squeeze(-1)
    return o, lse


# --------------------------------------------------------------------------
# dense prefill
# --------------------------------------------------------------------------
def dense_prefill_exact(q, k, v, cu_seq_lens, *, causal=True, scale=None,
                        dtype=torch.float32):
    """softmax(Q K^T * scale [+ causal mask]) V per packed sequence, GQA.

    Math of flash_attn_fwd_kernel (flash_attn_triton/flash_attn_triton.py:145-180)
    with kv head = h // (Hq/Hkv) (:87); ``causal=False`` is the tutorial's
    non-causal math (tutorial/4.3.multi_head_attention.py:11-19).  ``scale`` is
    the natural scale (default D**-0.5, :839 without the log2e factor).
    Returns (o [1,T,Hq,Dv] in ``dtype``, natural-log LSE [1,T,Hq])."""
    _, T, Hq, D = q.shape
    Hkv, Dv = k.shape[2], v.shape[3]
    g = Hq // Hkv
    if scale is None:
        scale = D ** -0.5
    o = torch.zeros(1, T, Hq, Dv, dtype=dtype)
    lse = torch.full((1, T, Hq), -math.inf, dtype=dtype)
    for s0, s1 in _lens(cu_seq_lens):
        n = s1 - s0
        if n <= 0:
            continue
        bq = q[0, s0:s1].to(dtype).permute(1, 0, 2)                       # [Hq,n,D]
        bk = k[0, s0:s1].to(dtype).permute(1, 0, 2).repeat_interleave(g, 0)
        bv = v[0, s0:s1].to(dtype).permute(1, 0, 2).repeat_interleave(g, 0)
        s = torch.matmul(bq, bk.transpose(1, 2)) * scale
        if causal:
            idx = torch.arange(n)
            s = s.masked_fill(~(idx[:, None] >= idx[None, :]), -math.inf)
        oo, ll = _masked_softmax_v(s, bv)
        o[0, s0:s1] = oo.permute(1, 0, 2)
        lse[0, s0:s1] = ll.permute(1, 0)
    return o, lse


def dense_prefill_grads_exact(q, k, v, cu_seq_lens, d_o, *, causal=True, scale=None,
                              dtype=torch.float32):
    """dQ, dK, dV of dense_prefill_exact by autograd in ``dtype`` (the math of
    flash_attn_triton_bwd, flash_attn_triton/flash_attn_triton.py:184-592: D =
    rowsum(dO o O), dS = P o (dP - D), dQ = scale dS K, dK = scale dS^T Q, dV =
    P^T dO, with dK / dV summed over each GQA group, :813)."""
    qf = q.detach().to(dtype).requires_grad_(True)
    kf = k.detach().to(dtype).requires_grad_(True)
    vf = v.detach().to(dtype).requires_grad_(True)
    _, T, Hq, D = q.shape
    Hkv = k.shape[2]
    g = Hq // Hkv
    if scale is None:
        scale = D ** -0.5
    loss = qf.sum() * 0
    for s0, s1 in _lens(cu_seq_lens):
        n = s1 - s0
        if n <= 0:
            continue
        bq = qf[0, s0:s1].permute(1, 0, 2)
        bk = kf[0, s0:s1].permute(1, 0, 2).repeat_interleave(g, 0)
        bv = vf[0, s0:s1].permute(1, 0, 2).repeat_interleave(g, 0)
        s = torch.matmul(bq, bk.transpose(1, 2)) * scale
        if causal:
            idx = torch.arange(n)
            s = s.masked_fill(~(idx[:, None] >= idx[None, :]), -math.inf)
        o = torch.matmul(torch.softmax(s, -1), bv).permute(1, 0, 2)        # [n, Hq, Dv]
        loss = loss + (o * d_o[0, s0:s1].to(dtype)).sum()
    loss.backward()
    return qf.grad, kf.grad, vf.grad


def dense_prefill_refpath(q, k, v, cu_seq_lens):
    """Restatement of flash_attn_torch (flash_attn_triton/flash_attn_triton.py:877-915):
    scores in the input dtype, causal fill, fp32 softmax, P cast back to the
    input dtype, P @ V in the input dtype.  Returns o in q.dtype."""
    _, T, H, Dq = q.shape
    Dv = v.shape[-1]
    kH = k.shape[2]
    k = k.repeat_interleave(H // kH, dim=2)
    v = v.repeat_interleave(H // kH, dim=2)
    o = torch.zeros(1, T, H, Dv, dtype=q.dtype)
    sm_scale = (1 / Dq) ** 0.5
    for s0, s1 in _lens(cu_seq_lens):
        n = s1 - s0
        bq, bk, bv = q[0, s0:s1], k[0, s0:s1], v[0, s0:s1]
        qk = torch.einsum("qhd,khd->hqk", bq, bk) * sm_scale
        idx = torch.arange(n)
        qk = qk.masked_fill(~(idx[:, None] >= idx[None, :])[None], -math.inf).float()
        p = torch.softmax(qk, dim=-1, dtype=torch.float32)
        o[0, s0:s1] = torch.einsum("hqk,khd->qhd", p.to(q.dtype), bv)
    return o


# --------------------------------------------------------------------------
# decoding over a padded cache
# --------------------------------------------------------------------------
def decoding_exact(q, k_cache, v_cache, seqlens, *, scale=None, dtype=torch.float32,
                   visible=None):
    """One query token per sequence against a padded cache [B,Tmax,Hkv,D].

    Math of flash_attn_decoding_kernel + correction kernel
    (flash_attn_triton/flash_attn_decoding.py:110-122, :173-208): the split
    into chunks does not change the value, so the oracle evaluates the
    un-split softmax.  ``visible(b, n) -> bool[n]`` optionally restricts the
    keys (used by the sparse variants).  Sequences of length 0 give o = 0
    (:49-50 plus the zero-initialised buffers).  Returns o [B,Hq,Dv]."""
    B, Hq, D = q.shape
    Hkv, Dv = k_cache.shape[2], v_cache.shape[3]
    g = Hq // Hkv
    if scale is None:
        scale = D ** -0.5
    o = torch.zeros(B, Hq, Dv, dtype=dtype)
    for b in range(B):
        n = int(seqlens[b])
        if n <= 0:
            continue
        bk = k_cache[b, :n].to(dtype).permute(1, 0, 2).repeat_interleave(g, 0)   # [Hq,n,D]
        bv = v_cache[b, :n].to(dtype).permute(1, 0, 2).repeat_interleave(g, 0)
        s = torch.einsum("hd,hkd->hk", q[b].to(dtype), bk) * scale
        if visible is not None:
            vis = visible(b, n)
            if vis.dim() == 1:
                vis = vis[None, :]
            s = s.masked_fill(~vis, -math.inf)
        oo, _ = _masked_softmax_v(s[:, None, :], bv)
        o[b] = oo[:, 0]
    return o


def decoding_refpath(q, k_packed, v_packed, cu_seq_lens, qk_scale=None):
    """Restatement of flash_attn_decoding_torch
    (flash_attn_triton/flash_attn_decoding.py:339-368): packed K/V
    [1, sum(len), H, D] with heads already expanded to Hq, everything in the
    input dtype (a low-precision oracle)."""
    _, T, H, Dv = v_packed.shape
    Dq = q.shape[-1]
    B = len(cu_seq_lens) - 1
    o = torch.zeros(B, H, Dv, dtype=q.dtype)
    if qk_scale is None:
        qk_scale = Dq ** -0.5
    for i, (s0, s1) in enumerate(_lens(cu_seq_lens)):
        bk, bv = k_packed[0, s0:s1], v_packed[0, s0:s1]
        qk = torch.einsum("hd,khd->hk", q[i], bk).to(q.dtype) * qk_scale
        p = qk.softmax(dim=-1)
        o[i] = torch.einsum("hk,khd->hd", p.to(q.dtype), bv)
    return o


def decoding_split_combine(q, k_cache, v_cache, seqlens, *, chunk, scale=None,
                           dtype=torch.float32):
    """The reference's two-launch algorithm spelled out: per chunk a partial
    that is normalised inside the chunk plus its base-2 LSE
    (flash_attn_decoding.py:110-122), then the LSE-weighted combine
    (:173-208).  Used to check that split + combine equals the un-split math
    for any chunk size, including the 512-token chunks of the CUDA path."""
    B, Hq, D = q.shape
    Hkv, Dv = k_cache.shape[2], v_cache.shape[3]
    g = Hq // Hkv
    if scale is None:
        scale = D ** -0.5
    o = torch.zeros(B, Hq, Dv, dtype=dtype)
    for b in range(B):
        n = int(seqlens[b])
        nchunk = (n + chunk - 1) // chunk
        parts, lses = [], []
        for c in range(nchunk):
            lo, hi = c * chunk, min(n, (c + 1) * chunk)
            bk = k_cache[b, lo:hi].to(dtype).permute(1, 0, 2).repeat_interleave(g, 0)
            bv = v_cache[b, lo:hi].to(dtype).permute(1, 0, 2).repeat_interleave(g, 0)
            s = torch.einsum("hd,hkd->hk", q[b].to(dtype), bk) * (scale * LOG2E)
            m = s.max(dim=-1).values
            lse2 = m + torch.log2(torch.exp2(s - m[:, None]).sum(-1))
            parts.append(torch.einsum("hk,hkd->hd", torch.exp2(s - lse2[:, None]), bv))
            lses.append(lse2)
        if nchunk == 0:
            continue
        lse2 = torch.stack(lses, 0)                                   # [C,Hq]
        gl = torch.logsumexp(lse2 / LOG2E, dim=0) * LOG2E
        w = torch.exp2(lse2 - gl[None])
        o[b] = (torch.stack(parts, 0) * w[:, :, None]).sum(0)
    return o


# --------------------------------------------------------------------------
# window-sparse prefill / decoding (the reference's "sparse": local + global)
# --------------------------------------------------------------------------
def window_mask(n: int, local: int, glob: int) -> torch.Tensor:
    """Query i sees key j iff j <= i and (i - j < local or j < glob)
    (flash_attn_sparse_attn_triton.py:422-433)."""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    return (i >= j) & ((i < j + local) | (j < glob))


def window_prefill_exact(q, k, v, cu_seq_lens, *, local, glob, scale=None,
                         dtype=torch.float32):
    """Oracle semantics of flash_attn_sparse_torch, the torch function
    (flash_attn_sparse_attn_triton.py:391-442), in fp32; natural scale.
    Returns (o, natural LSE)."""
    _, T, Hq, D = q.shape
    Hkv, Dv = k.shape[2], v.shape[3]
    g = Hq // Hkv
    if scale is None:
        scale = D ** -0.5
    o = torch.zeros(1, T, Hq, Dv, dtype=dtype)
    lse = torch.full((1, T, Hq), -math.inf, dtype=dtype)
    for s0, s1 in _lens(cu_seq_lens):
        n = s1 - s0
        if n <= 0:
            continue
        bq = q[0, s0:s1].to(dtype).permute(1, 0, 2)
        bk = k[0, s0:s1].to(dtype).permute(1, 0, 2).repeat_interleave(g, 0)
        bv = v[0, s0:s1].to(dtype).permute(1, 0, 2).repeat_interleave(g, 0)
        s = torch.matmul(bq, bk.transpose(1, 2)) * scale
        s = s.masked_fill(~window_mask(n, local, glob)[None], -math.inf)
        oo, ll = _masked_softmax_v(s, bv)
        o[0, s0:s1] = oo.permute(1, 0, 2)
        lse[0, s0:s1] = ll.permute(1, 0)
    return o, lse


def window_prefill_refpath(q, k, v, cu_seqlens, softmax_scale=None,
                           local_window_size=0, global_window_size=0):
    """Restatement of flash_attn_sparse_torch
    (flash_attn_sparse_attn_triton.py:391-442): per (b, h) dense scores in the
    input dtype, mask, scale, softmax in the input dtype."""
    _, T, H, Dq = q.shape
    Hk = k.shape[-2]
    g = H // Hk
    o = torch.zeros_like(q)
    if softmax_scale is None:
        softmax_scale = Dq ** -0.5
    for s0, s1 in _lens(cu_seqlens):
        n = s1 - s0
        mask = window_mask(n, local_window_size, global_window_size)
        for h in range(H):
            bq, bk, bv = q[0, s0:s1, h], k[0, s0:s1, h // g], v[0, s0:s1, h // g]
            qk = bq @ bk.T
            qk = torch.where(mask, qk, torch.full_like(qk, -math.inf)) * softmax_scale
            o[0, s0:s1, h] = qk.softmax(dim=-1) @ bv
    return o


def window_decode_visible(local: int, glob: int):
    """Key j of a length-n sequence is visible iff j < glob or j >= n - local
    (flash_attn_decoding_sparse.py:82-85, oracle :391-398)."""
    def vis(b, n):
        j = torch.arange(n)
        return (j < glob) | (j + local >= n)
    return vis


def window_decoding_exact(q, k_cache, v_cache, seqlens, *, glob, local, scale=None,
                          dtype=torch.float32):
    return decoding_exact(q, k_cache, v_cache, seqlens, scale=scale, dtype=dtype,
                          visible=window_decode_visible(local, glob))


def window_decoding_refpath(q, k_packed, v_packed, cu_seq_lens,
                            global_window_size=64, local_window_size=64):
    """Restatement of the sparse flash_attn_decoding_torch
    (flash_attn_decoding_sparse.py:368-406); heads already expanded."""
    _, T, H, Dv = v_packed.shape
    Dq = q.shape[-1]
    B = len(cu_seq_lens) - 1
    o = torch.zeros(B, H, Dv, dtype=q.dtype)
    qk_scale = Dq ** -0.5
    for i, (s0, s1) in enumerate(_lens(cu_seq_lens)):
        n = s1 - s0
        bk, bv = k_packed[0, s0:s1], v_packed[0, s0:s1]
        j = torch.arange(n)
        mask = (n <= j + local_window_size) | (j < global_window_size)
        qk = torch.einsum("hd,khd->hk", q[i], bk).to(q.dtype) * qk_scale
        qk = torch.where(mask[None, :], qk, torch.full_like(qk, -math.inf))
        o[i] = torch.einsum("hk,khd->hd", qk.softmax(dim=-1).to(q.dtype), bv)
    return o


# --------------------------------------------------------------------------
# block-index sparse layouts (defined by the benchmark configs, not the reference)
# --------------------------------------------------------------------------
def block_list_mask(n: int, block: int, idx_row: torch.Tensor, cnt_row: torch.Tensor,
                    causal: bool = True) -> torch.Tensor:
    """Expand one (b, h) block list to a dense [n, n] boolean mask.

    idx_row int32 [n_qblocks, max_nnz] ascending KV-block indices padded with
    -1, cnt_row int32 [n_qblocks].  Inside any block the element-wise causal
    mask applies (only the diagonal block is actually cut by it)."""
    nqb = (n + block - 1) // block
    m = torch.zeros(n, n, dtype=torch.bool)
    for qb in range(nqb):
        q0, q1 = qb * block, min(n, (qb + 1) * block)
        for t in range(int(cnt_row[qb])):
            kb = int(idx_row[qb, t])
            if kb < 0:
                continue
            k0, k1 = kb * block, min(n, (kb + 1) * block)
            m[q0:q1, k0:k1] = True
    if causal:
        i = torch.arange(n)
        m &= i[:, None] >= i[None, :]
    return m


def block_sparse_prefill_exact(q, k, v, cu_seq_lens, block_idx, block_cnt, *, block=64,
                               causal=True, scale=None, dtype=torch.float32):
    """Block-sparse prefill: block_idx int32 [B,Hq,n_qblocks,max_nnz],
    block_cnt int32 [B,Hq,n_qblocks]; block indices are relative to the
    sequence.  Returns (o, natural LSE)."""
    _, T, Hq, D = q.shape
    Hkv, Dv = k.shape[2], v.shape[3]
    g = Hq // Hkv
    if scale is None:
        scale = D ** -0.5
    o = torch.zeros(1, T, Hq, Dv, dtype=dtype)
    lse = torch.full((1, T, Hq), -math.inf, dtype=dtype)
    for b, (s0, s1) in enumerate(_lens(cu_seq_lens)):
        n = s1 - s0
        if n <= 0:
            continue
        for h in range(Hq):
            mask = block_list_mask(n, block, block_idx[b, h], block_cnt[b, h], causal)
            bq = q[0, s0:s1, h].to(dtype)
            bk = k[0, s0:s1, h // g].to(dtype)
            bv = v[0, s0:s1, h // g].to(dtype)
            s = (bq @ bk.T) * scale
            s = s.masked_fill(~mask, -math.inf)
            oo, ll = _masked_softmax_v(s[None], bv[None])
            o[0, s0:s1, h] = oo[0]
            lse[0, s0:s1, h] = ll[0]
    return o, lse


def block_sparse_decoding_exact(q, k_cache, v_cache, seqlens, block_idx, block_cnt=None, *,
                                block=64, scale=None, dtype=torch.float32):
    """Top-k block decoding: block_idx int32 [B,Hkv,n_sel] ascending (-1 =
    padding), optional block_cnt int32 [B,Hkv].  The query heads of a GQA
    group share their KV head's list.  Tokens >= seqlens[b] are never
    visible.  Gathers only the selected blocks, so the cache may be large."""
    B, Hq, D = q.shape
    Hkv, Dv = k_cache.shape[2], v_cache.shape[3]
    g = Hq // Hkv
    if scale is None:
        scale = D ** -0.5
    o = torch.zeros(B, Hq, Dv, dtype=dtype)
    for b in range(B):
        n = int(seqlens[b])
        for hk in range(Hkv):
            row = block_idx[b, hk]
            cnt = int(block_cnt[b, hk]) if block_cnt is not None else row.numel()
            toks = []
            for t in range(cnt):
                kb = int(row[t])
                if kb < 0 or kb * block >= n:
                    continue
                toks.append(torch.arange(kb * block, min(n, (kb + 1) * block)))
            if not toks or sum(t.numel() for t in toks) == 0:
                continue
            tok = torch.cat(toks)
            bk = k_cache[b, tok, hk].to(dtype)          # [n_tok, D]
            bv = v_cache[b, tok, hk].to(dtype)
            bq = q[b, hk * g:(hk + 1) * g].to(dtype)    # [g, D]
            s = (bq @ bk.T) * scale
            p = torch.softmax(s, dim=-1)
            o[b, hk * g:(hk + 1) * g] = p @ bv
    return o


def window_to_block_lists(n: int, block: int, local: int, glob: int):
    """KV blocks touched by the window mask for every q block of a length-n
    sequence, as (idx [nqb, max_nnz] padded with -1, cnt [nqb]).  A helper to
    tie the block-list layout back to the reference's window semantics."""
    nqb = (n + block - 1) // block
    rows = []
    m = window_mask(n, local, glob)
    for qb in range(nqb):
        q0, q1 = qb * block, min(n, (qb + 1) * block)
        act = [kb for kb in range(nqb)
               if bool(m[q0:q1, kb * block:min(n, (kb + 1) * block)].any())]
        rows.append(act)
    mx = max(len(r) for r in rows) if rows else 0
    idx = torch.full((nqb, max(mx, 1)), -1, dtype=torch.int32)
    cnt = torch.zeros(nqb, dtype=torch.int32)
    for i, r in enumerate(rows):
        idx[i, :len(r)] = torch.tensor(r, dtype=torch.int32)
        cnt[i] = len(r)
    return idx, cnt


def window_decode_block_cover(lens: Sequence[int], block: int, local: int, glob: int, max_sel: int):
    """Blocks holding at least one visible key of the decoding window pattern
    (flash_attn_decoding_sparse.py:82-85), per sequence, ascending, first
    max_sel kept: (idx [B, max_sel] padded with -1, cnt [B])."""
    vis = window_decode_visible(local, glob)
    idx = torch.full((len(lens), max_sel), -1, dtype=torch.int32)
    cnt = torch.zeros(len(lens), dtype=torch.int32)
    for b, n in enumerate(lens):
        n = max(int(n), 0)
        m = vis(b, n)
        act = [kb for kb in range((n + block - 1) // block) if bool(m[kb * block:(kb + 1) * block].any())]
        act = act[:max_sel]
        idx[b, :len(act)] = torch.tensor(act, dtype=torch.int32)
        cnt[b] = len(act)
    return idx, cnt


def topk_blocks(scores, top_k: int, n_valid=None, force_first: int = 0, force_last: int = 0):
    """Row-wise top-k block choice in ascending block order.  Candidates are
    blocks 0..n_valid-1; the first force_first and last force_last candidates
    always win; otherwise larger score wins, ties go to the lower block, NaN
    ranks below -inf.  Returns (idx [rows, top_k] padded with -1, cnt [rows])."""
    import numpy as np
    s = np.asarray(scores, dtype=np.float32)
    rows, n = s.shape
    idx = np.full((rows, top_k), -1, dtype=np.int32)
    cnt = np.zeros(rows, dtype=np.int32)
    for r in range(rows):
        nv = n if n_valid is None else max(0, min(int(n_valid[r]), n))
        # rank key: (class, score); class 2 forced, 1 real number, 0 NaN
        order = []
        for j in range(nv):
            forced = j < force_first or j >= nv - force_last
            x = float(s[r, j])
            if forced:
                key = (2, 0.0)
            elif x != x:
                key = (0, 0.0)
            else:
                key = (1, x)
            order.append((key, j))
        order.sort(key=lambda t: (-t[0][0], -t[0][1], t[1]))
        take = sorted(j for _, j in order[:min(top_k, nv)])
        idx[r, :len(take)] = take
        cnt[r] = len(take)
    return torch.from_numpy(idx), torch.from_numpy(cnt)


def paged_to_padded(pages, page_table, seqlens, capacity=None):
    """Gather a page pool [P, page, H, D] into the padded cache [B, capacity, H, D]
    the reference's decoding kernels index (flash_attn_decoding.py:62-69)."""
    P, page, H, D = pages.shape
    B = page_table.shape[0]
    cap = capacity or page_table.shape[1] * page
    out = torch.zeros(B, cap, H, D, dtype=pages.dtype)
    for b in range(B):
        n = max(int(seqlens[b]), 0)
        for i in range((n + page - 1) // page):
            t0 = i * page
            t1 = min(n, t0 + page)
            out[b, t0:t1] = pages[int(page_table[b, i]), :t1 - t0]
    return out


# --------------------------------------------------------------------------
# CPU-baseline forms of the block-index layouts: the reference's naive torch
# loops with the mask / gather of the block lists in place of its windows
# --------------------------------------------------------------------------
def block_sparse_prefill_refpath(q, k, v, cu_seqlens, block_idx, block_cnt, *, block=64, heads=None):
    """The dense masked per-(b, h) loop of flash_attn_sparse_torch
    (flash_attn_sparse_attn_triton.py:391-442) with the mask expanded from a block list instead
    of the two windows: scores, mask, scale and softmax all in the input dtype.  `heads` limits
    the loop to some (b, h) pairs (the CPU baseline times a stated subset)."""
    _, T, H, Dq = q.shape
    g = H // k.shape[-2]
    o = torch.zeros_like(q)
    softmax_scale = Dq ** -0.5
    for b, (s0, s1) in enumerate(_lens(cu_seqlens)):
        n = s1 - s0
        for h in range(H):
            if heads is not None and (b, h) not in heads:
                continue
            mask = block_list_mask(n, block, block_idx[b, h], block_cnt[b, h], True)
            bq, bk, bv = q[0, s0:s1, h], k[0, s0:s1, h // g], v[0, s0:s1, h // g]
            qk = bq @ bk.T
            qk = torch.where(mask, qk, torch.full_like(qk, -math.inf)) * softmax_scale
            o[0, s0:s1, h] = qk.softmax(dim=-1) @ bv
    return o


def block_sparse_decoding_refpath(q, k_cache, v_cache, block_idx, *, block=64):
    """Gather the listed blocks of each (b, KV head), then the math of the sparse
    flash_attn_decoding_torch (flash_attn_decoding_sparse.py:368-406) with every gathered key
    visible: scores, softmax and P V in the input dtype.  Lists are full (no -1 padding)."""
    B, Hq, D = q.shape
    Hkv = k_cache.shape[2]
    g = Hq // Hkv
    o = torch.zeros(B, Hq, v_cache.shape[3], dtype=q.dtype)
    qk_scale = D ** -0.5
    off = torch.arange(block)
    for b in range(B):
        for hk in range(Hkv):
            tok = (block_idx[b, hk].long()[:, None] * block + off[None, :]).reshape(-1)
            bk, bv = k_cache[b, tok, hk], v_cache[b, tok, hk]
            bq = q[b, hk * g:(hk + 1) * g]
            qk = torch.einsum("hd,kd->hk", bq, bk).to(q.dtype) * qk_scale
            o[b, hk * g:(hk + 1) * g] = torch.einsum("hk,kd->hd", qk.softmax(dim=-1).to(q.dtype), bv)
    return o
