"""Tensor-level entry points: torch custom ops ("b200attn::*") whose bodies unpack
the tensors into the C structs of include/b200attn.h and call the extern "C"
launchers on the current CUDA stream.  PyTorch only supplies device memory and
streams here; all arithmetic runs in libb200attn.so.  No CPU or eager fallback
exists: CPU tensors are rejected."""
import ctypes as C
import math
import os
import threading
from typing import Optional, Tuple

import torch
from torch import Tensor

from . import _lib
from ._lib import (BLOCK_LIST, DENSE, WINDOW, DecodeArgs, KvAppendArgs, KvPackArgs, PagedDecodeArgs,
                   PrefillArgs, PrefillBwdArgs, RmsNormBwdArgs, RmsNormFwdArgs, TopkBlocksArgs,
                   WindowBlocksDecodeArgs, WindowBlocksPrefillArgs)

LOG2E = 1.4426950408889634
_DT = {torch.float16: _lib.F16, torch.bfloat16: _lib.BF16}

# kernels launched through this module since import (bench accounting)
launch_counter = 0


# Debug mode (B200ATTN_DEBUG_STATUS=1): the prefill and decoding kernels get a status word and
# every call is followed by a stream synchronisation and a check of it, so a bounded device-side
# wait that gave up surfaces as an exception at the call that caused it.  Off by default (it costs
# a host sync).
DEBUG_STATUS = os.environ.get("B200ATTN_DEBUG_STATUS", "0") == "1"
_status_words = {}
_status_lock = threading.Lock()


def _status_word(dev) -> Tensor:
    key = torch.device(dev).index
    if key is None:
        key = torch.cuda.current_device()
    with _status_lock:      # calls may come from several host threads
        if key not in _status_words:
            _status_words[key] = torch.zeros(1, device=torch.device("cuda", key), dtype=torch.int32)
        return _status_words[key]


def _same_head_dim(q: Tensor, *others: Tensor):
    """One head_dim for Q, K, V (and O): the kernels take a single value.  The reference wrappers
    accept a narrower V (flash_attn_decoding.py:233-236) but allocate O with Q's width
    (flash_attn_triton.py:608), so only equal widths ever worked there either."""
    for t in others:
        if t.shape[-1] != q.shape[-1]:
            raise ValueError(f"b200attn: q, k and v must share head_dim (got {q.shape[-1]} and {t.shape[-1]})")


def _check_status(dev, what: str):
    if not DEBUG_STATUS:
        return
    w = _status_word(dev)
    torch.cuda.current_stream(dev).synchronize()
    if int(w.item()) != 0:
        w.zero_()
        raise RuntimeError(f"b200attn: a bounded device-side wait gave up inside {what}; its results are invalid")


def selftest_bounded_wait(budget_cycles: int = 2_000_000, device="cuda") -> Tuple[int, int]:
    """Run the library's wait-that-nothing-completes probe: (status word, cycles waited)."""
    dev = torch.device(device)
    if dev.type != "cuda":
        raise RuntimeError("b200attn ops take CUDA tensors only (there is no CPU path)")
    st = torch.zeros(1, device=dev, dtype=torch.int32)
    waited = torch.zeros(1, device=dev, dtype=torch.int64)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().b200attn_selftest_bounded_wait(_ptr(st), int(budget_cycles), _ptr(waited), _stream(st)))
    _count()
    return int(st.item()), int(waited.item())


def _count():
    global launch_counter
    launch_counter += _lib.lib().b200attn_last_launch_count()


def _stream(t: Tensor):
    return C.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("b200attn ops take CUDA tensors only (there is no CPU path)")


def _rowmajor16(t: Tensor) -> Tensor:
    """Keep arbitrary outer strides (the reference passes all strides through,
    flash_attn_triton.py:633-646) but require unit inner stride and 16-byte
    addressable rows; copy otherwise."""
    ok = t.stride(-1) == 1 and t.data_ptr() % 16 == 0 and all(s % 8 == 0 for s in t.stride()[:-1])
    return t if ok else t.contiguous()


def _ptr(t: Optional[Tensor]):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def _i32(t: Optional[Tensor], dev) -> Optional[Tensor]:
    if t is None:
        return None
    return t.to(device=dev, dtype=torch.int32).contiguous()


# --------------------------------------------------------------------------
# decoding
# --------------------------------------------------------------------------
def decode_workspace_bytes(batch, heads_q, heads_kv, head_dim, max_seqlen, chunk=0) -> int:
    """Scratch bytes dense decoding needs for this shape (the split size, when 0, depends on all of them)."""
    a = DecodeArgs(batch=batch, heads_q=heads_q, heads_kv=heads_kv, head_dim=head_dim,
                   max_seqlen=max_seqlen, chunk_tokens=chunk, sparsity=DENSE)
    return _lib.lib().b200attn_decode_workspace_bytes(C.byref(a))


def _decode_op_impl(q: Tensor, k: Tensor, v: Tensor, lens: Tensor, lens_are_cu: bool, max_seqlen: int,
               scale: float, chunk: int, sparsity: int, window_global: int, window_local: int,
               block_idx: Optional[Tensor], block_cnt: Optional[Tensor],
               block_size: int) -> Tensor:
    _same_head_dim(q, k, v)
    _need_cuda(q, k, v, lens, block_idx, block_cnt)
    if q.dtype not in _DT or k.dtype != q.dtype or v.dtype != q.dtype:
        raise ValueError("b200attn: q, k, v must share dtype float16 or bfloat16")
    q, k, v = _rowmajor16(q), _rowmajor16(k), _rowmajor16(v)
    B, Hq, D = q.shape
    Hkv = k.shape[2]
    o = torch.empty(B, Hq, v.shape[3], device=q.device, dtype=q.dtype)
    a = DecodeArgs()
    a.q, a.k_cache, a.v_cache, a.o = _ptr(q), _ptr(k), _ptr(v), _ptr(o)
    a.dtype, a.batch, a.heads_q, a.heads_kv, a.head_dim = _DT[q.dtype], B, Hq, Hkv, D
    a.max_seqlen = min(max_seqlen, k.shape[1])
    if lens_are_cu:
        a.cu_seqlens = _ptr(lens)
    else:
        a.seqlens = _ptr(lens)
    a.q_stride_b, a.q_stride_h = q.stride(0), q.stride(1)
    a.k_stride_b, a.k_stride_t, a.k_stride_h = k.stride(0), k.stride(1), k.stride(2)
    a.v_stride_b, a.v_stride_t, a.v_stride_h = v.stride(0), v.stride(1), v.stride(2)
    a.o_stride_b, a.o_stride_h = o.stride(0), o.stride(1)
    a.softmax_scale, a.chunk_tokens, a.sparsity = scale, chunk, sparsity
    a.window_global, a.window_local = window_global, window_local
    if block_idx is not None:
        a.block_idx, a.block_cnt = _ptr(block_idx), _ptr(block_cnt)
        a.block_size, a.max_sel = block_size, block_idx.shape[-1]
    L = _lib.lib()
    need = L.b200attn_decode_workspace_bytes(C.byref(a))
    ws = torch.empty(max(need, 16), device=q.device, dtype=torch.uint8)
    a.workspace, a.workspace_bytes = _ptr(ws), ws.numel()
    fn = L.b200attn_decode_fwd if sparsity == DENSE else L.b200attn_sparse_decode_fwd
    with torch.cuda.device(q.device):
        if DEBUG_STATUS:
            a.status_word = _ptr(_status_word(q.device))
        _lib.check(fn(C.byref(a), _stream(q)))
        _check_status(q.device, "decoding")
    _count()
    return o


_decode_op = torch.library.custom_op("b200attn::decode_fwd", _decode_op_impl, mutates_args=())


@_decode_op.register_fake
def _(q, k, v, lens, lens_are_cu, max_seqlen, scale, chunk, sparsity, window_global,
      window_local, block_idx, block_cnt, block_size):
    return q.new_empty(q.shape[0], q.shape[1], v.shape[3])


def decode(q, k_cache, v_cache, *, cu_seqlens=None, seqlens=None, max_seqlen=None, scale=None,
           chunk=0, sparsity=DENSE, window_global=0, window_local=0, block_idx=None,
           block_cnt=None, block_size=64) -> Tensor:
    """Split-KV GQA decoding; see b200attn_decode_fwd in include/b200attn.h."""
    if (cu_seqlens is None) == (seqlens is None):
        raise ValueError("give exactly one of cu_seqlens and seqlens")
    lens = _i32(cu_seqlens if cu_seqlens is not None else seqlens, q.device)
    if scale is None:
        scale = q.shape[-1] ** -0.5
    if max_seqlen is None:
        max_seqlen = k_cache.shape[1]
    fn = _decode_op if torch.compiler.is_compiling() else _decode_op_impl   # eager: skip the dispatcher
    return fn(q, k_cache, v_cache, lens, cu_seqlens is not None, int(max_seqlen),
                      float(scale), int(chunk), int(sparsity), int(window_global),
                      int(window_local), _i32(block_idx, q.device), _i32(block_cnt, q.device),
                      int(block_size))


def paged_decode(q: Tensor, k_pages: Tensor, v_pages: Tensor, page_table: Tensor, seqlens: Tensor, *,
                 max_seqlen: Optional[int] = None, scale: Optional[float] = None, chunk: int = 0) -> Tensor:
    """Split-KV GQA decoding over page pools [num_pages, page_size, Hkv, D] addressed through
    page_table int32 [B, max_pages]; see b200attn_paged_decode_fwd in include/b200attn.h."""
    _same_head_dim(q, k_pages, v_pages)
    _need_cuda(q, k_pages, v_pages, page_table, seqlens)
    if q.dtype not in _DT or k_pages.dtype != q.dtype or v_pages.dtype != q.dtype:
        raise ValueError("b200attn: q, k, v must share dtype float16 or bfloat16")
    q, k, v = _rowmajor16(q), _rowmajor16(k_pages), _rowmajor16(v_pages)
    table, sl = _i32(page_table, q.device), _i32(seqlens, q.device)
    B, Hq, D = q.shape
    P, page, Hkv, _ = k.shape
    o = torch.empty(B, Hq, v.shape[3], device=q.device, dtype=q.dtype)
    a = PagedDecodeArgs()
    a.q, a.k_pages, a.v_pages, a.o = _ptr(q), _ptr(k), _ptr(v), _ptr(o)
    a.dtype, a.batch, a.heads_q, a.heads_kv, a.head_dim = _DT[q.dtype], B, Hq, Hkv, D
    a.page_size, a.num_pages, a.max_pages_per_seq = page, P, table.shape[1]
    a.max_seqlen = int(max_seqlen) if max_seqlen is not None else table.shape[1] * page
    a.page_table, a.seqlens = _ptr(table), _ptr(sl)
    a.q_stride_b, a.q_stride_h = q.stride(0), q.stride(1)
    a.k_stride_page, a.k_stride_t, a.k_stride_h = k.stride(0), k.stride(1), k.stride(2)
    a.v_stride_page, a.v_stride_t, a.v_stride_h = v.stride(0), v.stride(1), v.stride(2)
    a.o_stride_b, a.o_stride_h = o.stride(0), o.stride(1)
    a.softmax_scale = float(scale) if scale is not None else D ** -0.5
    a.chunk_tokens = int(chunk)
    L = _lib.lib()
    need = L.b200attn_paged_decode_workspace_bytes(C.byref(a))
    ws = torch.empty(max(need, 16), device=q.device, dtype=torch.uint8)
    a.workspace, a.workspace_bytes = _ptr(ws), ws.numel()
    with torch.cuda.device(q.device):
        if DEBUG_STATUS:
            a.status_word = _ptr(_status_word(q.device))
        _lib.check(L.b200attn_paged_decode_fwd(C.byref(a), _stream(q)))
        _check_status(q.device, "paged decoding")
    _count()
    return o


# --------------------------------------------------------------------------
# block selection (builders of the BLOCK_LIST inputs)
# --------------------------------------------------------------------------
def window_blocks_prefill(batch: int, heads: int, n_qblocks: int, window_local: int, window_global: int,
                          *, block_size: int = 64, device="cuda") -> Tuple[Tensor, Tensor]:
    """(block_idx [B, H, n_qblocks, max_nnz], block_cnt [B, H, n_qblocks]): the block cover of the
    window pattern, in the layout prefill(sparsity=BLOCK_LIST) takes."""
    dev = torch.device(device)
    if dev.type != "cuda":
        raise RuntimeError("b200attn ops take CUDA tensors only (there is no CPU path)")
    L = _lib.lib()
    nnz = max(1, L.b200attn_window_blocks_prefill_max_nnz(block_size, window_local, window_global, n_qblocks))
    idx = torch.empty(batch, heads, n_qblocks, nnz, device=dev, dtype=torch.int32)
    cnt = torch.empty(batch, heads, n_qblocks, device=dev, dtype=torch.int32)
    a = WindowBlocksPrefillArgs(_ptr(idx), _ptr(cnt), batch, heads, n_qblocks, nnz, block_size,
                                window_local, window_global)
    with torch.cuda.device(dev):
        _lib.check(L.b200attn_window_blocks_prefill(C.byref(a), _stream(idx)))
    _count()
    return idx, cnt


def window_blocks_decode(seqlens: Tensor, heads_kv: int, window_local: int, window_global: int, *,
                         block_size: int = 64, max_sel: Optional[int] = None) -> Tuple[Tensor, Tensor]:
    """(block_idx [B, Hkv, max_sel], block_cnt [B, Hkv]): the blocks holding the sink and recent
    keys of each sequence, in the layout decode(sparsity=BLOCK_LIST) takes."""
    _need_cuda(seqlens)
    sl = _i32(seqlens, seqlens.device)
    B = sl.numel()
    if max_sel is None:
        max_sel = (window_global + block_size - 1) // block_size + (window_local + block_size - 2) // block_size + 1
    max_sel = max(1, int(max_sel))
    idx = torch.empty(B, heads_kv, max_sel, device=sl.device, dtype=torch.int32)
    cnt = torch.empty(B, heads_kv, device=sl.device, dtype=torch.int32)
    a = WindowBlocksDecodeArgs(_ptr(idx), _ptr(cnt), None, _ptr(sl), B, heads_kv, max_sel, block_size,
                               window_local, window_global)
    with torch.cuda.device(sl.device):
        _lib.check(_lib.lib().b200attn_window_blocks_decode(C.byref(a), _stream(sl)))
    _count()
    return idx, cnt


def topk_blocks(scores: Tensor, top_k: int, *, n_valid: Optional[Tensor] = None, force_first: int = 0,
                force_last: int = 0) -> Tuple[Tensor, Tensor]:
    """Per row of fp32 `scores` [..., n_blocks]: the top_k best candidate blocks in ascending block
    order, (block_idx [..., top_k] padded with -1, block_cnt [...])."""
    _need_cuda(scores, n_valid)
    if scores.dtype != torch.float32:
        raise ValueError("b200attn: block scores must be float32")
    lead = scores.shape[:-1]
    s2 = scores.reshape(-1, scores.shape[-1])
    if s2.stride(-1) != 1:
        s2 = s2.contiguous()
    rows, n = s2.shape
    nv = _i32(n_valid, scores.device)
    if nv is not None and nv.numel() != rows:
        raise ValueError("b200attn: n_valid needs one entry per row of scores")
    idx = torch.empty(rows, top_k, device=scores.device, dtype=torch.int32)
    cnt = torch.empty(rows, device=scores.device, dtype=torch.int32)
    a = TopkBlocksArgs(_ptr(s2), s2.stride(0), _ptr(nv), rows, n, top_k, force_first, force_last,
                       _ptr(idx), _ptr(cnt))
    with torch.cuda.device(scores.device):
        _lib.check(_lib.lib().b200attn_topk_blocks(C.byref(a), _stream(scores)))
    _count()
    return idx.reshape(*lead, top_k), cnt.reshape(lead)


# --------------------------------------------------------------------------
# prefill
# --------------------------------------------------------------------------
def _prefill_op_impl(q: Tensor, k: Tensor, v: Tensor, cu_seqlens: Optional[Tensor], max_seqlen: int,
                scale: float, scale_has_log2e: bool, causal: bool, lse_base2: bool, sparsity: int,
                window_local: int, window_global: int, block_idx: Optional[Tensor],
                block_cnt: Optional[Tensor], block_size: int) -> Tuple[Tensor, Tensor]:
    _same_head_dim(q, k, v)
    _need_cuda(q, k, v, cu_seqlens, block_idx, block_cnt)
    if q.dtype not in _DT or k.dtype != q.dtype or v.dtype != q.dtype:
        raise ValueError("b200attn: q, k, v must share dtype float16 or bfloat16")
    q, k, v = _rowmajor16(q), _rowmajor16(k), _rowmajor16(v)
    Bt, T, Hq, D = q.shape
    Hkv = k.shape[2]
    o = torch.empty(Bt, T, Hq, v.shape[3], device=q.device, dtype=q.dtype)
    lse = torch.empty(Bt, T, Hq, device=q.device, dtype=torch.float32)
    a = _prefill_args(q, k, v, o, lse, cu_seqlens, max_seqlen, scale, scale_has_log2e, causal, lse_base2,
                      sparsity, window_local, window_global, block_idx, block_cnt, block_size)
    L = _lib.lib()
    fn = L.b200attn_prefill_fwd if sparsity == DENSE else L.b200attn_sparse_prefill_fwd
    with torch.cuda.device(q.device):
        _lib.check(fn(C.byref(a), _stream(q)))
        _check_status(q.device, "the prefill forward")
    _count()
    return o, lse


def _prefill_args(q, k, v, o, lse, cu_seqlens, max_seqlen, scale, scale_has_log2e, causal, lse_base2,
                  sparsity=DENSE, window_local=0, window_global=0, block_idx=None, block_cnt=None,
                  block_size=64) -> "PrefillArgs":
    """b200attn_prefill_args for row-major tensors that have been checked by the caller."""
    Bt, T, Hq, D = q.shape
    Hkv = k.shape[2]
    a = PrefillArgs()
    a.q, a.k, a.v, a.o, a.lse = _ptr(q), _ptr(k), _ptr(v), _ptr(o), _ptr(lse)
    a.dtype, a.heads_q, a.heads_kv, a.head_dim = _DT[q.dtype], Hq, Hkv, D
    if cu_seqlens is not None:
        a.batch, a.cu_seqlens = cu_seqlens.numel() - 1, _ptr(cu_seqlens)
        a.max_seqlen, a.total_tokens, a.seqlen = max_seqlen, Bt * T if Bt == 1 else T, 0
        if Bt != 1:
            raise ValueError("packed varlen tensors must have a leading dimension of 1")
    else:
        a.batch, a.seqlen, a.max_seqlen, a.total_tokens = Bt, T, T, T
    a.q_stride_b, a.q_stride_t, a.q_stride_h = q.stride(0), q.stride(1), q.stride(2)
    a.k_stride_b, a.k_stride_t, a.k_stride_h = k.stride(0), k.stride(1), k.stride(2)
    a.v_stride_b, a.v_stride_t, a.v_stride_h = v.stride(0), v.stride(1), v.stride(2)
    a.o_stride_b, a.o_stride_t, a.o_stride_h = o.stride(0), o.stride(1), o.stride(2)
    a.lse_stride_b, a.lse_stride_t, a.lse_stride_h = lse.stride(0), lse.stride(1), lse.stride(2)
    a.softmax_scale, a.scale_has_log2e = scale, int(scale_has_log2e)
    a.causal, a.lse_base2, a.sparsity = int(causal), int(lse_base2), sparsity
    a.window_local, a.window_global = window_local, window_global
    if block_idx is not None:
        a.block_idx, a.block_cnt, a.block_size = _ptr(block_idx), _ptr(block_cnt), block_size
        a.n_qblocks, a.max_nnz = block_idx.shape[2], block_idx.shape[3]
    if DEBUG_STATUS:
        a.status_word = _ptr(_status_word(q.device))
    return a


def prefill_rows(q, k, v, o, lse, row_begin: int, row_end: int, *, scale=None, scale_has_log2e=False,
                 causal=True, lse_base2=False) -> None:
    """Dense prefill of the query rows [row_begin, row_end) only, written into the caller's
    `o` [Bt, T, Hq, D] and `lse` fp32 [Bt, T, Hq]; see b200attn_prefill_fwd_rows in
    include/b200attn.h.  q, k, v [Bt, T, H, D] with rows that are multiples of 8 elements apart;
    with causal=True no K / V row at or beyond row_end is read."""
    _same_head_dim(q, k, v, o)
    _need_cuda(q, k, v, o, lse)
    if q.dtype not in _DT or k.dtype != q.dtype or v.dtype != q.dtype or o.dtype != q.dtype:
        raise ValueError("b200attn: q, k, v, o must share dtype float16 or bfloat16")
    if lse.dtype != torch.float32 or tuple(lse.shape) != tuple(q.shape[:3]) or tuple(o.shape) != tuple(q.shape):
        raise ValueError("b200attn: o must have q's shape and lse must be float32 [Bt, T, Hq]")
    for t in (q, k, v, o):
        if t.stride(3) != 1 or any(st % 8 for st in t.stride()[:3]):
            raise ValueError("b200attn: prefill_rows takes row-major tensors with strides that are multiples of 8")
    if scale is None:
        scale, scale_has_log2e = q.shape[-1] ** -0.5, False
    a = _prefill_args(q, k, v, o, lse, None, q.shape[1], float(scale), bool(scale_has_log2e), bool(causal),
                      bool(lse_base2))
    L = _lib.lib()
    with torch.cuda.device(q.device):
        _lib.check(L.b200attn_prefill_fwd_rows(C.byref(a), int(row_begin), int(row_end), _stream(q)))
        _check_status(q.device, "the prefill forward")
    _count()


_prefill_op = torch.library.custom_op("b200attn::prefill_fwd", _prefill_op_impl, mutates_args=())


@_prefill_op.register_fake
def _(q, k, v, cu_seqlens, max_seqlen, scale, scale_has_log2e, causal, lse_base2, sparsity,
      window_local, window_global, block_idx, block_cnt, block_size):
    return (q.new_empty(*q.shape[:3], v.shape[3]),
            q.new_empty(q.shape[:3], dtype=torch.float32))


def prefill(q, k, v, *, cu_seqlens=None, max_seqlen=None, scale=None, scale_has_log2e=False,
            causal=True, lse_base2=False, sparsity=DENSE, window_local=0, window_global=0,
            block_idx=None, block_cnt=None, block_size=64) -> Tuple[Tensor, Tensor]:
    """Prefill attention forward -> (o, lse); see b200attn_prefill_fwd in include/b200attn.h.

    q [Bt, T, Hq, D]; with cu_seqlens the tensors are packed ([1, total, H, D])."""
    cu = _i32(cu_seqlens, q.device)
    if scale is None:
        scale, scale_has_log2e = q.shape[-1] ** -0.5, False
    if max_seqlen is None:
        if cu is not None:
            # the one host sync of the reference wrapper (flash_attn_triton.py:621);
            # pass max_seqlen to avoid it
            max_seqlen = int((cu[1:] - cu[:-1]).max().item()) if cu.numel() > 1 else 0
        else:
            max_seqlen = q.shape[1]
    fn = _prefill_op if torch.compiler.is_compiling() else _prefill_op_impl   # eager: skip the dispatcher
    return fn(q, k, v, cu, int(max_seqlen), float(scale), bool(scale_has_log2e),
                       bool(causal), bool(lse_base2), int(sparsity), int(window_local),
                       int(window_global), _i32(block_idx, q.device), _i32(block_cnt, q.device),
                       int(block_size))


# --------------------------------------------------------------------------
# prefill backward
# --------------------------------------------------------------------------
def _prefill_bwd_op_impl(q: Tensor, k: Tensor, v: Tensor, o: Tensor, d_o: Tensor, lse: Tensor,
                    cu_seqlens: Optional[Tensor], max_seqlen: int, scale: float,
                    scale_has_log2e: bool, causal: bool, lse_base2: bool) -> Tuple[Tensor, Tensor, Tensor]:
    _same_head_dim(q, k, v, o, d_o)
    _need_cuda(q, k, v, o, d_o, lse, cu_seqlens)
    if q.dtype not in _DT or any(t.dtype != q.dtype for t in (k, v, o, d_o)):
        raise ValueError("b200attn: q, k, v, o, do must share dtype float16 or bfloat16")
    q, k, v, o, d_o = (_rowmajor16(t) for t in (q, k, v, o, d_o))
    lse = lse.contiguous() if lse.dtype == torch.float32 else lse.float().contiguous()
    Bt, T, Hq, D = q.shape
    Hkv = k.shape[2]
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    dq, dk, dv = dq.contiguous(), dk.contiguous(), dv.contiguous()
    a = PrefillBwdArgs()
    a.q, a.k, a.v, a.o, a.d_o, a.lse = _ptr(q), _ptr(k), _ptr(v), _ptr(o), _ptr(d_o), _ptr(lse)
    a.dq, a.dk, a.dv = _ptr(dq), _ptr(dk), _ptr(dv)
    a.dtype, a.heads_q, a.heads_kv, a.head_dim = _DT[q.dtype], Hq, Hkv, D
    if cu_seqlens is not None:
        if Bt != 1:
            raise ValueError("packed varlen tensors must have a leading dimension of 1")
        a.batch, a.cu_seqlens = cu_seqlens.numel() - 1, _ptr(cu_seqlens)
        a.max_seqlen, a.total_tokens, a.seqlen = max_seqlen, T, 0
    else:
        a.batch, a.seqlen, a.max_seqlen, a.total_tokens = Bt, T, T, T
    for name, t in (("q", q), ("k", k), ("v", v), ("o", o), ("do", d_o), ("dq", dq), ("dk", dk),
                    ("dv", dv), ("lse", lse)):
        setattr(a, f"{name}_stride_b", t.stride(0))
        setattr(a, f"{name}_stride_t", t.stride(1))
        setattr(a, f"{name}_stride_h", t.stride(2))
    a.softmax_scale, a.scale_has_log2e = scale, int(scale_has_log2e)
    a.causal, a.lse_base2 = int(causal), int(lse_base2)
    L = _lib.lib()
    need = L.b200attn_prefill_bwd_workspace_bytes(C.byref(a))
    ws = torch.empty(max(need, 16), device=q.device, dtype=torch.uint8)
    a.workspace, a.workspace_bytes = _ptr(ws), ws.numel()
    with torch.cuda.device(q.device):
        if DEBUG_STATUS:
            a.status_word = _ptr(_status_word(q.device))
        _lib.check(L.b200attn_prefill_bwd(C.byref(a), _stream(q)))
        _check_status(q.device, "the prefill backward")
    _count()
    return dq, dk, dv


_prefill_bwd_op = torch.library.custom_op("b200attn::prefill_bwd", _prefill_bwd_op_impl, mutates_args=())


@_prefill_bwd_op.register_fake
def _(q, k, v, o, d_o, lse, cu_seqlens, max_seqlen, scale, scale_has_log2e, causal, lse_base2):
    return torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)


def prefill_bwd(q, k, v, o, d_o, lse, *, cu_seqlens=None, max_seqlen=None, scale=None,
                scale_has_log2e=False, causal=True, lse_base2=False):
    """Gradients (dq, dk, dv) of the dense prefill; see b200attn_prefill_bwd in include/b200attn.h.
    `o`, `lse` are the forward's outputs (lse in the form given by `lse_base2`)."""
    cu = _i32(cu_seqlens, q.device)
    if scale is None:
        scale, scale_has_log2e = q.shape[-1] ** -0.5, False
    if max_seqlen is None:
        if cu is not None:
            max_seqlen = int((cu[1:] - cu[:-1]).max().item()) if cu.numel() > 1 else 0
        else:
            max_seqlen = q.shape[1]
    fn = _prefill_bwd_op if torch.compiler.is_compiling() else _prefill_bwd_op_impl
    return fn(q, k, v, o, d_o, lse, cu, int(max_seqlen), float(scale),
                           bool(scale_has_log2e), bool(causal), bool(lse_base2))


# --------------------------------------------------------------------------
# KV-cache glue
# --------------------------------------------------------------------------
def pack_kv_cache(packed: Tensor, cu_seqlens: Tensor, capacity: int, out: Optional[Tensor] = None,
                  zero_pad: bool = True) -> Tensor:
    """Packed rows [1, T, H, D] (or [T, H, D]) -> padded cache [B, capacity, H, D], the copy
    the reference's decoding tests do in Python (flash_attn_decoding.py:404-425)."""
    _need_cuda(packed, cu_seqlens, out)
    if packed.dtype not in _DT:
        raise ValueError("b200attn: packed rows must be float16 or bfloat16")
    if packed.dim() == 4:
        packed = packed[0]
    packed = _rowmajor16(packed)
    cu = _i32(cu_seqlens, packed.device)
    B, (T, H, D) = cu.numel() - 1, packed.shape
    if out is None:
        out = torch.empty(B, capacity, H, D, device=packed.device, dtype=packed.dtype)
    a = KvPackArgs()
    a.packed, a.cache, a.cu_seqlens = _ptr(packed), _ptr(out), _ptr(cu)
    a.batch, a.heads, a.head_dim, a.capacity = B, H, D, out.shape[1]
    a.packed_stride_t, a.packed_stride_h = packed.stride(0), packed.stride(1)
    a.cache_stride_b, a.cache_stride_t, a.cache_stride_h = out.stride(0), out.stride(1), out.stride(2)
    a.zero_pad = int(zero_pad)
    with torch.cuda.device(packed.device):
        _lib.check(_lib.lib().b200attn_kv_pack_to_cache(C.byref(a), _stream(packed)))
    _count()
    return out


def append_kv(k_cache: Tensor, v_cache: Tensor, new_k: Tensor, new_v: Tensor, seqlens: Tensor) -> None:
    """In place: cache[b, seqlens[b]] = new[b] for K and V (one decoding step)."""
    _need_cuda(k_cache, v_cache, new_k, new_v, seqlens)
    if k_cache.stride() != v_cache.stride() or new_k.stride() != new_v.stride():
        raise ValueError("b200attn: K and V caches (and new rows) must share their strides")
    sl = _i32(seqlens, k_cache.device)
    B, cap, H, D = k_cache.shape
    a = KvAppendArgs()
    a.new_k, a.new_v, a.k_cache, a.v_cache, a.seqlens = _ptr(new_k), _ptr(new_v), _ptr(k_cache), _ptr(v_cache), _ptr(sl)
    a.batch, a.heads, a.head_dim, a.capacity = B, H, D, cap
    a.new_stride_b, a.new_stride_h = new_k.stride(0), new_k.stride(1)
    a.cache_stride_b, a.cache_stride_t, a.cache_stride_h = k_cache.stride(0), k_cache.stride(1), k_cache.stride(2)
    with torch.cuda.device(k_cache.device):
        _lib.check(_lib.lib().b200attn_kv_append(C.byref(a), _stream(k_cache)))
    _count()


# --------------------------------------------------------------------------
# RMSNorm
# --------------------------------------------------------------------------
_DT_RMS = {torch.float16: _lib.F16, torch.bfloat16: _lib.BF16, torch.float32: _lib.F32}


def _rows_view(t: Tensor) -> Tensor:
    """[..., D] -> [rows, D] with unit inner stride (copies only if it has to)."""
    t2 = t.reshape(-1, t.shape[-1])
    return t2 if t2.stride(-1) == 1 else t2.contiguous()


def _rms_dtypes(x: Tensor, weight: Tensor):
    if x.dtype not in _DT_RMS or (weight.dtype != x.dtype and weight.dtype != torch.float32):
        raise ValueError("b200attn: rmsnorm takes float16 / bfloat16 / float32 rows and weights of that dtype or float32")
    return _DT_RMS[x.dtype], _DT_RMS[weight.dtype]


def rmsnorm_fwd(x: Tensor, weight: Tensor, eps: float) -> Tuple[Tensor, Tensor]:
    """(y like x, rstd fp32 [rows]); see b200attn_rmsnorm_fwd in include/b200attn.h."""
    _need_cuda(x, weight)
    xd, wd = _rms_dtypes(x, weight)
    x2, w = _rows_view(x), weight.contiguous()
    if w.numel() != x2.shape[1]:
        raise ValueError(f"b200attn: expected weight dim {x2.shape[1]}, got {w.numel()}")
    y = torch.empty_like(x2, memory_format=torch.contiguous_format)
    rstd = torch.empty(x2.shape[0], device=x.device, dtype=torch.float32)
    if x2.shape[0] == 0:
        return y.view(x.shape), rstd
    a = RmsNormFwdArgs(_ptr(x2), _ptr(w), _ptr(y), _ptr(rstd), xd, wd, x2.shape[0], x2.shape[1],
                       x2.stride(0), y.stride(0), float(eps))
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().b200attn_rmsnorm_fwd(C.byref(a), _stream(x)))
    _count()
    return y.view(x.shape), rstd


def rmsnorm_bwd(dy: Tensor, x: Tensor, weight: Tensor, rstd: Tensor) -> Tuple[Tensor, Tensor]:
    """(dx like x, dweight like weight); see b200attn_rmsnorm_bwd in include/b200attn.h."""
    _need_cuda(dy, x, weight, rstd)
    xd, wd = _rms_dtypes(x, weight)
    if dy.dtype != x.dtype:
        dy = dy.to(x.dtype)
    x2, g2, w = _rows_view(x), _rows_view(dy), weight.contiguous()
    dx = torch.empty_like(x2, memory_format=torch.contiguous_format)
    dw = torch.empty_like(w)
    if x2.shape[0] == 0:
        return dx.view(x.shape), dw.zero_()
    a = RmsNormBwdArgs(_ptr(g2), _ptr(x2), _ptr(w), _ptr(rstd), _ptr(dx), _ptr(dw), xd, wd, x2.shape[0],
                       x2.shape[1], g2.stride(0), x2.stride(0), dx.stride(0), None, 0)
    L = _lib.lib()
    ws = torch.empty(max(L.b200attn_rmsnorm_bwd_workspace_bytes(C.byref(a)), 16), device=x.device, dtype=torch.uint8)
    a.workspace, a.workspace_bytes = _ptr(ws), ws.numel()
    with torch.cuda.device(x.device):
        _lib.check(L.b200attn_rmsnorm_bwd(C.byref(a), _stream(x)))
    _count()
    return dx.view(x.shape), dw
