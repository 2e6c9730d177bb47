"""Sparse causal prefill -- drop-in for the reference module
flash_attn_triton/flash_attn_sparse_attn_triton.py, plus the block-index layout."""
from .. import ops

LOG2E = 1.4426950408889634


def flash_attn_sparse_triton_fwd(q, k, v, cu_seqlens, softmax_scale=None, local_window_size=0,
                                 global_window_size=0, max_seqlen=None):
    """Positional order of the reference launcher body
    (flash_attn_sparse_attn_triton.py:237-245).  Query i sees key j iff j <= i and
    (i - j < local_window_size or j < global_window_size) -- the mask of the
    module's torch function (:422-433).  ``softmax_scale`` must already contain
    log2(e) as in the reference (default D**-0.5 * log2e, :266-267).  Returns
    (o, base-2 lse)."""
    if softmax_scale is None:
        softmax_scale = (1 / q.shape[-1]) ** 0.5 * LOG2E
    return ops.prefill(q, k, v, cu_seqlens=cu_seqlens, max_seqlen=max_seqlen, scale=softmax_scale,
                       scale_has_log2e=True, causal=True, lse_base2=True, sparsity=ops.WINDOW,
                       window_local=local_window_size, window_global=global_window_size)


def flash_attn_sparse_triton(q, k, v, cu_seqlens, local_window_size, global_window_size):
    """The call the reference's own test makes (flash_attn_sparse_attn_triton.py:480-482)."""
    return flash_attn_sparse_triton_fwd(q, k, v, cu_seqlens, None, local_window_size,
                                        global_window_size)


def flash_attn_block_sparse(q, k, v, cu_seqlens, block_idx, block_cnt, block_size=64,
                            softmax_scale=None, causal=True, max_seqlen=None):
    """Block-list sparse prefill (layout not present in the reference).
    block_idx int32 [B,Hq,n_qblocks,max_nnz]: ascending KV-block numbers
    (relative to the sequence) each query block attends to, -1 padded;
    block_cnt int32 [B,Hq,n_qblocks].  The element-wise causal mask applies
    inside blocks.  ``softmax_scale`` is the natural scale.  Returns
    (o, natural-log lse)."""
    return ops.prefill(q, k, v, cu_seqlens=cu_seqlens, max_seqlen=max_seqlen, scale=softmax_scale,
                       scale_has_log2e=False, causal=causal, lse_base2=False,
                       sparsity=ops.BLOCK_LIST, block_idx=block_idx, block_cnt=block_cnt,
                       block_size=block_size)
