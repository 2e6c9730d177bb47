"""Sparse decoding -- drop-in for the reference module
flash_attn_triton/flash_attn_decoding_sparse.py (:222-365), plus block-list decoding."""
from .. import ops


def flash_attention_sparse_decoding(q, k, v, cu_seq_lens, global_window_size=64,
                                    local_window_size=64):
    """The one query of sequence b sees key j iff j < global_window_size or
    j >= len_b - local_window_size (flash_attn_decoding_sparse.py:82-85).
    q [B,Hq,D]; k/v padded cache [B,Tmax,Hkv,D]; scale fixed to D**-0.5 (:246).
    Keeps the reference's restriction on the global window (:249-253)."""
    assert global_window_size in {64, 128, 256}, (
        f"global_window_size must be one of 64, 128, or 256, got {global_window_size}")
    return ops.decode(q, k, v, cu_seqlens=cu_seq_lens, sparsity=ops.WINDOW,
                      window_global=global_window_size, window_local=local_window_size)


def flash_attention_block_sparse_decoding(q, k, v, cu_seq_lens, block_idx, block_cnt=None,
                                          block_size=64, qk_scale=None):
    """Top-k block decoding (layout not present in the reference): block_idx
    int32 [B,Hkv,n_sel] ascending block numbers (-1 padded), optional block_cnt
    int32 [B,Hkv]; the query heads of a GQA group share their KV head's list."""
    return ops.decode(q, k, v, cu_seqlens=cu_seq_lens, scale=qk_scale, sparsity=ops.BLOCK_LIST,
                      block_idx=block_idx, block_cnt=block_cnt, block_size=block_size)
