"""Split-KV decoding over a padded KV cache -- drop-in for the reference module
flash_attn_triton/flash_attn_decoding.py (:213-336)."""
from .. import ops


def flash_attention_decoding(q, k, v, cu_seq_lens, qk_scale=None, max_seq_len=None):
    """q [B,Hq,D]; k/v padded cache [B,Tmax,Hkv,D]; ``cu_seq_lens`` int32 [B+1]
    is used for the lengths only (len_b = cu[b+1]-cu[b], flash_attn_decoding.py:46-48);
    ``qk_scale`` defaults to D**-0.5 (:236-237).  Returns [B,Hq,Dv].
    ``max_seq_len`` (an upper bound on the lengths) is optional; unlike the
    reference (:242) no host sync is needed without it."""
    return ops.decode(q, k, v, cu_seqlens=cu_seq_lens, scale=qk_scale, max_seqlen=max_seq_len)


flash_attn_decoding = flash_attention_decoding
