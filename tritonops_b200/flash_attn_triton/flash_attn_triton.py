"""Dense causal varlen GQA prefill -- drop-in for the reference module
flash_attn_triton/flash_attn_triton.py (entry points :595-658 and :816-874)."""
import torch

from .. import ops

LOG2E = 1.4426950408889634


def flash_attn_triton_fwd(q, k, v, cu_seq_lens, sm_scale, causal=True, max_seqlen=None):
    """Same contract as the reference launcher (flash_attn_triton.py:595-658):
    q [1,T,Hq,D], k/v [1,T,Hkv,D], cu_seq_lens int32 [B+1]; ``sm_scale``
    already contains log2(e) (:839); returns (o, lse) with lse the base-2 LSE
    of the prescaled scores (:170,:180).  ``causal`` and ``max_seqlen`` are
    additions: the reference kernel is always causal, and it syncs with the
    host to find the longest sequence (:621) -- pass ``max_seqlen`` to avoid that."""
    return ops.prefill(q, k, v, cu_seqlens=cu_seq_lens, max_seqlen=max_seqlen, scale=sm_scale,
                       scale_has_log2e=True, causal=causal, lse_base2=True)


def flash_attn_triton_bwd(q, k, v, o, do, lse, cu_seq_lens, sm_scale, causal=True, max_seqlen=None):
    """Same contract as the reference launcher (flash_attn_triton.py:661-813):
    ``lse`` is the base-2 LSE the forward returned, ``sm_scale`` contains
    log2(e); returns (dq, dk, dv) with dk / dv already summed over the query
    heads of each GQA group (:813)."""
    return ops.prefill_bwd(q, k, v, o, do, lse, cu_seqlens=cu_seq_lens, max_seqlen=max_seqlen,
                           scale=sm_scale, scale_has_log2e=True, causal=causal, lse_base2=True)


class flash_attn_triton(torch.autograd.Function):
    """``flash_attn_triton.apply(q, k, v, cu_seq_lens) -> o`` as in the reference
    (flash_attn_triton.py:816-874), forward and backward."""

    @staticmethod
    def forward(ctx, q, k, v, cu_seq_lens):
        sm_scale = (1 / q.shape[-1]) ** 0.5 * LOG2E
        o, lse = flash_attn_triton_fwd(q, k, v, cu_seq_lens, sm_scale)
        ctx.save_for_backward(q, k, v, o, lse, cu_seq_lens)
        ctx.sm_scale = sm_scale
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse, cu_seq_lens = ctx.saved_tensors
        dq, dk, dv = flash_attn_triton_bwd(q, k, v, o, do, lse, cu_seq_lens, ctx.sm_scale)
        return dq, dk, dv, None


def flash_attention(q, k, v, cu_seq_lens=None, causal=True, softmax_scale=None,
                    return_lse=False, max_seqlen=None):
    """The name the reference README uses (README.md:31).  q [1,T,Hq,D] packed
    with ``cu_seq_lens``, or [B,S,Hq,D] fixed-length when ``cu_seq_lens`` is
    None.  ``softmax_scale`` is the natural scale (default D**-0.5); the
    returned LSE is the natural log-sum-exp, fp32 [.., tokens, Hq]."""
    o, lse = ops.prefill(q, k, v, cu_seqlens=cu_seq_lens, max_seqlen=max_seqlen,
                         scale=softmax_scale, scale_has_log2e=False, causal=causal,
                         lse_base2=False)
    return (o, lse) if return_lse else o
