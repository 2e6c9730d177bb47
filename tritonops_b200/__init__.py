"""tritonops_b200 -- B200 (sm_100a) CUDA implementation of the flash_attn_triton
family of rookie-joe/TritonOps behind the same Python call signatures.

    from tritonops_b200.flash_attn_triton.flash_attn_triton import flash_attn_triton, flash_attention
    from tritonops_b200.flash_attn_triton.flash_attn_decoding import flash_attention_decoding
    from tritonops_b200.flash_attn_triton.flash_attn_sparse_attn_triton import flash_attn_sparse_triton
    from tritonops_b200.flash_attn_triton.flash_attn_decoding_sparse import flash_attention_sparse_decoding

All arithmetic runs in csrc/libb200attn.so (build: python -m tritonops_b200.build)."""
from . import _lib  # noqa: F401

__all__ = ["_lib"]
