"""ctypes binding of libb200attn.so (the C ABI declared in include/b200attn.h).

There is no fallback: if the shared library is missing or a call fails, the
Python layer raises."""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "csrc", "libb200attn.so")

F16, BF16, F32 = 0, 1, 2
DENSE, WINDOW, BLOCK_LIST = 0, 1, 2

i32, i64, f32, vp = C.c_int32, C.c_int64, C.c_float, C.c_void_p


class PrefillArgs(C.Structure):
    _fields_ = [
        ("q", vp), ("k", vp), ("v", vp), ("o", vp), ("lse", vp),
        ("dtype", i32), ("batch", i32), ("heads_q", i32), ("heads_kv", i32), ("head_dim", i32),
        ("seqlen", i32), ("max_seqlen", i32), ("total_tokens", i64), ("cu_seqlens", vp),
        ("q_stride_b", i64), ("q_stride_t", i64), ("q_stride_h", i64),
        ("k_stride_b", i64), ("k_stride_t", i64), ("k_stride_h", i64),
        ("v_stride_b", i64), ("v_stride_t", i64), ("v_stride_h", i64),
        ("o_stride_b", i64), ("o_stride_t", i64), ("o_stride_h", i64),
        ("lse_stride_b", i64), ("lse_stride_t", i64), ("lse_stride_h", i64),
        ("softmax_scale", f32), ("scale_has_log2e", i32), ("causal", i32), ("lse_base2", i32),
        ("sparsity", i32), ("window_local", i32), ("window_global", i32),
        ("block_idx", vp), ("block_cnt", vp), ("block_size", i32), ("n_qblocks", i32),
        ("max_nnz", i32), ("status_word", vp),
    ]


class DecodeArgs(C.Structure):
    _fields_ = [
        ("q", vp), ("k_cache", vp), ("v_cache", vp), ("o", vp),
        ("dtype", i32), ("batch", i32), ("heads_q", i32), ("heads_kv", i32), ("head_dim", i32),
        ("max_seqlen", i32), ("cu_seqlens", vp), ("seqlens", vp),
        ("q_stride_b", i64), ("q_stride_h", i64),
        ("k_stride_b", i64), ("k_stride_t", i64), ("k_stride_h", i64),
        ("v_stride_b", i64), ("v_stride_t", i64), ("v_stride_h", i64),
        ("o_stride_b", i64), ("o_stride_h", i64),
        ("softmax_scale", f32), ("chunk_tokens", i32),
        ("sparsity", i32), ("window_global", i32), ("window_local", i32),
        ("block_idx", vp), ("block_cnt", vp), ("block_size", i32), ("max_sel", i32),
        ("workspace", vp), ("workspace_bytes", C.c_size_t), ("status_word", vp),
    ]


class PrefillBwdArgs(C.Structure):
    _fields_ = [
        ("q", vp), ("k", vp), ("v", vp), ("o", vp), ("d_o", vp), ("lse", vp),
        ("dq", vp), ("dk", vp), ("dv", vp),
        ("dtype", i32), ("batch", i32), ("heads_q", i32), ("heads_kv", i32), ("head_dim", i32),
        ("seqlen", i32), ("max_seqlen", i32), ("total_tokens", i64), ("cu_seqlens", vp),
    ] + [(f"{n}_stride_{a}", i64) for n in ("q", "k", "v", "o", "do", "dq", "dk", "dv", "lse")
         for a in ("b", "t", "h")] + [
        ("softmax_scale", f32), ("scale_has_log2e", i32), ("causal", i32), ("lse_base2", i32),
        ("workspace", vp), ("workspace_bytes", C.c_size_t), ("status_word", vp),
    ]


class KvPackArgs(C.Structure):
    _fields_ = [("packed", vp), ("cache", vp), ("cu_seqlens", vp),
                ("batch", i32), ("heads", i32), ("head_dim", i32), ("capacity", i32),
                ("packed_stride_t", i64), ("packed_stride_h", i64),
                ("cache_stride_b", i64), ("cache_stride_t", i64), ("cache_stride_h", i64),
                ("zero_pad", i32)]


class KvAppendArgs(C.Structure):
    _fields_ = [("new_k", vp), ("new_v", vp), ("k_cache", vp), ("v_cache", vp), ("seqlens", vp),
                ("batch", i32), ("heads", i32), ("head_dim", i32), ("capacity", i32),
                ("new_stride_b", i64), ("new_stride_h", i64),
                ("cache_stride_b", i64), ("cache_stride_t", i64), ("cache_stride_h", i64)]


class PagedDecodeArgs(C.Structure):
    _fields_ = [
        ("q", vp), ("k_pages", vp), ("v_pages", vp), ("o", vp),
        ("dtype", i32), ("batch", i32), ("heads_q", i32), ("heads_kv", i32), ("head_dim", i32),
        ("page_size", i32), ("num_pages", i32), ("max_pages_per_seq", i32), ("max_seqlen", i32),
        ("page_table", vp), ("seqlens", vp),
        ("q_stride_b", i64), ("q_stride_h", i64),
        ("k_stride_page", i64), ("k_stride_t", i64), ("k_stride_h", i64),
        ("v_stride_page", i64), ("v_stride_t", i64), ("v_stride_h", i64),
        ("o_stride_b", i64), ("o_stride_h", i64),
        ("softmax_scale", f32), ("chunk_tokens", i32),
        ("workspace", vp), ("workspace_bytes", C.c_size_t), ("status_word", vp),
    ]


class WindowBlocksPrefillArgs(C.Structure):
    _fields_ = [("block_idx", vp), ("block_cnt", vp),
                ("batch", i32), ("heads", i32), ("n_qblocks", i32), ("max_nnz", i32),
                ("block_size", i32), ("window_local", i32), ("window_global", i32)]


class WindowBlocksDecodeArgs(C.Structure):
    _fields_ = [("block_idx", vp), ("block_cnt", vp), ("cu_seqlens", vp), ("seqlens", vp),
                ("batch", i32), ("heads_kv", i32), ("max_sel", i32),
                ("block_size", i32), ("window_local", i32), ("window_global", i32)]


class TopkBlocksArgs(C.Structure):
    _fields_ = [("scores", vp), ("score_stride_row", i64), ("n_valid", vp),
                ("rows", i32), ("n_blocks", i32), ("top_k", i32),
                ("force_first", i32), ("force_last", i32),
                ("block_idx", vp), ("block_cnt", vp)]


class RmsNormFwdArgs(C.Structure):
    _fields_ = [("x", vp), ("weight", vp), ("y", vp), ("rstd", vp),
                ("x_dtype", i32), ("w_dtype", i32), ("rows", i64), ("dim", i32),
                ("x_stride_row", i64), ("y_stride_row", i64), ("eps", f32)]


class RmsNormBwdArgs(C.Structure):
    _fields_ = [("dy", vp), ("x", vp), ("weight", vp), ("rstd", vp), ("dx", vp), ("dweight", vp),
                ("x_dtype", i32), ("w_dtype", i32), ("rows", i64), ("dim", i32),
                ("dy_stride_row", i64), ("x_stride_row", i64), ("dx_stride_row", i64),
                ("workspace", vp), ("workspace_bytes", C.c_size_t)]


# every symbol include/b200attn.h declares: name -> (restype, argtypes)
SYMBOLS = {
    "b200attn_abi_version": (C.c_int, []),
    "b200attn_last_launch_count": (C.c_int, []),
    "b200attn_strerror": (C.c_char_p, [C.c_int]),
    "b200attn_prefill_workspace_bytes": (C.c_size_t, [C.POINTER(PrefillArgs)]),
    "b200attn_prefill_fwd": (C.c_int, [C.POINTER(PrefillArgs), vp]),
    "b200attn_prefill_fwd_rows": (C.c_int, [C.POINTER(PrefillArgs), C.c_int32, C.c_int32, vp]),
    "b200attn_sparse_prefill_fwd": (C.c_int, [C.POINTER(PrefillArgs), vp]),
    "b200attn_decode_workspace_bytes": (C.c_size_t, [C.POINTER(DecodeArgs)]),
    "b200attn_decode_fwd": (C.c_int, [C.POINTER(DecodeArgs), vp]),
    "b200attn_sparse_decode_fwd": (C.c_int, [C.POINTER(DecodeArgs), vp]),
    "b200attn_decode_fwd_noalloc": (C.c_int, [C.POINTER(DecodeArgs), vp]),
    "b200attn_prefill_bwd_workspace_bytes": (C.c_size_t, [C.POINTER(PrefillBwdArgs)]),
    "b200attn_prefill_bwd": (C.c_int, [C.POINTER(PrefillBwdArgs), vp]),
    "b200attn_kv_pack_to_cache": (C.c_int, [C.POINTER(KvPackArgs), vp]),
    "b200attn_kv_append": (C.c_int, [C.POINTER(KvAppendArgs), vp]),
    "b200attn_paged_decode_workspace_bytes": (C.c_size_t, [C.POINTER(PagedDecodeArgs)]),
    "b200attn_paged_decode_fwd": (C.c_int, [C.POINTER(PagedDecodeArgs), vp]),
    "b200attn_window_blocks_prefill_max_nnz": (i32, [i32, i32, i32, i32]),
    "b200attn_window_blocks_prefill": (C.c_int, [C.POINTER(WindowBlocksPrefillArgs), vp]),
    "b200attn_window_blocks_decode": (C.c_int, [C.POINTER(WindowBlocksDecodeArgs), vp]),
    "b200attn_topk_blocks": (C.c_int, [C.POINTER(TopkBlocksArgs), vp]),
    "b200attn_selftest_bounded_wait": (C.c_int, [vp, i64, vp, vp]),
    "b200attn_rmsnorm_fwd": (C.c_int, [C.POINTER(RmsNormFwdArgs), vp]),
    "b200attn_rmsnorm_bwd_workspace_bytes": (C.c_size_t, [C.POINTER(RmsNormBwdArgs)]),
    "b200attn_rmsnorm_bwd": (C.c_int, [C.POINTER(RmsNormBwdArgs), vp]),
}
NOALLOC_SCRATCH_BYTES = 32 << 20

_lib = None


def lib():
    """The loaded library; raises if it has not been built (python -m tritonops_b200.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m tritonops_b200.build` "
                "(there is no CPU or PyTorch fallback)")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        if handle.b200attn_abi_version() != 1:
            raise RuntimeError("libb200attn.so ABI version mismatch; rebuild it")
        _lib = handle
    return _lib


def check(status):
    if status != 0:
        msg = lib().b200attn_strerror(status).decode()
        if status in (-8, -10, -12):
            raise RuntimeError(f"b200attn: {msg} (status {status})")
        raise ValueError(f"b200attn: {msg} (status {status})")
