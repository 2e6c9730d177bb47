"""The C-ABI library builds, loads and exports every symbol include/b200attn.h
declares; argument validation returns the documented status codes without
touching a GPU."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from tritonops_b200 import _lib, build
    build.build_library()
    return _lib.lib()


def declared_functions():
    src = open(os.path.join(ROOT, "include", "b200attn.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(b200attn_[a-z0-9_]+)\s*\(", src)))


def test_header_symbols_exported(lib):
    from tritonops_b200 import _lib
    names = declared_functions()
    assert "b200attn_prefill_fwd" in names and "b200attn_decode_fwd" in names
    for n in names:
        assert hasattr(lib, n), f"{n} declared in b200attn.h but not exported"
        assert n in _lib.SYMBOLS, f"{n} has no ctypes prototype"


def test_struct_sizes_match_header(lib):
    """ctypes mirrors must have the C layout: compile a tiny probe with gcc."""
    import subprocess
    import tempfile
    from tritonops_b200 import _lib
    with tempfile.TemporaryDirectory() as d:
        src = os.path.join(d, "p.c")
        open(src, "w").write(
            '#include <stdio.h>\n#include <stddef.h>\n#include "b200attn.h"\n'
            'int main(){printf("%zu %zu %zu %zu %zu %zu\\n", sizeof(b200attn_prefill_args),'
            ' sizeof(b200attn_decode_args), offsetof(b200attn_prefill_args, status_word),'
            ' offsetof(b200attn_decode_args, workspace_bytes), sizeof(b200attn_prefill_bwd_args),'
            ' offsetof(b200attn_prefill_bwd_args, workspace_bytes));return 0;}\n')
        exe = os.path.join(d, "p")
        subprocess.check_call(["gcc", "-I", os.path.join(ROOT, "include"), src, "-o", exe])
        a, b, c, e, f, g = map(int, subprocess.check_output([exe]).split())
    assert a == C.sizeof(_lib.PrefillArgs) and b == C.sizeof(_lib.DecodeArgs)
    assert f == C.sizeof(_lib.PrefillBwdArgs) and g == _lib.PrefillBwdArgs.workspace_bytes.offset
    assert c == _lib.PrefillArgs.status_word.offset
    assert e == _lib.DecodeArgs.workspace_bytes.offset


def test_version_and_strerror(lib):
    assert lib.b200attn_abi_version() == 1
    assert lib.b200attn_strerror(0) == b"ok"
    for code in range(-12, 0):
        assert b"unknown" not in lib.b200attn_strerror(code)
    assert b"unknown" in lib.b200attn_strerror(-99)


def test_decode_validation_codes(lib):
    from tritonops_b200._lib import DecodeArgs
    a = DecodeArgs()
    assert lib.b200attn_decode_fwd(C.byref(a), None) == -1           # NULL pointers
    a.q = a.k_cache = a.v_cache = a.o = 0x1000
    a.seqlens = 0x1000
    a.dtype = 7
    assert lib.b200attn_decode_fwd(C.byref(a), None) == -2
    a.dtype, a.head_dim = 1, 48
    assert lib.b200attn_decode_fwd(C.byref(a), None) == -3
    a.head_dim, a.batch, a.heads_q, a.heads_kv = 128, 2, 6, 4
    assert lib.b200attn_decode_fwd(C.byref(a), None) == -4
    a.heads_kv = 2
    a.q = 0x1008
    assert lib.b200attn_decode_fwd(C.byref(a), None) == -5
    a.q, a.k_stride_t = 0x1000, 100
    assert lib.b200attn_decode_fwd(C.byref(a), None) == -6
    a.k_stride_t, a.max_seqlen = 256, 1024
    assert lib.b200attn_decode_fwd(C.byref(a), None) == -8           # no workspace
    a.cu_seqlens = 0x1000
    assert lib.b200attn_decode_fwd(C.byref(a), None) == -1           # both length forms
    a.cu_seqlens = None
    a.sparsity = 2
    assert lib.b200attn_sparse_decode_fwd(C.byref(a), None) == -1    # block list missing
    a.sparsity = 5
    assert lib.b200attn_sparse_decode_fwd(C.byref(a), None) == -9


def test_decode_workspace_formula(lib):
    from tritonops_b200._lib import DecodeArgs
    a = DecodeArgs(batch=64, heads_q=32, heads_kv=8, head_dim=128, max_seqlen=8192, chunk_tokens=512)
    rows = 64 * 32 * 16
    assert lib.b200attn_decode_workspace_bytes(C.byref(a)) == rows * 128 * 4 + rows * 4
    a.chunk_tokens = 0                        # automatic: 2048-key chunks for this size
    assert lib.b200attn_decode_workspace_bytes(C.byref(a)) == 64 * 32 * 4 * (128 * 4 + 4)
    a.batch = 1                               # few units (8): the longest chunk that still gives 148 CTAs (256 keys)
    assert lib.b200attn_decode_workspace_bytes(C.byref(a)) == 1 * 32 * 32 * (128 * 4 + 4)
    a.max_seqlen = 131072                     # ... which is 4096 keys for one long sequence
    assert lib.b200attn_decode_workspace_bytes(C.byref(a)) == 1 * 32 * 32 * (128 * 4 + 4)
    a.max_seqlen = 8192
    a.batch, a.chunk_tokens = 64, 512
    a.sparsity, a.window_global, a.window_local = 1, 64, 1024
    assert lib.b200attn_decode_workspace_bytes(C.byref(a)) == 64 * 32 * 3 * (128 * 4 + 4)


def test_ops_reject_cpu_tensors(lib):
    import torch
    from tritonops_b200 import ops
    q = torch.zeros(1, 2, 64, dtype=torch.float16)
    kv = torch.zeros(1, 8, 2, 64, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        ops.decode(q, kv, kv, seqlens=torch.tensor([8], dtype=torch.int32))


def test_prefill_validation_codes(lib):
    from tritonops_b200._lib import PrefillArgs
    a = PrefillArgs()
    assert lib.b200attn_prefill_fwd(C.byref(a), None) == -1            # NULL pointers
    a.q = a.k = a.v = a.o = 0x1000
    a.dtype = 3
    assert lib.b200attn_prefill_fwd(C.byref(a), None) == -2
    a.dtype, a.head_dim = 1, 80
    assert lib.b200attn_prefill_fwd(C.byref(a), None) == -3
    a.head_dim, a.batch, a.heads_q, a.heads_kv = 128, 1, 5, 2
    assert lib.b200attn_prefill_fwd(C.byref(a), None) == -4
    a.heads_q = 4
    assert lib.b200attn_prefill_fwd(C.byref(a), None) == -7            # seqlen 0, no cu_seqlens
    a.seqlen = 256
    a.k = 0x1004
    assert lib.b200attn_prefill_fwd(C.byref(a), None) == -5
    a.k, a.v_stride_t = 0x1000, 12
    assert lib.b200attn_prefill_fwd(C.byref(a), None) == -6
    a.v_stride_t, a.softmax_scale = 256, 0.0
    assert lib.b200attn_prefill_fwd(C.byref(a), None) == -7            # scale must be positive
    a.softmax_scale = 0.1
    # row ranges: start on a multiple of 256, end on one unless they reach the end of the sequence
    a.seqlen = 1024
    assert lib.b200attn_prefill_fwd_rows(C.byref(a), 100, 512, None) == -7
    assert lib.b200attn_prefill_fwd_rows(C.byref(a), 256, 300, None) == -7
    assert lib.b200attn_prefill_fwd_rows(C.byref(a), 512, 512, None) == -7
    assert lib.b200attn_prefill_fwd_rows(C.byref(a), 2048, 4096, None) == 0    # past the end: nothing to do
    a.seqlen = 256
    a.sparsity = 2                                                      # block list without lists
    assert lib.b200attn_sparse_prefill_fwd(C.byref(a), None) == -1
    a.block_idx = a.block_cnt = 0x1000
    a.block_size, a.n_qblocks, a.max_nnz = 32, 4, 4
    assert lib.b200attn_sparse_prefill_fwd(C.byref(a), None) == -9     # only 64-token blocks
    a.block_size, a.seqlen = 64, 64 * 2048 + 1
    assert lib.b200attn_sparse_prefill_fwd(C.byref(a), None) == -11    # list capacity exceeded
    a.sparsity, a.window_local = 1, -1
    assert lib.b200attn_sparse_prefill_fwd(C.byref(a), None) == -9
    a.sparsity = 9
    assert lib.b200attn_sparse_prefill_fwd(C.byref(a), None) == -9
    assert lib.b200attn_prefill_workspace_bytes(C.byref(a)) == 0


def test_prefill_bwd_validation_codes(lib):
    from tritonops_b200._lib import PrefillBwdArgs
    a = PrefillBwdArgs()
    assert lib.b200attn_prefill_bwd(C.byref(a), None) == -1
    for n in ("q", "k", "v", "o", "d_o", "lse", "dq", "dk", "dv"):
        setattr(a, n, 0x1000)
    a.dtype, a.head_dim, a.batch, a.heads_q, a.heads_kv, a.seqlen = 1, 128, 2, 8, 2, 256
    a.softmax_scale = 0.1
    assert lib.b200attn_prefill_bwd(C.byref(a), None) == -8          # no workspace
    rows = 2 * 256 * 8
    assert lib.b200attn_prefill_bwd_workspace_bytes(C.byref(a)) == rows * 128 * 4 + rows * 4
    a.head_dim = 96
    assert lib.b200attn_prefill_bwd_workspace_bytes(C.byref(a)) == rows * 128 * 4 + rows * 4
    a.head_dim = 64
    assert lib.b200attn_prefill_bwd_workspace_bytes(C.byref(a)) == rows * 64 * 4 + rows * 4
    a.dk_stride_t = 4
    assert lib.b200attn_prefill_bwd(C.byref(a), None) == -6


def test_struct_sizes_of_selection_and_paged_args(lib):
    import subprocess
    import tempfile
    from tritonops_b200 import _lib
    names = [("b200attn_paged_decode_args", _lib.PagedDecodeArgs),
             ("b200attn_window_blocks_prefill_args", _lib.WindowBlocksPrefillArgs),
             ("b200attn_window_blocks_decode_args", _lib.WindowBlocksDecodeArgs),
             ("b200attn_topk_blocks_args", _lib.TopkBlocksArgs),
             ("b200attn_kv_pack_args", _lib.KvPackArgs), ("b200attn_kv_append_args", _lib.KvAppendArgs),
             ("b200attn_rmsnorm_fwd_args", _lib.RmsNormFwdArgs), ("b200attn_rmsnorm_bwd_args", _lib.RmsNormBwdArgs)]
    with tempfile.TemporaryDirectory() as d:
        src = os.path.join(d, "p.c")
        body = "".join(f'printf("%zu\\n", sizeof({n}));' for n, _ in names)
        open(src, "w").write('#include <stdio.h>\n#include "b200attn.h"\nint main(){' + body + 'return 0;}\n')
        exe = os.path.join(d, "p")
        subprocess.check_call(["gcc", "-I", os.path.join(ROOT, "include"), src, "-o", exe])
        sizes = list(map(int, subprocess.check_output([exe]).split()))
    for (n, cls), size in zip(names, sizes):
        assert size == C.sizeof(cls), n
    assert _lib.PagedDecodeArgs.workspace_bytes.offset % 8 == 0


def test_window_cover_width_is_host_side_and_matches_brute_force(lib):
    """b200attn_window_blocks_prefill_max_nnz needs no GPU; it must equal the widest
    row of the brute-force block cover of the window mask."""
    from oracle import attention_oracle as orc
    L = lib
    for nqb in (1, 3, 12):
        for local, glob in [(64, 64), (200, 256), (1, 0), (0, 128), (2, 0), (65, 1), (0, 0), (129, 100)]:
            _, cnt = orc.window_to_block_lists(nqb * 64, 64, local, glob)
            assert L.b200attn_window_blocks_prefill_max_nnz(64, local, glob, nqb) == int(cnt.max())


def test_new_entry_points_validate_before_touching_the_device(lib):
    from tritonops_b200 import _lib
    L = lib
    a = _lib.TopkBlocksArgs()
    assert L.b200attn_topk_blocks(C.byref(a), None) == -1
    b = _lib.WindowBlocksPrefillArgs()
    assert L.b200attn_window_blocks_prefill(C.byref(b), None) == -1
    c = _lib.WindowBlocksDecodeArgs()
    assert L.b200attn_window_blocks_decode(C.byref(c), None) == -1
    d = _lib.PagedDecodeArgs()
    assert L.b200attn_paged_decode_fwd(C.byref(d), None) == -1
    assert L.b200attn_rmsnorm_fwd(C.byref(_lib.RmsNormFwdArgs()), None) == -1
    assert L.b200attn_rmsnorm_bwd(C.byref(_lib.RmsNormBwdArgs()), None) == -1
    assert L.b200attn_rmsnorm_bwd_workspace_bytes(C.byref(_lib.RmsNormBwdArgs(rows=1000, dim=4096))) == 592 * 4096 * 4
    assert L.b200attn_paged_decode_workspace_bytes(C.byref(d)) == 0


def test_head_dim_mismatch_is_rejected_before_any_launch(lib):
    """One head_dim for Q, K, V: a narrower V (which the reference wrapper lets through,
    flash_attn_decoding.py:233-236) must raise in Python, before any pointer reaches a kernel."""
    import torch
    from tritonops_b200 import ops
    q = torch.zeros(2, 4, 64, dtype=torch.float16)
    kc = torch.zeros(2, 16, 2, 64, dtype=torch.float16)
    vc = torch.zeros(2, 16, 2, 32, dtype=torch.float16)
    sl = torch.tensor([16, 16], dtype=torch.int32)
    with pytest.raises(ValueError, match="share head_dim"):
        ops.decode(q, kc, vc, seqlens=sl)
    with pytest.raises(ValueError, match="share head_dim"):
        ops.paged_decode(q, kc, vc, torch.zeros(2, 1, dtype=torch.int32), sl)
    qp, kp, vp = torch.zeros(1, 16, 4, 64, dtype=torch.float16), torch.zeros(1, 16, 2, 64, dtype=torch.float16), \
        torch.zeros(1, 16, 2, 32, dtype=torch.float16)
    with pytest.raises(ValueError, match="share head_dim"):
        ops.prefill(qp, kp, vp)
    with pytest.raises(ValueError, match="share head_dim"):
        ops.prefill_bwd(qp, kp, kp, qp, torch.zeros(1, 16, 4, 32, dtype=torch.float16), torch.zeros(1, 16, 4))


def test_valid_call_without_a_device_reports_cuda_error(lib):
    """Arguments that pass validation reach the device probe; with no CUDA device it answers
    B200ATTN_ERR_CUDA (never run where a device exists: the pointers are made up)."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    from tritonops_b200 import _lib
    a = _lib.RmsNormFwdArgs(0x1000, 0x1000, 0x2000, None, _lib.BF16, _lib.BF16, 4, 64, 64, 64, 1e-6)
    assert lib.b200attn_rmsnorm_fwd(C.byref(a), None) == -10


@pytest.mark.gpu
def test_wrong_architecture_is_refused():
    """B200ATTN_ERR_DEVICE: every launcher probes the current device once (the counterpart of the
    reference's arch probe, utils/utils.py:19-24) and refuses anything but compute capability
    10.x.  All GPUs here are sm_100, so a child process is told to assume another architecture."""
    import subprocess
    import sys
    code = (
        "import torch\n"
        "from tritonops_b200 import ops\n"
        "x = torch.randn(4, 64, device='cuda', dtype=torch.bfloat16)\n"
        "w = torch.ones(64, device='cuda', dtype=torch.bfloat16)\n"
        "q = torch.randn(2, 4, 64, device='cuda', dtype=torch.float16)\n"
        "kc = torch.randn(2, 64, 2, 64, device='cuda', dtype=torch.float16)\n"
        "sl = torch.tensor([64, 10], dtype=torch.int32, device='cuda')\n"
        "n = 0\n"
        "for f in (lambda: ops.rmsnorm_fwd(x, w, 1e-6), lambda: ops.decode(q, kc, kc, seqlens=sl),\n"
        "          lambda: ops.prefill(kc[:1], kc[:1], kc[:1])):\n"
        "    try:\n"
        "        f()\n"
        "    except RuntimeError as e:\n"
        "        assert 'status -12' in str(e) and 'compute capability' in str(e), str(e)\n"
        "        n += 1\n"
        "print('refused', n)\n")
    env = dict(os.environ, B200ATTN_ASSUME_CC_MAJOR="9", PYTHONPATH=ROOT)
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    assert "refused 3" in out.stdout
