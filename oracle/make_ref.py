"""Stage the reference's own attention modules next to the oracle so that they travel to a GPU
machine, where the reference checkout itself does not exist.

    REFERENCE_ROOT=<checkout of rookie-joe/TritonOps> python -m oracle.make_ref

Copies flash_attn_triton/*.py, utils/utils.py and common/rms.py, unmodified, into oracle/_ref/ (git-ignored: the
reference's sources never enter this repository's history).  The staged modules are test
infrastructure like the rest of oracle/: the GPU parity tests run the reference's Triton kernels
from there beside this library's kernels, and bench.py times them as a second baseline.  Nothing
under tritonops_b200/ imports them."""
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
FILES = [("flash_attn_triton", "flash_attn_triton.py"), ("flash_attn_triton", "flash_attn_decoding.py"),
         ("flash_attn_triton", "flash_attn_decoding_sparse.py"), ("flash_attn_triton", "flash_attn_sparse_attn_triton.py"),
         ("utils", "utils.py"), ("common", "rms.py")]


def reference_root():
    """REFERENCE_ROOT, else a checkout named `reference` beside this repository; None if neither exists."""
    cand = os.environ.get("REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    return cand if os.path.isdir(os.path.join(cand, "flash_attn_triton")) else None


def stage(root=None) -> bool:
    """Copy the modules; False (and nothing done) when no reference checkout is reachable."""
    root = root or reference_root()
    if root is None:
        return False
    for sub, name in FILES:
        os.makedirs(os.path.join(REF_DIR, sub), exist_ok=True)
        shutil.copyfile(os.path.join(root, sub, name), os.path.join(REF_DIR, sub, name))
    return True


if __name__ == "__main__":
    ok = stage()
    print("staged into", REF_DIR if ok else "nothing: set REFERENCE_ROOT")
    sys.exit(0 if ok else 1)
