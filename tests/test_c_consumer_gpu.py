"""A plain C program (tests/c_abi/consumer.c) includes include/b200attn.h, links libb200attn.so and the
CUDA runtime, and runs decoding and paged decoding without Python or torch in the process."""
import os
import shutil
import subprocess

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_c_program_drives_the_library(tmp_path):
    from tritonops_b200 import _lib, build
    build.build_library()
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    exe = str(tmp_path / "consumer")
    libdir = os.path.dirname(_lib.LIB_PATH)
    cmd = [shutil.which("gcc") or "gcc", "-std=c99", "-O1", "-I", os.path.join(ROOT, "include"),
           "-I", os.path.join(cuda, "include"), os.path.join(ROOT, "tests", "c_abi", "consumer.c"), "-o", exe,
           "-L", libdir, "-lb200attn", "-L", os.path.join(cuda, "lib64"), "-lcudart", "-lm",
           "-Wl,-rpath," + libdir, "-Wl,-rpath," + os.path.join(cuda, "lib64")]
    subprocess.check_call(cmd)
    out = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "c-abi consumer ok" in out.stdout
