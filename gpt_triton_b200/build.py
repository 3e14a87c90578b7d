"""Build libb200gpt.so (the sm_100a kernels + C ABI) in-tree with nvcc.

    python -m gpt_triton_b200.build [--force]

nvcc cross-compiles for sm_100a, so this works on a machine without a GPU.
"""

import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_PATH = os.path.join(PKG_DIR, "libb200gpt.so")
SOURCES = ["api.cu", "elementwise.cu", "gemm_sm100.cu", "attention.cu", "attention_sm100.cu", "decode.cu", "ffn_static_scratch.cu", "selftest.cu"]
HEADERS = [os.path.join(CSRC, "common.cuh"), os.path.join(CSRC, "sm100_primitives.cuh"),
           os.path.join(os.path.dirname(PKG_DIR), "include", "b200_gpt.h")]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17", "-shared", "-Xcompiler", "-fPIC",
]


def _nvcc():
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: libb200gpt.so cannot be built")
    return exe


def is_stale():
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, s) for s in SOURCES] + HEADERS
    return any(os.path.getmtime(d) > built for d in deps)


def build(force=False, verbose=False):
    """Compile the library if it is missing or older than its sources; return its path."""
    if not force and not is_stale():
        return LIB_PATH
    cmd = [_nvcc(), *NVCC_FLAGS, "-o", LIB_PATH] + [os.path.join(CSRC, s) for s in SOURCES]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    if verbose:
        print(res.stderr)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
