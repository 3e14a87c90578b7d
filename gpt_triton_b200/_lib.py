"""ctypes binding of libb200gpt.so (declared in include/b200_gpt.h).

There is no fallback: if the library is missing or a symbol cannot be bound, importing
the operators fails with an error that says how to build it.
"""

import ctypes
import os

import torch

from .build import LIB_PATH

F32, F16, BF16 = 0, 1, 2
_TORCH_TO_CODE = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}

c_i64, c_int, c_float, c_void_p, c_size_t = ctypes.c_int64, ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_size_t
_p_i64 = ctypes.POINTER(ctypes.c_int64)

# name -> (restype, argtypes); must list every function include/b200_gpt.h declares
SIGNATURES = {
    "b200_status_string": (ctypes.c_char_p, [c_int]),
    "b200_last_cuda_error": (ctypes.c_char_p, []),
    "b200_abi_version": (c_int, []),
    "b200_launch_count": (ctypes.c_uint64, []),
    "b200_embedding": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_i64, c_i64, c_i64, c_i64, c_i64, c_int, c_void_p, c_void_p]),
    "b200_embedding_ln_stats": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_i64, c_i64, c_i64, c_i64, c_i64, c_int, c_void_p, c_float, c_void_p, c_void_p,
                                        c_void_p]),
    "b200_row_ln_stats": (c_int, [c_void_p, c_void_p, c_void_p, c_i64, c_i64, c_float, c_int, c_void_p]),
    "b200_fold_layernorm": (c_int, [c_void_p] * 8 + [c_i64, c_i64, c_i64, c_int, c_void_p]),
    "b200_gemm_ln_workspace_bytes": (c_size_t, [c_i64, c_i64]),
    "b200_gemm_ln": (c_int, [c_void_p] * 5 + [c_i64] * 7 + [c_int, c_int, c_int] + [c_void_p] * 5 + [c_float, c_void_p, c_size_t, c_void_p, c_void_p]),
    "b200_layernorm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_i64, c_i64, c_float, c_int, c_int, c_void_p]),
    "b200_pack_operand": (c_int, [c_void_p, c_void_p, c_i64, c_i64, c_i64, c_i64, c_int, c_int, c_int, c_void_p]),
    "b200_gemm": (c_int, [c_void_p] * 5 + [c_i64] * 7 + [c_int, c_int, c_int, c_void_p, c_void_p]),
    "b200_gemm_argmax_workspace_bytes": (c_size_t, [c_i64, c_i64]),
    "b200_gemm_argmax": (c_int, [c_void_p] * 5 + [c_i64] * 7 + [c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p, c_void_p]),
    "b200_gemm_rowstats": (c_int, [c_void_p] * 3 + [c_i64] * 5 + [c_int, c_int] + [c_void_p] * 5 + [c_size_t, c_void_p, c_void_p]),
    "b200_ffn_workspace_bytes": (c_size_t, [c_i64, c_i64, c_i64, c_int, c_int]),
    "b200_ffn": (c_int, [c_void_p] * 5 + [c_i64] * 4 + [c_int, c_int, c_int, c_void_p, c_size_t, c_void_p, c_void_p]),
    "b200_ffn_static_scratch": (c_int, [c_void_p] * 5 + [c_i64] * 4 + [c_int, c_int, c_int, c_void_p, c_void_p]),
    "b200_attention": (c_int, [c_void_p] * 4 + [c_i64] * 4 + [_p_i64] * 4 + [c_float, c_int, c_int, c_void_p, c_void_p]),
    "b200_embedding_at": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_i64, c_i64, c_i64, c_i64, c_i64, c_int, c_void_p, c_float, c_void_p, c_void_p,
                                  c_void_p, c_void_p]),
    "b200_kv_cache_fill": (c_int, [c_void_p, c_void_p, c_i64, c_i64, c_i64, c_i64, c_int, c_void_p]),
    "b200_attention_decode": (c_int, [c_void_p, c_void_p, c_void_p, c_i64, c_i64, c_i64, c_i64, c_float, c_int, c_void_p, c_void_p, c_void_p]),
    "b200_decode_append": (c_int, [c_void_p, c_void_p, c_i64, c_i64, c_i64, c_void_p, c_int, c_void_p, c_void_p, c_void_p]),
    "b200_sample_logits": (c_int, [c_void_p, c_i64, c_i64, c_i64, c_int, c_float, c_int, ctypes.c_uint64, c_void_p, c_void_p, c_void_p]),
    "b200_selftest_bounded_wait": (c_int, [c_void_p, c_i64, c_void_p]),
}

_lib = None


class B200Error(RuntimeError):
    """A libb200gpt entry point returned a non-zero status."""


def load():
    """Load the shared library once and bind every declared symbol."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: the CUDA extension has not been built. "
            "Run `python -m gpt_triton_b200.build` (needs nvcc); there is no CPU or PyTorch fallback."
        )
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library does not export it
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def dtype_code(dtype):
    try:
        return _TORCH_TO_CODE[dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {dtype}; expected float32, float16 or bfloat16") from None


def check(status, what):
    if status != 0:
        lib = load()
        msg = lib.b200_status_string(status).decode()
        if status == 3:
            msg += ": " + lib.b200_last_cuda_error().decode()
        raise B200Error(f"{what}: {msg} (status {status})")


def stream_ptr(device):
    return torch.cuda.current_stream(device).cuda_stream


def require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError(
                "gpt_triton_b200 operators run only on CUDA tensors (sm_100a kernels); got a tensor on " + str(t.device)
            )
