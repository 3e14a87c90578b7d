"""The five operators of the reference's ``kernels.py``, backed by libb200gpt (sm_100a).

Same names, positional arguments, assertions and result shapes/dtypes as the reference
(kernels.py:76, 149, 261, 348, 478), so code written against it keeps working:

    fused_embeddings, fused_layer_norm, fused_ffn, matmul_and_split_qkv, flash_attention_v1

Differences, all deliberate:
* forward/eval only: a non-zero ``dropout_prob`` raises ``NotImplementedError`` (the
  reference's modules always pass 0 in eval mode, gpt.py:44, 92, 165);
* ``matmul_and_split_qkv`` returns q, k, v as strided views into one fused buffer instead of
  three transposed copies (kernels.py:359-365), and ``flash_attention_v1`` accepts such views;
* keyword-only extras (``weight_is_nk``, ``merged_heads``, ``out`` ...) used by the model to
  avoid copies; defaults reproduce the reference's behaviour;
* LayerNorm folded into the following GEMM (the fusion the reference leaves as a TODO, kernels.py:132-133):
  ``fold_layer_norm`` prepares the weights once, ``fused_ffn(..., ln_stats=...)`` consumes the raw rows with
  their ``RowStats`` (mean, rstd per row), which ``fused_embeddings`` / ``fused_ffn(..., return_row_stats=True)`` /
  ``row_stats`` produce -- the normalised activations are never written (16-bit dtypes only).

Every operator launches on torch's current CUDA stream and never synchronises.  There is
no CPU path: tensors must live on a CUDA device and the shared library must be built.
"""

import ctypes
import math

import torch

from . import _lib
from ._lib import check, dtype_code, require_cuda, stream_ptr

_lib.load()  # fail at import time, loudly, if the extension is not built

LN_EPS = 1e-5  # kernels.py:106
LN_EXT_COLS = 64  # B200_LN_EXT_COLS: width of the row / weight extensions of a folded LayerNorm


def _no_dropout(p):
    if p != 0.0:
        raise NotImplementedError("libb200gpt implements the forward/eval path only: dropout_prob must be 0")


def _ptr(t):
    return None if t is None else t.data_ptr()


_status_words = {}


def _status_ptr(dev):
    """Address of the device int32 (one per GPU, allocated at first use) into which the tensor-core kernels report
    when one of them abandons a bounded wait; None while a CUDA graph is being captured before the word exists."""
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    word = _status_words.get(idx)
    if word is None:
        if torch.cuda.is_current_stream_capturing():
            return None
        word = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _status_words[idx] = word
    return word.data_ptr()


def device_status(device=None, reset=True):
    """0, or the code left by the first kernel on `device` that gave up a bounded on-chip wait since the last reset
    (its results are then invalid).  Synchronises the device."""
    idx = torch.cuda.current_device() if device is None else torch.device(device).index
    word = _status_words.get(idx)
    if word is None:
        return 0
    code = int(word.item())
    if code and reset:
        word.zero_()
    return code


def bounded_wait_selftest(limit_cycles=200_000_000, device=None):
    """Launch the library's self-test (one warp waiting on a barrier that nothing completes) and return the status
    code it reports once the wait has run out: B200_ERR_DEVICE_WAIT (6) on a healthy GPU.  Synchronises."""
    dev = torch.device("cuda", torch.cuda.current_device() if device is None else torch.device(device).index)
    word = torch.zeros(1, dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        check(_lib.load().b200_selftest_bounded_wait(word.data_ptr(), int(limit_cycles), stream_ptr(dev)), "bounded_wait_selftest")
    return int(word.item())


def _same_device(*tensors):
    """Operands must live on one CUDA device; make it current so the launch lands there."""
    ts = [t for t in tensors if t is not None]
    dev = ts[0].device
    for t in ts:
        assert t.device == dev, f"operands on different devices: {t.device} vs {dev}"
    return dev


# ----------------------------------------------------------------------------- embeddings
class RowStats:
    """LayerNorm statistics of the rows of an (M, cols) matrix: ``data[row] = (mean, 1 / sqrt(variance + eps))``,
    float32, shape (M, 2), variance biased -- the two numbers the reference's fused_layer_norm derives per row
    (kernels.py:116-130).  Producers: ``fused_embeddings(..., return_row_stats=True)``, ``row_stats`` and
    ``fused_ffn(..., return_row_stats=True)``; consumer: ``fused_ffn(..., ln_stats=...)``.  For 16-bit rows ``ext``
    (M, 64) holds, in the rows' dtype, the "row extension" the consuming GEMM multiplies as one extra k-block
    (-mean and 1/rstd as high/low parts; see include/b200_gpt.h); None for float32 rows."""

    __slots__ = ("data", "cols", "ext")

    def __init__(self, data, cols, ext=None):
        self.data, self.cols, self.ext = data, cols, ext

    @property
    def mean(self):
        return self.data[:, 0]

    @property
    def rstd(self):
        return self.data[:, 1]


@torch.no_grad()
def row_stats(x):
    """RowStats of the rows of x (*, H) (the statistics half of the reference's fused_layer_norm,
    kernels.py:116-130): what ``fused_ffn(..., ln_stats=...)`` needs for rows that no operator of this
    library produced."""
    require_cuda(x)
    assert x.is_contiguous()
    H = x.shape[-1]
    M = x.numel() // H if H else 0
    data = torch.empty((max(M, 1), 2), device=x.device, dtype=torch.float32)
    ext = torch.empty((max(M, 1), LN_EXT_COLS), device=x.device, dtype=x.dtype) if x.dtype != torch.float32 else None
    with torch.cuda.device(x.device):
        st = _lib.load().b200_row_ln_stats(x.data_ptr(), data.data_ptr(), _ptr(ext), M, H, LN_EPS, dtype_code(x.dtype), stream_ptr(x.device))
    check(st, "row_stats")
    return RowStats(data[:M], H, None if ext is None else ext[:M])


@torch.no_grad()
def fused_embeddings(x, wte, wpe, dropout_prob=0.0, *, return_row_stats=False, position=None):
    """z[b, l, :] = wte[x[b, l], :] + wpe[l, :]  (reference kernels.py:76-101).  With ``return_row_stats`` the
    result is ``(z, RowStats of z's rows)``, taken while the rows are written.  ``position`` (a CUDA int32 tensor;
    token-by-token generation) makes the first position ``position[0]``, read on the device at run time, instead
    of 0."""
    _no_dropout(dropout_prob)
    require_cuda(x, wte, wpe)
    assert wte.shape[1] == wpe.shape[1]
    assert x.is_contiguous()
    assert wte.is_contiguous()
    assert wpe.is_contiguous()
    assert wte.dtype == wpe.dtype
    B, L = x.shape
    V, H = wte.shape
    P = wpe.shape[0]
    assert L <= P, f"sequence length {L} exceeds the position table ({P} rows)"
    dev = _same_device(x, wte, wpe)
    if x.dtype != torch.int64:
        x = x.to(torch.int64)
    z = torch.empty((B * L, H), device=dev, dtype=wte.dtype)
    if position is not None:
        assert position.dtype == torch.int32 and position.device == dev and position.numel() >= 1
        stats = torch.empty((max(B * L, 1), 2), device=dev, dtype=torch.float32) if return_row_stats else None
        ext = torch.empty((max(B * L, 1), LN_EXT_COLS), device=dev, dtype=wte.dtype) if return_row_stats and wte.dtype != torch.float32 else None
        with torch.cuda.device(dev):
            st = _lib.load().b200_embedding_at(x.data_ptr(), wte.data_ptr(), wpe.data_ptr(), z.data_ptr(), B, L, V, P, H, dtype_code(wte.dtype),
                                               None, LN_EPS, _ptr(stats), _ptr(ext), position.data_ptr(), stream_ptr(dev))
        check(st, "fused_embeddings(position)")
        z = z.view((B, L, H))
        return (z, RowStats(stats[:B * L], H, None if ext is None else ext[:B * L])) if return_row_stats else z
    if return_row_stats:
        stats = torch.empty((max(B * L, 1), 2), device=dev, dtype=torch.float32)
        ext = torch.empty((max(B * L, 1), LN_EXT_COLS), device=dev, dtype=wte.dtype) if wte.dtype != torch.float32 else None
        with torch.cuda.device(dev):
            st = _lib.load().b200_embedding_ln_stats(x.data_ptr(), wte.data_ptr(), wpe.data_ptr(), z.data_ptr(), B, L, V, P, H,
                                                     dtype_code(wte.dtype), None, LN_EPS, stats.data_ptr(), _ptr(ext), stream_ptr(dev))
        check(st, "fused_embeddings")
        return z.view((B, L, H)), RowStats(stats[:B * L], H, None if ext is None else ext[:B * L])
    with torch.cuda.device(dev):
        st = _lib.load().b200_embedding(x.data_ptr(), wte.data_ptr(), wpe.data_ptr(), z.data_ptr(), B, L, V, P, H,
                                        dtype_code(wte.dtype), None, stream_ptr(dev))
    check(st, "fused_embeddings")
    return z.view((B, L, H))


# ----------------------------------------------------------------------------- layer norm
@torch.no_grad()
def fused_layer_norm(x, weight, bias, *, out_dtype=None):
    """Row LayerNorm, fp32 statistics, eps 1e-5 (reference kernels.py:149-164)."""
    require_cuda(x, weight, bias)
    assert x.is_contiguous()
    assert weight.is_contiguous()
    assert bias.is_contiguous()
    assert weight.shape == bias.shape
    assert x.shape[-1] == weight.shape[0]
    assert x.dtype == weight.dtype == bias.dtype
    out_shape = x.shape
    H = x.shape[-1]
    M = x.numel() // H if H else 0
    dev = _same_device(x, weight, bias)
    z = torch.empty(x.shape, device=dev, dtype=out_dtype or x.dtype)
    with torch.cuda.device(dev):
        st = _lib.load().b200_layernorm(x.data_ptr(), weight.data_ptr(), bias.data_ptr(), z.data_ptr(), M, H, LN_EPS,
                                        dtype_code(x.dtype), dtype_code(z.dtype), stream_ptr(dev))
    check(st, "fused_layer_norm")
    return z.view(out_shape)


# ----------------------------------------------------------------------------- GEMM
class PackedWeight:
    """A GEMM weight laid out once for the tensor cores: [N, K_padded], 16-bit, K-major.

    ``fused_ffn`` accepts it in place of the [K, N] tensor; the model caches one per
    parameter so the per-call repacking of ``fused_ffn`` disappears from the hot path.
    """

    __slots__ = ("data", "K", "N", "storage_dtype")

    def __init__(self, data, K, N, storage_dtype):
        self.data, self.K, self.N, self.storage_dtype = data, K, N, storage_dtype


@torch.no_grad()
def pack_weight(weight, *, weight_is_nk=False):
    """Round a [K, N] (or, with weight_is_nk, [N, K]) weight to its 16-bit operand type and
    store it [N, K_padded] K-major.  fp32 and fp16 weights become fp16 (the rounding the
    reference applies to every dot operand, kernels.py:234), bf16 stays bf16."""
    require_cuda(weight)
    assert weight.dim() == 2 and weight.is_contiguous()
    K, N = (weight.shape[1], weight.shape[0]) if weight_is_nk else weight.shape
    kp = (K + 7) // 8 * 8
    op_dtype = torch.bfloat16 if weight.dtype == torch.bfloat16 else torch.float16
    if weight_is_nk and weight.dtype == op_dtype and kp == K and weight.data_ptr() % 16 == 0:
        return PackedWeight(weight, K, N, weight.dtype)  # already in operand layout
    dev = weight.device
    packed = torch.empty((N, kp), device=dev, dtype=op_dtype)
    rows, cols = weight.shape
    with torch.cuda.device(dev):
        st = _lib.load().b200_pack_operand(weight.data_ptr(), packed.data_ptr(), rows, cols, cols, kp,
                                           0 if weight_is_nk else 1, dtype_code(weight.dtype), dtype_code(op_dtype),
                                           stream_ptr(dev))
    check(st, "pack_weight")
    return PackedWeight(packed, K, N, weight.dtype)


class FoldedWeight:
    """A (K, N) GEMM weight with the LayerNorm that precedes it folded in (``fold_layer_norm``): ``data`` (N, K)
    K-major 16-bit = LayerNorm weight * weight; ``colsum`` (N,) float32 its column sums and ``bias`` (N,) float32 =
    bias + LayerNorm bias @ weight; ``ext`` (N, 64) the "weight extension" made of the two, which the consuming
    GEMM multiplies as one extra k-block."""

    __slots__ = ("data", "colsum", "bias", "ext", "K", "N", "storage_dtype")

    def __init__(self, data, colsum, bias, ext, K, N, storage_dtype):
        self.data, self.colsum, self.bias, self.ext, self.K, self.N, self.storage_dtype = data, colsum, bias, ext, K, N, storage_dtype


@torch.no_grad()
def fold_layer_norm(weight, ln_weight, ln_bias, bias=None):
    """Fold ``fused_layer_norm(x, ln_weight, ln_bias)`` into the GEMM ``fused_ffn(., weight, bias)`` that follows it
    (reference gpt.py:40-43, 94-101; its author's TODO at kernels.py:132-133):

        LN(x) @ W + b = rstd * (x @ (g * W) - mean * colsum(g * W) + (beta @ W + b) / rstd)

    Returns the FoldedWeight that ``fused_ffn(x, folded, ln_stats=RowStats of x)`` takes.  16-bit dtypes with
    K % 8 == 0 only; done once per weight version, not per forward."""
    require_cuda(weight, ln_weight, ln_bias, bias)
    assert weight.dim() == 2 and weight.is_contiguous() and weight.dtype in (torch.float16, torch.bfloat16)
    K, N = weight.shape
    assert K % 8 == 0, "the folded operand is used in place: K must be a multiple of 8"
    assert ln_weight.shape == (K,) and ln_bias.shape == (K,) and ln_weight.dtype == ln_bias.dtype == weight.dtype
    assert ln_weight.is_contiguous() and ln_bias.is_contiguous()
    if bias is not None:
        assert bias.shape == (N,) and bias.dtype == weight.dtype and bias.is_contiguous()
    dev = _same_device(weight, ln_weight, ln_bias, bias)
    data = torch.empty((N, K), device=dev, dtype=weight.dtype)
    colsum = torch.empty((N,), device=dev, dtype=torch.float32)
    fbias = torch.empty((N,), device=dev, dtype=torch.float32)
    ext = torch.empty((N, LN_EXT_COLS), device=dev, dtype=weight.dtype)
    with torch.cuda.device(dev):
        st = _lib.load().b200_fold_layernorm(weight.data_ptr(), ln_weight.data_ptr(), ln_bias.data_ptr(), _ptr(bias), data.data_ptr(),
                                             colsum.data_ptr(), fbias.data_ptr(), ext.data_ptr(), K, N, K, dtype_code(weight.dtype),
                                             stream_ptr(dev))
    check(st, "fold_layer_norm")
    return FoldedWeight(data, colsum, fbias, ext, K, N, weight.dtype)


def _ffn_layer_norm_aware(x, weight, bias, residual, add_gelu, out, ln_stats, return_row_stats):
    """fused_ffn through b200_gemm_ln: either consuming RowStats (weight a FoldedWeight) or producing them."""
    lead = x.shape[:-1]
    x = x.view((-1, x.shape[-1]))
    M, K = x.shape
    assert isinstance(weight, (FoldedWeight, PackedWeight))
    N = weight.N
    assert K == weight.K and weight.storage_dtype == x.dtype and x.dtype in (torch.float16, torch.bfloat16)
    assert x.is_contiguous() and K % 8 == 0 and x.data_ptr() % 16 == 0
    assert (ln_stats is not None) != bool(return_row_stats), "one launch either consumes or produces row statistics"
    dev = _same_device(x, weight.data, bias, residual)
    z = torch.empty((M, N), device=dev, dtype=x.dtype) if out is None else out
    assert z.shape == (M, N) and z.dtype == x.dtype and z.stride(1) == 1 and z.device == dev
    if residual is not None:
        residual = residual.view((M, N))
        assert residual.is_contiguous() and residual.dtype == x.dtype
    ld_out = z.stride(0) if M > 1 else max(N, z.stride(0))
    lib = _lib.load()
    dt = dtype_code(x.dtype)
    stats_out = None
    with torch.cuda.device(dev):
        if ln_stats is not None:
            assert isinstance(weight, FoldedWeight), "ln_stats needs the FoldedWeight made by fold_layer_norm"
            assert bias is None, "the bias is part of the FoldedWeight"
            assert ln_stats.cols == K and ln_stats.data.shape[0] >= M and ln_stats.data.device == dev and ln_stats.data.is_contiguous()
            assert ln_stats.ext is not None and ln_stats.ext.dtype == x.dtype and ln_stats.ext.is_contiguous() and ln_stats.ext.shape[0] >= M
            st = lib.b200_gemm_ln(x.data_ptr(), weight.data.data_ptr(), None, _ptr(residual), z.data_ptr(), M, N, K, K, weight.data.stride(0),
                                  N, ld_out, dt, dt, int(bool(add_gelu)), ln_stats.data.data_ptr(), ln_stats.ext.data_ptr(),
                                  weight.ext.data_ptr(), None, None, LN_EPS, None, 0, _status_ptr(dev), stream_ptr(dev))
        else:
            assert isinstance(weight, PackedWeight) and not add_gelu
            if bias is not None:
                assert bias.is_contiguous() and bias.shape[0] == N and bias.dtype == x.dtype
            stats_out = torch.empty((max(M, 1), 2), device=dev, dtype=torch.float32)
            ext_out = torch.empty((max(M, 1), LN_EXT_COLS), device=dev, dtype=x.dtype)
            need = lib.b200_gemm_ln_workspace_bytes(M, N)
            ws = torch.empty((max(need, 16),), device=dev, dtype=torch.uint8)
            st = lib.b200_gemm_ln(x.data_ptr(), weight.data.data_ptr(), _ptr(bias), _ptr(residual), z.data_ptr(), M, N, K, K,
                                  weight.data.stride(0), N, ld_out, dtype_code(weight.data.dtype), dt, 0, None, None, None,
                                  stats_out.data_ptr(), ext_out.data_ptr(), LN_EPS, ws.data_ptr(), need, _status_ptr(dev), stream_ptr(dev))
    check(st, "fused_ffn(layer norm)")
    zz = z if out is not None else z.view((*lead, N))
    return (zz, RowStats(stats_out[:M], N, ext_out[:M])) if return_row_stats else zz


@torch.no_grad()
def fused_ffn(x, weight, bias=None, residual=None, add_gelu=False, dropout_prob=0.0, *, weight_is_nk=False, out=None,
              return_argmax=False, return_lse=False, ln_stats=None, return_row_stats=False):
    """z = [gelu_new](x @ weight + bias) + residual  (reference kernels.py:261-315).

    x (*, K); weight (K, N) -- or (N, K) with ``weight_is_nk=True``, or a PackedWeight;
    bias (N,); residual viewable as (M, N).  Returns (*, N) in x.dtype.  ``out`` may be a
    preallocated (M, N) tensor whose rows are strided (last dim contiguous).  With
    ``return_argmax=True`` (needs a PackedWeight and 16-bit operands usable in place) the result
    is ``(z, ids)``, ids (M,) int64 being the argmax over each row of z (lowest column on ties),
    produced by the GEMM's epilogue rather than by a second pass over z; with ``return_lse=True`` as well,
    ``(z, ids, lse)`` where lse (M,) float32 is log(sum_j exp(z[row, j])).

    LayerNorm fusion (16-bit dtypes, N % 8 == 0): with ``ln_stats`` (the RowStats of x's rows) and ``weight`` a
    FoldedWeight, x is the RAW input of a LayerNorm and z = [gelu](LN(x) @ W + b) + residual without the
    normalised tensor; with ``return_row_stats=True`` (``weight`` a PackedWeight, no GELU) the result is
    ``(z, RowStats of z's rows)`` for the next folded GEMM.
    """
    _no_dropout(dropout_prob)
    if ln_stats is not None or return_row_stats:
        assert not (return_argmax or return_lse)
        require_cuda(x, bias, residual)
        return _ffn_layer_norm_aware(x, weight, bias, residual, add_gelu, out, ln_stats, return_row_stats)
    packed = weight if isinstance(weight, PackedWeight) else None
    require_cuda(x, None if packed else weight, bias, residual)
    out_shape_0 = x.shape[:-1]
    x = x.view((-1, x.shape[-1]))
    M, K = x.shape
    if packed is not None:
        N = packed.N
        assert K == packed.K
        assert packed.storage_dtype == x.dtype
    else:
        assert weight.is_contiguous()
        N = weight.shape[0] if weight_is_nk else weight.shape[1]
        assert x.shape[1] == (weight.shape[1] if weight_is_nk else weight.shape[0])
        assert weight.dtype == x.dtype
    assert x.is_contiguous()
    dev = _same_device(x, packed.data if packed else weight, bias, residual)
    if out is None:
        z = torch.empty((M, N), device=dev, dtype=x.dtype)
    else:
        z = out
        assert z.shape == (M, N) and z.dtype == x.dtype and z.stride(1) == 1 and z.device == dev
    if bias is not None:
        assert bias.is_contiguous()
        assert N == bias.shape[0]
        assert bias.dtype == x.dtype
    if residual is not None:
        residual = residual.view((M, N))
        assert residual.is_contiguous()
        assert residual.dtype == x.dtype
    ld_out = z.stride(0) if M > 1 else max(N, z.stride(0))
    lib = _lib.load()
    dt = dtype_code(x.dtype)
    with torch.cuda.device(dev):
        stream = stream_ptr(dev)
        if return_argmax or return_lse:
            assert packed is not None and dt != _lib.F32 and K % 8 == 0 and x.data_ptr() % 16 == 0, \
                "return_argmax needs a PackedWeight and 16-bit, 16-byte aligned activations with K % 8 == 0"
            ids = torch.empty((M,), device=dev, dtype=torch.int64)
            lse = torch.empty((M,), device=dev, dtype=torch.float32) if return_lse else None
            need = lib.b200_gemm_argmax_workspace_bytes(M, N)
            ws = torch.empty((max(need, 16),), device=dev, dtype=torch.uint8)
            if M > 0:  # (an empty tensor has a null data pointer, which the entry point takes for "not requested")
                st = lib.b200_gemm_argmax(x.data_ptr(), packed.data.data_ptr(), _ptr(bias), _ptr(residual), z.data_ptr(), M, N, K, K,
                                          packed.data.stride(0), N, ld_out, dtype_code(packed.data.dtype), dt, int(bool(add_gelu)),
                                          ids.data_ptr(), _ptr(lse), ws.data_ptr(), need, _status_ptr(dev), stream)
                check(st, "fused_ffn(argmax)")
            zz = z if out is not None else z.view((*out_shape_0, N))
            return (zz, ids.view(out_shape_0), lse.view(out_shape_0)) if return_lse else (zz, ids.view(out_shape_0))
        if packed is not None and dt != _lib.F32 and K % 8 == 0 and x.data_ptr() % 16 == 0:
            # operands usable in place: straight to the tensor-core kernel
            st = lib.b200_gemm(x.data_ptr(), packed.data.data_ptr(), _ptr(bias), _ptr(residual), z.data_ptr(), M, N, K, K,
                               packed.data.stride(0), N, ld_out, dtype_code(packed.data.dtype), dt, int(bool(add_gelu)),
                               _status_ptr(dev), stream)
        elif packed is not None:
            # fp32 storage or ragged K: x still has to be rounded/padded into scratch
            kp = packed.data.stride(0)
            xs = torch.empty((M, kp), device=dev, dtype=packed.data.dtype)
            st = lib.b200_pack_operand(x.data_ptr(), xs.data_ptr(), M, K, K, kp, 0, dt, dtype_code(xs.dtype), stream)
            check(st, "fused_ffn(pack x)")
            st = lib.b200_gemm(xs.data_ptr(), packed.data.data_ptr(), _ptr(bias), _ptr(residual), z.data_ptr(), M, N, K, kp,
                               kp, N, ld_out, dtype_code(xs.dtype), dt, int(bool(add_gelu)), _status_ptr(dev), stream)
        else:
            need = lib.b200_ffn_workspace_bytes(M, N, K, int(weight_is_nk), dt)
            # an unaligned x or weight view needs its operand packed too; ask for the worst case then
            if x.data_ptr() % 16 or weight.data_ptr() % 16:
                need = lib.b200_ffn_workspace_bytes(M, N, K, 0, _lib.F32)
            ws = torch.empty((need,), device=dev, dtype=torch.uint8) if need else None
            st = lib.b200_ffn(x.data_ptr(), weight.data_ptr(), _ptr(bias), _ptr(residual), z.data_ptr(), M, N, K, ld_out,
                              int(weight_is_nk), int(bool(add_gelu)), dt, _ptr(ws), need, _status_ptr(dev), stream)
    check(st, "fused_ffn")
    if out is not None:
        return z
    return z.view((*out_shape_0, N))


@torch.no_grad()
def ffn_row_statistics(x, weight, bias=None, targets=None, want_lse=True):
    """Row statistics of z = x @ weight (+ bias) without materialising z (no counterpart in the reference, whose
    lm_head is commented out, gpt.py:172-179): ``(ids, lse, target_value)`` with ids (*,) int64 the argmax of each
    row (lowest column on ties), lse (*,) float32 = log(sum_j exp(z[row, j])) and, when ``targets`` (*,) int64 is
    given, target_value (*,) float32 = z[row, targets[row]] (NaN where the target is outside [0, N); else None) --
    all over z rounded to x.dtype exactly as fused_ffn would store it.  ``want_lse=False`` skips the log-sum-exp
    (lse is None; one exponential per element less).  ``weight`` must be a PackedWeight, x 16-bit with K % 8 == 0."""
    assert isinstance(weight, PackedWeight), "ffn_row_statistics needs a PackedWeight"
    require_cuda(x, bias, targets)
    lead = x.shape[:-1]
    x = x.view((-1, x.shape[-1]))
    M, K = x.shape
    N = weight.N
    dt = dtype_code(x.dtype)
    assert K == weight.K and weight.storage_dtype == x.dtype and x.is_contiguous()
    assert dt != _lib.F32 and K % 8 == 0 and x.data_ptr() % 16 == 0, "16-bit, 16-byte aligned activations with K % 8 == 0 only"
    dev = _same_device(x, weight.data, bias, targets)
    if bias is not None:
        assert bias.is_contiguous() and bias.shape[0] == N and bias.dtype == x.dtype
    ids = torch.empty((M,), device=dev, dtype=torch.int64)
    lse = torch.empty((M,), device=dev, dtype=torch.float32) if want_lse else None
    picked = None
    if targets is not None:
        targets = targets.reshape(-1)
        assert targets.dtype == torch.int64 and targets.is_contiguous() and targets.shape[0] == M
        picked = torch.full((M,), float("nan"), device=dev, dtype=torch.float32)
    if M == 0:
        return ids.view(lead), (lse.view(lead) if want_lse else None), (picked.view(lead) if picked is not None else None)
    lib = _lib.load()
    need = lib.b200_gemm_argmax_workspace_bytes(M, N)
    ws = torch.empty((max(need, 16),), device=dev, dtype=torch.uint8)
    with torch.cuda.device(dev):
        st = lib.b200_gemm_rowstats(x.data_ptr(), weight.data.data_ptr(), _ptr(bias), M, N, K, K, weight.data.stride(0),
                                    dtype_code(weight.data.dtype), dt, _ptr(targets), ids.data_ptr(), _ptr(lse), _ptr(picked),
                                    ws.data_ptr(), need, _status_ptr(dev), stream_ptr(dev))
    check(st, "ffn_row_statistics")
    return ids.view(lead), (lse.view(lead) if want_lse else None), (picked.view(lead) if picked is not None else None)


# ----------------------------------------------------------------------------- qkv split
@torch.no_grad()
def matmul_and_split_qkv(x, weight, bias, num_heads):
    """c_attn projection and head split (reference kernels.py:348-367).

    Returns q, k, v of logical shape (batch, heads, seqlen, head_size) -- as views into the
    single (batch, seqlen, 3*hidden) projection output rather than transposed copies.
    """
    return split_qkv(fused_ffn(x, weight, bias=bias), num_heads)


def split_qkv(x, num_heads):
    """(batch, seqlen, 3 * hidden) projection output -> q, k, v views of logical shape (batch, heads, seqlen,
    head_size): the head split of the reference (kernels.py:355-365) without its three transposed copies."""
    batch_size, seqlen, hidden_size = x.shape
    assert hidden_size % 3 == 0, hidden_size
    hidden_size = hidden_size // 3
    q, k, v = x.split(hidden_size, dim=2)
    assert hidden_size % num_heads == 0, (hidden_size, num_heads)
    head_size = hidden_size // num_heads
    q, k, v = map(lambda t: t.view(batch_size, seqlen, num_heads, head_size).transpose(1, 2), (q, k, v))
    return q, k, v


# ----------------------------------------------------------------------------- attention
def _bhl_strides(t):
    """(batch, head, row) element strides of a (B, N, L, H) tensor whose last dim is contiguous."""
    assert t.stride(3) == 1 or t.shape[3] == 1, "head dimension must be contiguous"
    return (ctypes.c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2))


@torch.no_grad()
def flash_attention_v1(q, k, v, dropout_prob=0.0, *, merged_heads=False):
    """Causal softmax(q k^T / sqrt(H)) v with the reference's 64-key online softmax
    (reference kernels.py:478-525).  q, k, v: (batch, heads, seqlen, head_size), contiguous or
    strided views with a contiguous last dim.  Returns a contiguous (B, N, L, H) tensor, or with
    ``merged_heads=True`` the (B, L, N*H) tensor the reference gets by transposing afterwards
    (gpt.py:51)."""
    _no_dropout(dropout_prob)
    require_cuda(q, k, v)
    assert q.shape[:2] == k.shape[:2]
    assert q.shape[-1] == k.shape[-1]
    assert k.shape == v.shape
    B, N, Lq, H = q.shape
    Lk = k.shape[2]
    assert H in {16, 32, 64, 128, 256}
    assert Lq == Lk, "the causal mask doubles as the padding mask only when Lq == Lk"
    assert q.dtype == k.dtype == v.dtype
    dev = _same_device(q, k, v)
    if merged_heads:
        z = torch.empty((B, Lq, N, H), device=dev, dtype=q.dtype)
        zv = z.transpose(1, 2)
    else:
        z = torch.empty((B, N, Lq, H), device=dev, dtype=q.dtype)
        zv = z
    scale = 1 / math.sqrt(H)
    with torch.cuda.device(dev):
        st = _lib.load().b200_attention(q.data_ptr(), k.data_ptr(), v.data_ptr(), z.data_ptr(), B, N, Lq, H, _bhl_strides(q),
                                        _bhl_strides(k), _bhl_strides(v), _bhl_strides(zv), scale, dtype_code(q.dtype),
                                        dtype_code(z.dtype), _status_ptr(dev), stream_ptr(dev))
    check(st, "flash_attention_v1")
    return z.view(B, Lq, N * H) if merged_heads else z


# ----------------------------------------------------------------------------- token-by-token generation
# No counterpart in the reference (its README.md:55 lists "KV cache + sampling" as not built).  ``pos`` below is a
# CUDA int32 tensor of two elements, {tokens in the cache, prompt length}: the kernels read it on the device, so the
# launches of a decode step can be captured once in a CUDA graph and replayed for every step.
@torch.no_grad()
def kv_cache_fill(qkv, cache):
    """cache[b, l, :] = qkv[b, l, H:3H] for the L positions of a prompt: qkv (B, L, 3H) is the fused c_attn output
    (q | k | v), cache (B, cache_len, 2H) holds k | v.  Both contiguous, same dtype."""
    require_cuda(qkv, cache)
    B, L, H3 = qkv.shape
    H = H3 // 3
    assert H3 == 3 * H and cache.dim() == 3 and cache.shape[0] == B and cache.shape[2] == 2 * H and cache.shape[1] >= L
    assert qkv.is_contiguous() and cache.is_contiguous() and qkv.dtype == cache.dtype
    dev = _same_device(qkv, cache)
    with torch.cuda.device(dev):
        st = _lib.load().b200_kv_cache_fill(qkv.data_ptr(), cache.data_ptr(), B, L, H, cache.shape[1], dtype_code(qkv.dtype), stream_ptr(dev))
    check(st, "kv_cache_fill")
    return cache


@torch.no_grad()
def attention_decode(qkv_new, cache, pos, num_heads):
    """One decode step of causal attention: qkv_new (B, 3H) is q | k | v of the token at position pos[0]; its k, v are
    stored into cache[:, pos[0]] and the result (B, H) is softmax(q K^T / sqrt(D)) V over positions 0..pos[0], with the
    64-key online softmax of the reference's flash_attention_v1 (kernels.py:417-474)."""
    require_cuda(qkv_new, cache, pos)
    B, H3 = qkv_new.shape
    H = H3 // 3
    assert H3 == 3 * H and H % num_heads == 0
    D = H // num_heads
    assert D in (32, 64, 128), f"head size {D}: the decode kernel is built for 32, 64 and 128"
    assert cache.dim() == 3 and cache.shape[0] == B and cache.shape[2] == 2 * H
    assert qkv_new.is_contiguous() and cache.is_contiguous() and qkv_new.dtype == cache.dtype
    assert pos.dtype == torch.int32 and pos.numel() >= 2
    dev = _same_device(qkv_new, cache, pos)
    out = torch.empty((B, H), device=dev, dtype=qkv_new.dtype)
    with torch.cuda.device(dev):
        st = _lib.load().b200_attention_decode(qkv_new.data_ptr(), cache.data_ptr(), out.data_ptr(), B, num_heads, D, cache.shape[1],
                                               1 / math.sqrt(D), dtype_code(qkv_new.dtype), pos.data_ptr(), _status_ptr(dev), stream_ptr(dev))
    check(st, "attention_decode")
    return out


@torch.no_grad()
def decode_append(next_ids, tokens, pos, advance, feedback=None):
    """tokens[:, pos[0] - pos[1] + advance] = next_ids (and feedback[:] = next_ids, the buffer the next decode step
    embeds), then pos[0] += 1 if advance -- all on the device."""
    require_cuda(next_ids, tokens, pos, feedback)
    if feedback is not None:
        assert feedback.dtype == torch.int64 and feedback.is_contiguous() and feedback.numel() == next_ids.numel()
    assert next_ids.dtype == tokens.dtype == torch.int64 and next_ids.is_contiguous() and tokens.dim() == 2 and tokens.stride(1) == 1
    assert tokens.shape[0] == next_ids.numel() and pos.dtype == torch.int32 and pos.numel() >= 2
    dev = _same_device(next_ids, tokens, pos, feedback)
    with torch.cuda.device(dev):
        st = _lib.load().b200_decode_append(next_ids.data_ptr(), tokens.data_ptr(), tokens.stride(0) if tokens.shape[0] > 1 else tokens.shape[1],
                                            tokens.shape[1], tokens.shape[0], pos.data_ptr(), int(bool(advance)), _ptr(feedback), _status_ptr(dev), stream_ptr(dev))
    check(st, "decode_append")


@torch.no_grad()
def sample_logits(logits, temperature=1.0, top_k=0, seed=0, step=None, out=None):
    """One id per row of logits (B, V), drawn from softmax(logits / temperature) over the row's top_k largest logits
    (0 = all; ties with the k-th largest stay in).  Gumbel-max with counter-based uniforms: the same
    (seed, step[0], row) always gives the same id.  ``step``: CUDA int32 tensor read on the device, or None for 0."""
    require_cuda(logits, step)
    assert logits.dim() == 2 and logits.stride(1) == 1 and temperature > 0 and top_k >= 0
    B, V = logits.shape
    dev = _same_device(logits, step)
    ids = torch.empty((B,), device=dev, dtype=torch.int64) if out is None else out
    assert ids.dtype == torch.int64 and ids.is_contiguous() and ids.numel() == B and ids.device == dev
    if step is not None:
        assert step.dtype == torch.int32 and step.numel() >= 1
    with torch.cuda.device(dev):
        st = _lib.load().b200_sample_logits(logits.data_ptr(), logits.stride(0) if B > 1 else V, B, V, dtype_code(logits.dtype), float(temperature),
                                            int(top_k), int(seed) & 0xFFFFFFFFFFFFFFFF, _ptr(step), ids.data_ptr(), stream_ptr(dev))
    check(st, "sample_logits")
    return ids
