"""GPU parity tests, per operator: the sm_100a kernels (called through the C ABI by the
operators of gpt_triton_b200.kernels) against the golden vectors of the unmodified reference and
against the CPU oracle on seeded inputs.

Tolerances.  fp32 storage: max-abs 1e-4 (scaled by max(1, |ref|) for the reference's own GEMM
test inputs, whose outputs reach 80).  fp16/bf16 storage: one unit in the last place or 1e-4
absolute, whichever is larger -- far inside the path's stated 2e-2.  Embeddings: bit-exact."""

import math

import pytest
import torch

from conftest import golden_names, load_golden, ulp_tolerance
from oracle import gpt2_oracle as orc

pytestmark = pytest.mark.gpu

FP32_TOL = 1e-4
DEV = "cuda"


def K():
    import gpt_triton_b200.kernels as k

    return k


def cu(t):
    return None if t is None else t.to(DEV)


ATTN_TOL = 5e-4  # see test_attention_vs_oracle


def assert_close(z, ref, scale_big=True, n_ulp=1.0, floor=FP32_TOL):
    z = z.detach().cpu()
    assert z.dtype == ref.dtype and z.shape == ref.shape, (z.dtype, ref.dtype, z.shape, ref.shape)
    assert torch.isfinite(z.float()).all()
    d = (z.float() - ref.float()).abs()
    if ref.dtype == torch.float32:
        tol = floor * (torch.clamp(ref.abs(), min=1.0) if scale_big else torch.ones_like(ref))
    else:
        tol = ulp_tolerance(torch.maximum(ref.float().abs(), z.float().abs()), ref.dtype, n_ulp, floor=floor)
    bad = d > tol
    assert not bad.any(), f"max|d|={d.max().item():.3e}, {int(bad.sum())} of {d.numel()} elements out of tolerance"


# ----------------------------------------------------------------------------- embeddings
@pytest.mark.parametrize("name", golden_names("emb_"))
def test_embeddings_golden(name):
    g = load_golden(name)
    z = K().fused_embeddings(cu(g["x"]), cu(g["wte"]), cu(g["wpe"]))
    assert torch.equal(z.cpu(), g["z"])


@pytest.mark.parametrize("vocab_size", [2, 32])
@pytest.mark.parametrize("hidden_size", [32, 128, 256, 123])
@pytest.mark.parametrize("seqlen,block_size", [(10, 20), (20, 20)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_embeddings_reference_shapes(vocab_size, hidden_size, seqlen, block_size, dtype):
    """Shapes of the reference's test (test.py:28-44) plus an odd hidden size, all dtypes; exact."""
    g = torch.Generator().manual_seed(vocab_size * 1000 + hidden_size + seqlen)
    x = torch.randint(0, vocab_size, (8, seqlen), generator=g)
    wte = torch.rand((vocab_size, hidden_size), generator=g).to(dtype)
    wpe = torch.rand((block_size, hidden_size), generator=g).to(dtype)
    z = K().fused_embeddings(cu(x), cu(wte), cu(wpe))
    assert torch.equal(z.cpu(), orc.fused_embeddings(x, wte, wpe))


def test_embeddings_int32_ids_and_asserts():
    x = torch.randint(0, 50, (3, 7), dtype=torch.int32)
    wte, wpe = torch.rand(50, 64), torch.rand(7, 64)
    z = K().fused_embeddings(cu(x), cu(wte), cu(wpe))
    assert torch.equal(z.cpu(), orc.fused_embeddings(x.long(), wte, wpe))
    with pytest.raises(AssertionError):
        K().fused_embeddings(cu(torch.zeros((1, 9), dtype=torch.long)), cu(wte), cu(wpe))  # L > block_size
    with pytest.raises(NotImplementedError):
        K().fused_embeddings(cu(x), cu(wte), cu(wpe), dropout_prob=0.1)


def test_embeddings_full_size_fp16():
    """153600 x 768 fp16 (the benchmark batch): exact against the oracle on a strided row sample,
    and position-periodic: rows t and t + L of the same id carry the same position vector."""
    g = torch.Generator().manual_seed(0)
    B, L, V, H = 512, 300, 50257, 768
    x = torch.randint(0, V, (B, L), generator=g)
    wte = (torch.randn((V, H), generator=g) * 0.02).half()
    wpe = (torch.randn((1024, H), generator=g) * 0.02).half()
    z = K().fused_embeddings(cu(x), cu(wte), cu(wpe)).cpu()
    rows = torch.arange(0, B, 37)
    assert torch.equal(z[rows], orc.fused_embeddings(x[rows], wte, wpe))


# ----------------------------------------------------------------------------- layer norm
@pytest.mark.parametrize("name", golden_names("ln_"))
def test_layer_norm_golden(name):
    g = load_golden(name)
    assert_close(K().fused_layer_norm(cu(g["x"]), cu(g["w"]), cu(g["b"])), g["z"], scale_big=False)


@pytest.mark.parametrize("M", [249, 32, 1])
@pytest.mark.parametrize("H", [123, 128, 64, 768, 1024, 1600, 4096, 5000, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_layer_norm_vs_oracle(M, H, dtype):
    g = torch.Generator().manual_seed(M * 7 + H)
    x = (torch.randn((M, H), generator=g) * 2 + 0.5).to(dtype)
    w = (1 + 0.3 * torch.randn(H, generator=g)).to(dtype)
    b = (0.2 * torch.randn(H, generator=g)).to(dtype)
    assert_close(K().fused_layer_norm(cu(x), cu(w), cu(b)), orc.fused_layer_norm(x, w, b), scale_big=False)


def test_layer_norm_3d_and_fp32_to_fp16():
    g = torch.Generator().manual_seed(3)
    x = torch.randn((2, 5, 128), generator=g)
    w, b = torch.rand(128, generator=g), torch.rand(128, generator=g)
    z = K().fused_layer_norm(cu(x), cu(w), cu(b))
    assert z.shape == x.shape
    assert_close(z, orc.fused_layer_norm(x, w, b), scale_big=False)
    z16 = K().fused_layer_norm(cu(x), cu(w), cu(b), out_dtype=torch.float16)
    assert_close(z16, orc.fused_layer_norm(x, w, b).half(), scale_big=False)


def test_layer_norm_full_size_fp16():
    """153600 x 768 fp16, gamma 1, beta 0: oracle parity on a row sample; every row of the output
    has mean ~ 0 and variance ~ 1 (size-independent property)."""
    g = torch.Generator().manual_seed(0)
    x = torch.randn((153600, 768), generator=g).half()
    w, b = torch.ones(768).half(), torch.zeros(768).half()
    z = K().fused_layer_norm(cu(x), cu(w), cu(b))
    rows = torch.arange(0, 153600, 997)
    assert_close(z[rows.to(DEV)], orc.fused_layer_norm(x[rows], w, b), scale_big=False)
    zf = z.float()
    assert zf.mean(dim=1).abs().max().item() < 2e-3
    assert (zf.var(dim=1, unbiased=False) - 1).abs().max().item() < 5e-3


# ----------------------------------------------------------------------------- GEMM
@pytest.mark.parametrize("name", golden_names("ffn_"))
def test_ffn_golden(name):
    g = load_golden(name)
    gelu = "_g1" in name or name.endswith("_gelu")
    bias = None if "_b0" in name else g["b"]
    res = g.get("r") if not name.endswith("_gelu") else None
    z = K().fused_ffn(cu(g["x"]), cu(g["w"]), bias=cu(bias), residual=cu(res), add_gelu=gelu)
    assert_close(z, g["z"])


def _ffn_inputs(M, N, K_, dtype, seed, act_scale=1.0, w_scale=0.05, with_res=True):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn((M, K_), generator=g) * act_scale).to(dtype)
    w = (torch.randn((K_, N), generator=g) * w_scale).to(dtype)
    b = (torch.randn(N, generator=g) * 0.1).to(dtype)
    r = torch.randn((M, N), generator=g).to(dtype) if with_res else None
    return x, w, b, r


@pytest.mark.parametrize("M,N,K_", [(128, 128, 256), (199, 129, 129), (61, 31, 23), (1, 8, 8), (300, 520, 72), (257, 1000, 1096)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("add_gelu,use_bias,use_res", [(True, True, False), (False, True, True), (False, False, False), (True, False, True)])
def test_ffn_vs_oracle(M, N, K_, dtype, add_gelu, use_bias, use_res):
    """The reference's test shapes (test.py:72) and ragged multi-tile shapes, every epilogue."""
    x, w, b, r = _ffn_inputs(M, N, K_, dtype, seed=M + N + K_)
    z = K().fused_ffn(cu(x), cu(w), bias=cu(b) if use_bias else None, residual=cu(r) if use_res else None, add_gelu=add_gelu)
    ref = orc.fused_ffn(x, w, b if use_bias else None, r if use_res else None, add_gelu)
    assert_close(z, ref)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
def test_ffn_many_tiles_per_cta(dtype):
    """More tiles than SMs (157 x 9 = 1413): exercises the persistent loop, the 4-stage ring's
    phase flips and both accumulator buffers."""
    x, w, b, r = _ffn_inputs(20000, 2304, 768, dtype, seed=5, w_scale=0.02, with_res=False)
    z = K().fused_ffn(cu(x), cu(w), bias=cu(b), add_gelu=True)
    rows = torch.cat([torch.arange(0, 300), torch.arange(9000, 9300), torch.arange(19800, 20000)])
    assert_close(z[rows.to(DEV)], orc.fused_ffn(x[rows], w, b, None, True))
    # every row against a same-precision torch matmul on the GPU
    ref = torch.nn.functional.gelu((cu(x).half().float() @ cu(w).half().float()) + cu(b).float(), approximate="tanh")
    assert (z.float() - ref).abs().max().item() < (2e-4 if dtype == torch.float32 else 2e-2)


def test_ffn_weight_layouts_and_packed():
    """[N, K] weights (the tied lm_head operand), PackedWeight, 3-D inputs and a strided `out`."""
    k = K()
    x, w, b, r = _ffn_inputs(2 * 77, 200, 64, torch.float16, seed=9)
    ref = orc.fused_ffn(x, w, b, r, False)
    assert_close(k.fused_ffn(cu(x), cu(w.T.contiguous()), bias=cu(b), residual=cu(r), weight_is_nk=True), ref)
    pw = k.pack_weight(cu(w))
    assert_close(k.fused_ffn(cu(x), pw, bias=cu(b), residual=cu(r)), ref)
    z3 = k.fused_ffn(cu(x).view(2, 77, 64), cu(w), bias=cu(b), residual=cu(r).view(2, 77, 200))
    assert z3.shape == (2, 77, 200)
    assert_close(z3.view(154, 200), ref)
    buf = torch.zeros((154, 208), device=DEV, dtype=torch.float16)
    k.fused_ffn(cu(x), pw, bias=cu(b), residual=cu(r), out=buf[:, :200])
    assert_close(buf[:, :200], ref)
    assert buf[:, 200:].abs().max().item() == 0  # padding untouched
    # odd N with a padded pitch, as the lm_head uses (vocab 50257 -> pitch 50264)
    x2, w2, _, _ = _ffn_inputs(130, 1001, 128, torch.float16, seed=10)
    buf2 = torch.zeros((130, 1008), device=DEV, dtype=torch.float16)
    k.fused_ffn(cu(x2), k.pack_weight(cu(w2.T.contiguous()), weight_is_nk=True), out=buf2[:, :1001])
    assert_close(buf2[:, :1001], orc.fused_ffn(x2, w2))
    assert buf2[:, 1001:].abs().max().item() == 0


def _first_argmax(z):
    """Lowest column holding the row maximum (what the fused argmax promises)."""
    zf = z.float().cpu()
    is_max = zf == zf.max(dim=1, keepdim=True).values
    cols = torch.arange(zf.shape[1]).expand_as(zf)
    return torch.where(is_max, cols, torch.full_like(cols, zf.shape[1])).min(dim=1).values


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("M,N,K_", [(300, 1001, 128), (1, 8, 8), (1000, 50257, 64), (129, 256, 72)])
def test_ffn_fused_argmax(M, N, K_, dtype):
    """Row argmax out of the GEMM epilogue == first-occurrence argmax of the stored output, including
    ragged N, many column slices (vocabulary-sized N) and rows full of ties (coarse values)."""
    k = K()
    g = torch.Generator().manual_seed(M + N)
    x = (torch.randn((M, K_), generator=g) * 0.5).to(dtype)
    w = torch.randint(-2, 3, (N, K_), generator=g).to(dtype) * 0.25  # coarse weights -> many exact ties
    pw = k.pack_weight(cu(w), weight_is_nk=True)
    pitch = (N + 63) // 64 * 64
    buf = torch.zeros((M, pitch), device=DEV, dtype=dtype)
    z, ids, lse = k.fused_ffn(cu(x), pw, out=buf[:, :N], return_argmax=True, return_lse=True)
    assert ids.shape == (M,) and ids.dtype == torch.int64
    ref_lse = torch.logsumexp(z.float(), dim=1)
    assert (lse - ref_lse).abs().max().item() < 1e-4 * max(1.0, ref_lse.abs().max().item())
    z2, ids2 = k.fused_ffn(cu(x), pw, return_argmax=True)
    assert torch.equal(ids2, ids) and torch.equal(z2, z)
    assert_close(z, orc.fused_ffn(x, w.T.contiguous()))
    assert torch.equal(ids.cpu(), _first_argmax(z))
    plain = k.fused_ffn(cu(x), pw)
    assert torch.equal(plain, z)  # asking for the argmax does not change the output


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("M,N,K_,use_bias", [(300, 1001, 128, False), (1, 8, 8, True), (1000, 50257, 64, False), (129, 256, 72, True),
                                             (513, 700, 768, True)])
def test_ffn_row_statistics_without_the_product(M, N, K_, use_bias, dtype):
    """Argmax, log-sum-exp and the value at a per-row target column, taken in the GEMM epilogue with nothing of
    size M x N written: bit-identical to the same statistics of the product that fused_ffn stores (ties, ragged N,
    vocabulary-sized N, bias), NaN where a target is out of range."""
    k = K()
    g = torch.Generator().manual_seed(M * 7 + N)
    x = (torch.randn((M, K_), generator=g) * 0.5).to(dtype)
    w = torch.randint(-2, 3, (N, K_), generator=g).to(dtype) * 0.25  # coarse weights -> many exact ties
    b = torch.randn((N,), generator=g).to(dtype) if use_bias else None
    tgt = torch.randint(0, N, (M,), generator=g)
    tgt[0] = N - 1
    if M > 2:
        tgt[1], tgt[2] = -1, N  # outside [0, N)
    pw = k.pack_weight(cu(w), weight_is_nk=True)
    z, ids_ref, lse_ref = k.fused_ffn(cu(x), pw, bias=cu(b), return_argmax=True, return_lse=True)
    ids, lse, picked = k.ffn_row_statistics(cu(x), pw, bias=cu(b), targets=cu(tgt))
    assert ids.shape == (M,) and ids.dtype == torch.int64 and lse.dtype == torch.float32 and picked.dtype == torch.float32
    assert torch.equal(ids, ids_ref)
    assert torch.equal(ids.cpu(), _first_argmax(z))
    assert (lse - lse_ref).abs().max().item() <= 1e-6 * max(1.0, lse_ref.abs().max().item())
    ok = (tgt >= 0) & (tgt < N)
    want = z.float().cpu().gather(1, tgt.clamp(0, N - 1)[:, None])[:, 0]
    assert torch.equal(picked.cpu()[ok], want[ok])
    assert torch.isnan(picked.cpu()[~ok]).all()
    ids2, lse2, none = k.ffn_row_statistics(cu(x), pw, bias=cu(b))
    assert none is None and torch.equal(ids2, ids) and torch.equal(lse2, lse)
    ids3, none_lse, _ = k.ffn_row_statistics(cu(x), pw, bias=cu(b), want_lse=False)
    assert none_lse is None and torch.equal(ids3, ids)
    # leading dimensions are kept
    if M % 3 == 0:
        i3, l3, p3 = k.ffn_row_statistics(cu(x).view(3, M // 3, K_), pw, bias=cu(b), targets=cu(tgt).view(3, M // 3))
        assert i3.shape == (3, M // 3) and torch.equal(i3.view(-1), ids) and torch.equal(p3.view(-1)[cu(ok)], picked[cu(ok)])


def test_ffn_row_statistics_asserts():
    k = K()
    x = torch.zeros((4, 64), device=DEV, dtype=torch.float16)
    w = torch.zeros((64, 32), device=DEV, dtype=torch.float16)
    with pytest.raises(AssertionError):
        k.ffn_row_statistics(x, w)  # needs a PackedWeight
    with pytest.raises(AssertionError):
        k.ffn_row_statistics(x.float(), k.pack_weight(w.float()))  # 16-bit only
    with pytest.raises(AssertionError):
        k.ffn_row_statistics(x, k.pack_weight(w), targets=torch.zeros((3,), device=DEV, dtype=torch.int64))


def test_ffn_full_size_fp16_gelu():
    """The kernel-sweep GEMM: M=153600, K=768, N=3072, fp16, bias + GELU.  Oracle parity on a row
    sample, and row independence: the same rows computed as a small problem give the same bits."""
    x, w, b, _ = _ffn_inputs(153600, 3072, 768, torch.float16, seed=0, w_scale=0.02, with_res=False)
    k = K()
    pw = k.pack_weight(cu(w))
    z = k.fused_ffn(cu(x), pw, bias=cu(b), add_gelu=True)
    rows = torch.cat([torch.arange(0, 64), torch.arange(77777, 77777 + 64), torch.arange(153600 - 64, 153600)])
    assert_close(z[rows.to(DEV)], orc.fused_ffn(x[rows], w, b, None, True))
    small = k.fused_ffn(cu(x[rows]), pw, bias=cu(b), add_gelu=True)
    assert torch.equal(small, z[rows.to(DEV)])


def test_ffn_asserts():
    k = K()
    x, w = torch.rand(4, 8, device=DEV), torch.rand(9, 8, device=DEV)
    with pytest.raises(AssertionError):
        k.fused_ffn(x, w)
    with pytest.raises(NotImplementedError):
        k.fused_ffn(x, torch.rand(8, 8, device=DEV), dropout_prob=0.5)
    with pytest.raises(RuntimeError):
        k.fused_ffn(torch.rand(4, 8), torch.rand(8, 8))


# ----------------------------------------------------------------------------- attention
@pytest.mark.parametrize("name", golden_names("attn_"))
def test_attention_golden(name):
    g = load_golden(name)
    assert_close(K().flash_attention_v1(cu(g["q"]), cu(g["k"]), cu(g["v"])), g["z"], scale_big=False)


@pytest.mark.parametrize("B,N", [(3, 9), (2, 7)])
@pytest.mark.parametrize("L", [199, 128, 63, 1, 300])
@pytest.mark.parametrize("H", [16, 32, 64, 128, 256])
@pytest.mark.parametrize("dtype,dist", [(torch.float32, "rand"), (torch.float32, "randn"), (torch.float16, "randn"), (torch.bfloat16, "randn")])
def test_attention_vs_oracle(B, N, L, H, dtype, dist):
    """The reference's test grid (test.py:90-117: uniform [0,1) inputs) widened to every supported
    head size and dtype, plus unit-normal inputs.  Tolerance against the oracle: 5e-4 absolute
    (fp32), or one 16-bit ulp if that is larger.  The golden-vector test above holds 1e-4 on the
    reference's own outputs; on arbitrary seeded inputs the bound is set by the algorithm, not the
    implementation: P is rounded to fp16, so a last-bit difference in an fp32 score (another
    summation order in QK^T) can flip one rounding of P by 2^-11 relative, and on a row with few
    keys or a peaked softmax that single flip moves the output by 1e-4..5e-4."""
    if (B, N) == (3, 9) and dtype != torch.float32:
        pytest.skip("one batch/head pair per 16-bit dtype is enough")
    g = torch.Generator().manual_seed(L * 1000 + H)
    draw = torch.rand if dist == "rand" else torch.randn
    q, k, v = (draw((B, N, L, H), generator=g).to(dtype) for _ in range(3))
    z = K().flash_attention_v1(cu(q), cu(k), cu(v))
    assert_close(z, orc.flash_attention_v1(q, k, v), scale_big=False, floor=ATTN_TOL)


@pytest.mark.parametrize("B,N,L", [(2, 3, 300), (1, 2, 64), (1, 1, 129), (3, 2, 1000), (1, 12, 1), (2, 2, 128)])
@pytest.mark.parametrize("layout", ["contiguous", "fused_qkv"])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_attention_tensor_core_path_16bit(B, N, L, layout, dtype):
    """Head size 64, fp16/bf16: the tcgen05/TMA kernel, from contiguous [B, N, L, 64] tensors and from
    strided views of a fused [B, L, 3*N*64] projection, writing contiguous and merged-head output."""
    g = torch.Generator().manual_seed(B * 100 + L)
    if layout == "contiguous":
        q, k, v = (torch.randn((B, N, L, 64), generator=g).to(dtype) for _ in range(3))
        qc, kc, vc = cu(q), cu(k), cu(v)
    else:
        qkv = torch.randn((B, L, 3 * N * 64), generator=g).to(dtype)
        q, k, v = (t.reshape(B, L, N, 64).transpose(1, 2) for t in qkv.split(N * 64, dim=2))
        qc, kc, vc = (t.reshape(B, L, N, 64).transpose(1, 2) for t in cu(qkv).split(N * 64, dim=2))
    ref = orc.flash_attention_v1(q.contiguous(), k.contiguous(), v.contiguous())
    assert_close(K().flash_attention_v1(qc, kc, vc), ref, scale_big=False, floor=ATTN_TOL)
    merged = K().flash_attention_v1(qc, kc, vc, merged_heads=True)
    assert_close(merged, ref.transpose(1, 2).reshape(B, L, N * 64), scale_big=False, floor=ATTN_TOL)


def test_qkv_split_views_and_merged_heads():
    k = K()
    g = load_golden("qkv_f32")
    q, kk, v = k.matmul_and_split_qkv(cu(g["x"]), cu(g["w"]), cu(g["b"]), 4)
    for a, b in ((q, g["q"]), (kk, g["k"]), (v, g["v"])):
        assert a.shape == b.shape
        assert_close(a.contiguous(), b, scale_big=False)
    # attention straight from such strided views (head size 16, fp32); merged-head output equals transpose+reshape
    gen = torch.Generator().manual_seed(21)
    x = torch.randn((2, 70, 64), generator=gen)
    w = 0.2 * torch.randn((64, 192), generator=gen)
    b = 0.1 * torch.randn(192, generator=gen)
    q, kk, v = k.matmul_and_split_qkv(cu(x), cu(w), cu(b), 4)
    assert not q.is_contiguous() and q.shape == (2, 4, 70, 16)
    # same q, k, v on both sides: differences in the projection's last bit would otherwise flip fp16 operand roundings
    ref = orc.flash_attention_v1(q.cpu().contiguous(), kk.cpu().contiguous(), v.cpu().contiguous())
    assert_close(k.flash_attention_v1(q, kk, v), ref, scale_big=False, floor=ATTN_TOL)
    merged = k.flash_attention_v1(q, kk, v, merged_heads=True)
    B, N, L, H = ref.shape
    assert_close(merged, ref.transpose(1, 2).reshape(B, L, N * H), scale_big=False, floor=ATTN_TOL)


@pytest.mark.parametrize("S", [300, 1024])
def test_attention_sweep_shapes_fp16(S):
    """Kernel-sweep attention (H=12, D=64, q,k,v ~ N(0,1)/8) on a batch slice: oracle parity, and
    causality: outputs for the first 100 rows do not change when later keys/values change."""
    g = torch.Generator().manual_seed(0)
    B = 8
    q, k, v = ((torch.randn((B, 12, S, 64), generator=g) / 8).half() for _ in range(3))
    z = K().flash_attention_v1(cu(q), cu(k), cu(v))
    assert_close(z[:2], orc.flash_attention_v1(q[:2], k[:2], v[:2]), scale_big=False, floor=ATTN_TOL)
    k2, v2 = k.clone(), v.clone()
    k2[:, :, 100:] = 0.5
    v2[:, :, 100:] = -3.0
    z2 = K().flash_attention_v1(cu(q), cu(k2), cu(v2))
    assert torch.equal(z[:, :, :100], z2[:, :, :100])


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("layout", ["contiguous", "fused_qkv"])
def test_attention_seq_2048_vs_oracle(dtype, layout):
    """The longest kernel-sweep sequence, S = 2048 (B=2, H=12, D=64): 16 query tiles per (batch, head) and up to 32
    key blocks per tile, i.e. the longest chain of online-softmax rescales and the deepest longest-first work
    ordering the tensor-core kernel sees; every output row against the oracle."""
    g = torch.Generator().manual_seed(2048)
    B, N, S = 2, 12, 2048
    if layout == "contiguous":
        q, k, v = ((torch.randn((B, N, S, 64), generator=g) / 8).to(dtype) for _ in range(3))
        qc, kc, vc = cu(q), cu(k), cu(v)
    else:
        qkv = (torch.randn((B, S, 3 * N * 64), generator=g) / 8).to(dtype)
        q, k, v = (t.reshape(B, S, N, 64).transpose(1, 2) for t in qkv.split(N * 64, dim=2))
        qc, kc, vc = (t.reshape(B, S, N, 64).transpose(1, 2) for t in cu(qkv).split(N * 64, dim=2))
    ref = orc.flash_attention_v1(q.contiguous(), k.contiguous(), v.contiguous())
    z = K().flash_attention_v1(qc, kc, vc)
    assert_close(z, ref, scale_big=False, floor=ATTN_TOL)
    merged = K().flash_attention_v1(qc, kc, vc, merged_heads=True)
    assert torch.equal(merged.view(B, S, N, 64).transpose(1, 2), z)
    # N(0,1) scores (16 times the variance): peaked rows, frequent changes of the running maximum
    q2 = (q.float() * 8).to(dtype).contiguous()
    ref2 = orc.flash_attention_v1(q2, k.contiguous(), v.contiguous())
    assert_close(K().flash_attention_v1(cu(q2), kc, vc), ref2, scale_big=False, floor=ATTN_TOL)


def test_attention_asserts():
    k = K()
    q = torch.rand(1, 2, 8, 24, device=DEV)
    with pytest.raises(AssertionError):
        k.flash_attention_v1(q, q, q)  # head size not in {16, 32, 64, 128, 256}
    q = torch.rand(1, 2, 8, 32, device=DEV)
    with pytest.raises(NotImplementedError):
        k.flash_attention_v1(q, q, q, dropout_prob=0.1)


# ----------------------------------------------------------------------------- edge cases
def test_empty_inputs_are_no_ops():
    k = K()
    wte, wpe = torch.rand(10, 64, device=DEV), torch.rand(8, 64, device=DEV)
    assert k.fused_embeddings(torch.zeros((0, 5), dtype=torch.long, device=DEV), wte, wpe).shape == (0, 5, 64)
    assert k.fused_layer_norm(torch.zeros((0, 64), device=DEV), torch.ones(64, device=DEV), torch.zeros(64, device=DEV)).shape == (0, 64)
    assert k.fused_ffn(torch.zeros((0, 64), device=DEV), torch.rand(64, 32, device=DEV)).shape == (0, 32)
    q = torch.zeros((0, 2, 7, 64), device=DEV, dtype=torch.float16)
    assert k.flash_attention_v1(q, q, q).shape == (0, 2, 7, 64)
    pw = k.pack_weight(torch.rand(64, 32, device=DEV).half())
    ids, lse, picked = k.ffn_row_statistics(torch.zeros((0, 64), device=DEV, dtype=torch.float16), pw,
                                            targets=torch.zeros((0,), dtype=torch.long, device=DEV))
    assert ids.shape == (0,) and lse.shape == (0,) and picked.shape == (0,)
    z, ids = k.fused_ffn(torch.zeros((0, 64), device=DEV, dtype=torch.float16), pw, return_argmax=True)
    assert z.shape == (0, 32) and ids.shape == (0,)
    torch.cuda.synchronize()


def test_single_token_and_single_row():
    k = K()
    g = torch.Generator().manual_seed(5)
    for dtype in (torch.float32, torch.float16):
        q, kk, v = (torch.randn((2, 3, 1, 64), generator=g).to(dtype) for _ in range(3))
        z = k.flash_attention_v1(cu(q), cu(kk), cu(v))
        assert_close(z, v.half().to(dtype), scale_big=False)  # one key: softmax is 1, output is the fp16-rounded v
        assert_close(z, orc.flash_attention_v1(q, kk, v), scale_big=False)
        x, w, b, _ = _ffn_inputs(1, 768, 768, dtype, seed=3)
        assert_close(k.fused_ffn(cu(x), cu(w), bias=cu(b), add_gelu=True), orc.fused_ffn(x, w, b, None, True))


def test_non_contiguous_inputs_are_rejected_like_the_reference():
    k = K()
    x = torch.rand(8, 16, device=DEV)
    with pytest.raises(AssertionError):
        k.fused_layer_norm(x.t(), torch.ones(8, device=DEV), torch.zeros(8, device=DEV))
    with pytest.raises(AssertionError):
        k.fused_embeddings(torch.zeros((4, 6), dtype=torch.long, device=DEV).t(), torch.rand(4, 8, device=DEV), torch.rand(8, 8, device=DEV))
    with pytest.raises(AssertionError):
        k.fused_ffn(x, torch.rand(8, 16, device=DEV).t())


# ----------------------------------------------------------------------------- seeded random shapes
def test_ffn_random_shapes_all_epilogues():
    """40 seeded random (M, N, K, dtype, epilogue) problems, ragged in every dimension, both kernel variants
    (single CTA for M <= 128, CTA pair above), TMA and register epilogues (N or K not multiples of 8)."""
    rng = torch.Generator().manual_seed(2024)
    k = K()
    for case in range(40):
        M = int(torch.randint(1, 700, (1,), generator=rng))
        N = int(torch.randint(1, 900, (1,), generator=rng))
        K_ = int(torch.randint(1, 400, (1,), generator=rng))
        if case % 3 == 0:
            N, K_ = (N + 7) // 8 * 8, (K_ + 7) // 8 * 8  # aligned: operands in place, TMA epilogue
        dtype = (torch.float16, torch.bfloat16, torch.float32)[case % 3 if case % 5 else 0]
        gelu, use_b, use_r = bool(case & 1), bool(case & 2), bool(case & 4)
        x, w, b, r = _ffn_inputs(M, N, K_, dtype, seed=1000 + case)
        z = k.fused_ffn(cu(x), cu(w), bias=cu(b) if use_b else None, residual=cu(r) if use_r else None, add_gelu=gelu)
        ref = orc.fused_ffn(x, w, b if use_b else None, r if use_r else None, gelu)
        try:
            assert_close(z, ref)
        except AssertionError as e:
            raise AssertionError(f"case {case}: M={M} N={N} K={K_} {dtype} gelu={gelu} bias={use_b} res={use_r}: {e}") from None


def test_attention_random_shapes():
    """24 seeded random (B, heads, L, head size, dtype) problems against the oracle."""
    rng = torch.Generator().manual_seed(77)
    k = K()
    for case in range(24):
        B = int(torch.randint(1, 4, (1,), generator=rng))
        N = int(torch.randint(1, 5, (1,), generator=rng))
        L = int(torch.randint(1, 520, (1,), generator=rng))
        H = (64, 64, 32, 16, 128)[case % 5]
        dtype = (torch.float16, torch.bfloat16, torch.float32)[case % 3]
        q, kk, v = (torch.randn((B, N, L, H), generator=rng).to(dtype) for _ in range(3))
        z = k.flash_attention_v1(cu(q), cu(kk), cu(v))
        try:
            assert_close(z, orc.flash_attention_v1(q, kk, v), scale_big=False, floor=ATTN_TOL)
        except AssertionError as e:
            raise AssertionError(f"case {case}: B={B} N={N} L={L} H={H} {dtype}: {e}") from None
