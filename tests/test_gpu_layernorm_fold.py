"""GPU: LayerNorm folded into the GEMM that follows it (the fusion the reference's author leaves as a TODO,
kernels.py:132-133 of the reference).  The oracle stays the reference's operator sequence (fused_layer_norm, then
fused_ffn, kernels.py:149-164, 261-315): the folded path must match it within a few units in the last place of
the storage type, because it differs by roundings only (the normalised row is not rounded to 16 bits)."""

import pytest
import torch

from conftest import TINY, ulp_tolerance
from oracle import gpt2_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"
# smallest tolerance of a folded GEMM output: the perturbation that dropping one 16-bit rounding of a unit-variance
# row causes in a K ~ 1000 dot product with N(0, 0.02)-sized weights (fp16: ~2e-4, bf16: ~1.5e-3), with margin
FLOOR = {torch.float16: 1.5e-3, torch.bfloat16: 1.2e-2}


def _within(got, ref, dtype, n_ulp, floor):
    return ((got.float() - ref.float()).abs() <= ulp_tolerance(ref, dtype, n_ulp, floor=floor)).all().item()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M,H,offset", [(300, 768, 0.0), (77, 1600, 0.0), (33, 100, 0.0), (129, 768, 100.0), (5, 8, -3.0)])
def test_row_stats_match_torch(dtype, M, H, offset):
    """(mean, rstd) from the row-statistics kernel against float64 torch on the stored values, including rows whose
    mean is a hundred standard deviations away from zero (no cancellation in the sum of squares)."""
    from gpt_triton_b200 import kernels as K

    g = torch.Generator().manual_seed(M * 1000 + H)
    x = (torch.randn((M, H), generator=g) + offset).to(dtype).to(DEV)
    st = K.row_stats(x)
    assert st.data.shape == (M, 2) and st.cols == H
    assert (st.ext is None) if dtype == torch.float32 else (st.ext.shape == (M, 64) and st.ext.dtype == dtype)
    if st.ext is not None:
        # row extension: [-mean, 1 / rstd] as (high, low) pairs, each pair twice, then zeros
        e = st.ext.float()
        assert torch.equal(e[:, 0:2], e[:, 2:4]) and torch.equal(e[:, 4:6], e[:, 6:8]) and not e[:, 8:].any()
        assert torch.allclose(e[:, 0] + e[:, 1], -st.mean, rtol=2e-5, atol=1e-6) and torch.allclose(e[:, 4] + e[:, 5], 1 / st.rstd, rtol=2e-5, atol=1e-6)
    xd = x.double()
    ref_rstd = 1.0 / torch.sqrt(xd.var(-1, unbiased=False) + 1e-5)
    assert (st.mean.double() - xd.mean(-1)).abs().max().item() < 1e-5 * max(1.0, abs(offset))
    assert ((st.rstd.double() - ref_rstd).abs() / ref_rstd).max().item() < 2e-5


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
def test_embedding_stats_are_those_of_the_stored_rows(dtype):
    from gpt_triton_b200 import kernels as K

    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, 500, (3, 70), generator=g).to(DEV)
    wte = torch.randn((500, 264), generator=g).to(dtype).to(DEV)
    wpe = torch.randn((128, 264), generator=g).to(dtype).to(DEV)
    z, st = K.fused_embeddings(ids, wte, wpe, return_row_stats=True)
    assert torch.equal(z, K.fused_embeddings(ids, wte, wpe))
    again = K.row_stats(z)
    assert torch.allclose(st.data, again.data, rtol=1e-5, atol=1e-5)
    if dtype != torch.float32:
        assert torch.allclose(st.ext.float(), again.ext.float(), rtol=1e-2, atol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("M,N,K_", [(300, 768, 768), (515, 1600, 64), (129, 2304, 96), (40, 200, 3072)])
def test_producer_stats_and_unchanged_output(dtype, M, N, K_):
    """fused_ffn(..., return_row_stats=True): the product is bit-identical to the plain call, and the statistics
    (merged from 128-column partial sums, ragged last slice at N = 1600 and 200) are those of the stored rows.
    They are taken before the final rounding, so the match is to rounding noise: 1/sqrt(N) of a unit in the last
    place."""
    from gpt_triton_b200 import kernels as K

    g = torch.Generator().manual_seed(N + K_)
    x = torch.randn((M, K_), generator=g).to(dtype).to(DEV)
    w = (torch.randn((K_, N), generator=g) * 0.05).to(dtype).to(DEV)
    b = torch.randn(N, generator=g).to(dtype).to(DEV)
    r = (torch.randn((M, N), generator=g) * 2 + 1.5).to(dtype).to(DEV)
    pw = K.pack_weight(w)
    plain = K.fused_ffn(x, pw, bias=b, residual=r)
    z, st = K.fused_ffn(x, pw, bias=b, residual=r, return_row_stats=True)
    assert torch.equal(z, plain)
    assert st.cols == N and st.data.shape == (M, 2)
    zd = z.double()
    eps_t = 2.0 ** (-10 if dtype == torch.float16 else -7)
    assert (st.mean.double() - zd.mean(-1)).abs().max().item() < 8.0 * eps_t / (N ** 0.5) + 1e-5
    ref_rstd = 1.0 / torch.sqrt(zd.var(-1, unbiased=False) + 1e-5)
    assert ((st.rstd.double() - ref_rstd).abs() / ref_rstd).max().item() < eps_t / 4


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("gelu", [False, True])
@pytest.mark.parametrize("M,K_,N", [(300, 768, 2304), (300, 768, 3072), (131, 1600, 520), (64, 64, 104), (1, 128, 256)])
def test_folded_gemm_matches_layernorm_then_gemm(dtype, gelu, M, K_, N):
    """fused_ffn(x, FoldedWeight, ln_stats=...) against the oracle's fused_layer_norm -> fused_ffn on the same
    inputs, with non-trivial LayerNorm weight and bias, a bias, and rows with a large common offset."""
    from gpt_triton_b200 import kernels as K

    g = torch.Generator().manual_seed(K_ * 7 + N)
    x = (torch.randn((M, K_), generator=g) * 1.7 + torch.randn((M, 1), generator=g) * 3).to(dtype)
    gamma = (1 + 0.2 * torch.randn(K_, generator=g)).to(dtype)
    beta = (0.3 * torch.randn(K_, generator=g)).to(dtype)
    w = (torch.randn((K_, N), generator=g) * 0.02).to(dtype)
    b = (torch.randn(N, generator=g) * 0.1).to(dtype)
    ref = orc.fused_ffn(orc.fused_layer_norm(x, gamma, beta), w, bias=b, add_gelu=gelu)
    xd, fw = x.to(DEV), K.fold_layer_norm(w.to(DEV), gamma.to(DEV), beta.to(DEV), b.to(DEV))
    assert fw.data.shape == (N, K_) and fw.colsum.shape == (N,) and fw.bias.shape == (N,) and fw.ext.shape == (N, 64)
    we = fw.ext.float()
    assert torch.allclose(we[:, 0] + we[:, 2], fw.colsum, rtol=2e-5, atol=1e-6) and torch.allclose(we[:, 4] + we[:, 6], fw.bias, rtol=2e-5, atol=1e-6)
    assert torch.equal(we[:, 0], we[:, 1]) and torch.equal(we[:, 2], we[:, 3]) and not we[:, 8:].any()
    got = K.fused_ffn(xd, fw, add_gelu=gelu, ln_stats=K.row_stats(xd)).cpu()
    assert got.dtype == dtype and got.shape == ref.shape
    err = (got.float() - ref.float()).abs()
    assert _within(got, ref, dtype, 3.0, FLOOR[dtype] * max(1.0, (K_ / 768) ** 0.5)), err.max().item()
    # and against exact arithmetic the folded form is as close as the reference's own rounding allows
    exact = torch.nn.functional.layer_norm(x.double(), (K_,), gamma.double(), beta.double(), 1e-5) @ w.double() + b.double()
    if gelu:
        exact = 0.5 * exact * (1 + torch.tanh(0.7978845608028654 * (exact + 0.044715 * exact ** 3)))
    assert (got.double() - exact).abs().mean().item() <= 1.5 * (ref.double() - exact).abs().mean().item() + 1e-6


def test_folded_gemm_needs_a_tile_storable_output():
    """The LayerNorm-aware epilogues exist on the staged (TMA-store) path only: an output pitch that is not a multiple
    of 8 elements is refused with B200_ERR_UNSUPPORTED rather than computed some slower way."""
    from gpt_triton_b200 import _lib
    from gpt_triton_b200 import kernels as K

    x = torch.randn((64, 64), device=DEV, dtype=torch.float16)
    w = torch.randn((64, 100), device=DEV, dtype=torch.float16)
    g, b = torch.ones(64, device=DEV, dtype=torch.float16), torch.zeros(64, device=DEV, dtype=torch.float16)
    fw = K.fold_layer_norm(w, g, b, None)
    with pytest.raises(_lib.B200Error, match="not supported"):
        K.fused_ffn(x, fw, ln_stats=K.row_stats(x))
    with pytest.raises(_lib.B200Error, match="not supported"):
        K.fused_ffn(x, K.pack_weight(w), return_row_stats=True)
    torch.cuda.synchronize()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_folded_gemm_takes_statistics_from_a_producer(dtype):
    """Producer -> consumer chain as in a transformer block: c_proj (+ residual) leaves the statistics of the rows
    it stores (13 partial slices at N = 1600, the last one 64 wide), the next GEMM consumes them.  Same result as
    with statistics recomputed from the stored rows, up to single roundings (the producer takes them before the final
    rounding of the rows)."""
    from gpt_triton_b200 import kernels as K

    g = torch.Generator().manual_seed(9)
    h = 1600
    a = torch.randn((260, 320), generator=g).to(dtype).to(DEV)
    w1 = (torch.randn((320, h), generator=g) * 0.05).to(dtype).to(DEV)
    r = torch.randn((260, h), generator=g).to(dtype).to(DEV)
    x, st = K.fused_ffn(a, K.pack_weight(w1), residual=r, return_row_stats=True)
    gamma = (1 + 0.1 * torch.randn(h, generator=g)).to(dtype).to(DEV)
    beta = (0.1 * torch.randn(h, generator=g)).to(dtype).to(DEV)
    w2 = (torch.randn((h, 384), generator=g) * 0.02).to(dtype).to(DEV)
    b2 = (torch.randn(384, generator=g) * 0.1).to(dtype).to(DEV)
    fw = K.fold_layer_norm(w2, gamma, beta, b2)
    via_producer = K.fused_ffn(x, fw, ln_stats=st)
    via_rows = K.fused_ffn(x, fw, ln_stats=K.row_stats(x))
    assert _within(via_producer, via_rows, dtype, 1.0, FLOOR[dtype] / 8)
    ref = orc.fused_ffn(orc.fused_layer_norm(x.cpu(), gamma.cpu(), beta.cpu()), w2.cpu(), bias=b2.cpu())
    assert _within(via_producer.cpu(), ref, dtype, 3.0, FLOOR[dtype] * 1.5)


def _build(cfg_kwargs, dtype, **kw):
    from gpt_triton_b200.gpt import FusedGPT, GPTConfig

    ocfg = orc.OracleConfig(**cfg_kwargs)
    sd = orc.seeded_state_dict(ocfg, seed=0, **kw)
    model = FusedGPT(GPTConfig(**cfg_kwargs))
    model.load_state_dict(sd)
    return model.to(dtype).to(DEV).eval(), ocfg, {k: v.to(dtype) for k, v in sd.items()}


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_blocks_teacher_forced_folded_vs_oracle(dtype):
    """Every block of a 4-layer GPT-2-small-width model, fed the ORACLE's own block input, through the folded path
    (statistics of that input, LayerNorm inside c_attn / ffn1): within 3 units in the last place of the oracle's
    block output, i.e. the fold adds no more than the reference's own rounding noise per block."""
    from gpt_triton_b200 import kernels as K

    kw = dict(vocab_size=1000, block_size=256, n_layer=4, n_head=12, n_embd=768, dropout=0.1)
    model, cfg, sd = _build(kw, dtype, random_affine=True, scale_residual_proj=True)
    ids = torch.randint(0, 1000, (2, 150), generator=torch.Generator().manual_seed(1))
    x = orc.fused_embeddings(ids, sd["wte_weight"], sd["wpe_weight"])
    for i in range(cfg.n_layer):
        ref_a = orc.attention_block(sd, f"blocks.{i}.0.", x, cfg.n_head)
        xd = x.to(DEV)
        got_a, st_a = model.blocks[i][0].forward_folded(xd, K.row_stats(xd))
        assert _within(got_a.cpu(), ref_a, dtype, 3.0, FLOOR[dtype])
        # the statistics the block emits describe the rows it stored
        again = K.row_stats(got_a)
        assert torch.allclose(st_a.mean, again.mean, atol=2e-3 if dtype == torch.bfloat16 else 3e-4) and torch.allclose(st_a.rstd, again.rstd, rtol=2e-3)
        ref_m = orc.mlp_block(sd, f"blocks.{i}.1.", ref_a)
        rd = ref_a.to(DEV)
        got_m, _ = model.blocks[i][1].forward_folded(rd, K.row_stats(rd))
        assert _within(got_m.cpu(), ref_m, dtype, 3.0, FLOOR[dtype])
        x = ref_m


@pytest.mark.parametrize("dtype,tol", [(torch.float16, 2e-2), (torch.bfloat16, 6.3e-2)])
def test_model_folded_vs_unfolded_vs_oracle(dtype, tol):
    """The whole tiny model with non-trivial LayerNorm parameters: folded (default) and operator-by-operator paths
    both sit inside the tolerance of the oracle's logits and agree with each other more closely than that; the
    folded path launches one LayerNorm (the final one) instead of 2 * n_layer + 1."""
    from gpt_triton_b200 import _lib

    model, cfg, sd = _build(TINY, dtype, random_affine=True)
    ids = torch.randint(0, 1024, (3, 100), generator=torch.Generator().manual_seed(1))
    ref = orc.lm_head(sd, orc.gpt_forward(sd, cfg, ids)).float()
    lib = _lib.load()
    model.fold_layer_norm = True
    model.logits(ids.to(DEV))  # packs and folds the weights
    n0 = lib.b200_launch_count()
    folded = model.logits(ids.to(DEV)).cpu().float()
    n_folded = lib.b200_launch_count() - n0
    model.fold_layer_norm = False
    model.logits(ids.to(DEV))
    n0 = lib.b200_launch_count()
    plain = model.logits(ids.to(DEV)).cpu().float()
    n_plain = lib.b200_launch_count() - n0
    # plain: embedding + 7 per layer + final LayerNorm + lm_head; folded: the two LayerNorms of a layer are gone and
    # each of its two residual GEMMs is followed by the small kernel that merges its row statistics (none after the last)
    assert n_plain == 1 + 7 * cfg.n_layer + 2 and n_folded == 1 + 7 * cfg.n_layer - 1 + 2
    assert (folded - ref).abs().max().item() < tol and (plain - ref).abs().max().item() < tol
    assert (folded - plain).abs().max().item() < tol / 2
    top2 = ref.topk(2, dim=-1).values
    clear = (top2[..., 0] - top2[..., 1]) > tol
    assert torch.equal(folded.argmax(-1)[clear], ref.argmax(-1)[clear])


def test_fp32_model_keeps_separate_layernorm():
    """fp32 storage keeps the reference's operator sequence (its 1e-4 per-operator bound leaves no room for the
    fold's re-association), whatever the switch says."""
    from gpt_triton_b200 import _lib

    model, cfg, _ = _build(TINY, torch.float32)
    ids = torch.randint(0, 1024, (2, 64), generator=torch.Generator().manual_seed(0)).to(DEV)
    model(ids)
    n0 = _lib.load().b200_launch_count()
    model(ids)
    # embedding + per layer (LN, pack x, c_attn, attention, pack, c_proj, LN, pack, ffn1, pack, ffn2) + final LN
    assert _lib.load().b200_launch_count() - n0 == 1 + 11 * cfg.n_layer + 1
