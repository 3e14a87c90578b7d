"""GPU tests of the narrow-tile GEMM kernel (one 128 x 64 tile per CTA, taken by products of at most 512 rows): it
must give the wide kernel's bits for the same rows (same operands, same order of k-blocks, same epilogue arithmetic),
and the oracle's fused_ffn (kernels.py:261-315 of the reference) within the 16-bit tolerance."""

import pytest
import torch

from oracle import gpt2_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"
WIDE_ROWS = 640  # more than 512 rows: the wide kernel


def _operands(M, K, N, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((M, K), generator=g).to(dtype)
    w = (torch.randn((K, N), generator=g) * 0.05).to(dtype)
    b = torch.randn(N, generator=g).to(dtype)
    r = torch.randn((M, N), generator=g).to(dtype)
    return x, w, b, r


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows,K,N", [(512, 768, 768), (300, 3072, 768), (8, 768, 2304), (1, 768, 3072), (129, 200, 104), (64, 64, 50257)])
@pytest.mark.parametrize("gelu,res", [(False, False), (True, False), (False, True)])
def test_narrow_tiles_give_the_wide_kernels_bits(dtype, rows, K, N, gelu, res):
    from gpt_triton_b200 import kernels as Kn

    x, w, b, r = _operands(WIDE_ROWS, K, N, dtype, rows + N)
    pw = Kn.pack_weight(w.to(DEV))
    pitch = (N + 63) // 64 * 64  # a padded pitch keeps ragged N on the vector paths of both kernels
    wide = torch.zeros((WIDE_ROWS, pitch), dtype=dtype, device=DEV)
    narrow = torch.zeros((rows, pitch), dtype=dtype, device=DEV)
    rr = torch.zeros((WIDE_ROWS, pitch), dtype=dtype, device=DEV)
    rr[:, :N] = r.to(DEV)
    # (residual rows must be contiguous for the operator: give it an (M, N) tensor when N == pitch, else skip the residual)
    use_res = res and pitch == N
    Kn.fused_ffn(x.to(DEV), pw, bias=b.to(DEV), residual=r.to(DEV) if use_res else None, add_gelu=gelu, out=wide[:, :N])
    Kn.fused_ffn(x[:rows].to(DEV), pw, bias=b.to(DEV), residual=r[:rows].contiguous().to(DEV) if use_res else None, add_gelu=gelu, out=narrow[:, :N])
    assert Kn.device_status() == 0
    assert torch.equal(narrow[:, :N].cpu(), wide[:rows, :N].cpu())
    ref = orc.fused_ffn(x[:rows], w, b, r[:rows] if use_res else None, add_gelu=gelu).float()
    tol = 2e-2 if dtype == torch.float16 else 1.6e-1
    assert (narrow[:, :N].cpu().float() - ref).abs().max().item() < tol * max(1.0, ref.abs().max().item() / 8)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows,H,N2", [(512, 768, 3072), (77, 256, 520), (1, 128, 128)])
def test_narrow_layer_norm_pair_matches_the_wide_kernels(dtype, rows, H, N2):
    """Producer (bias + residual + row statistics) then consumer (LayerNorm folded in, GELU) on few rows against the
    same pair on 640 rows: outputs bit-identical; the statistics agree to rounding (their partial sums run over
    64-column slices in one kernel and 128-column slices in the other)."""
    from gpt_triton_b200 import kernels as Kn

    x, w1, b1, r = _operands(WIDE_ROWS, H, H, dtype, rows)
    g = torch.Generator().manual_seed(rows + 1)
    w2 = (torch.randn((H, N2), generator=g) * 0.05).to(dtype)
    b2 = torch.randn(N2, generator=g).to(dtype)
    gamma = (1 + 0.1 * torch.randn(H, generator=g)).to(dtype)
    beta = (0.1 * torch.randn(H, generator=g)).to(dtype)
    pw1 = Kn.pack_weight(w1.to(DEV))
    fw2 = Kn.fold_layer_norm(w2.to(DEV), gamma.to(DEV), beta.to(DEV), b2.to(DEV))
    yw, sw = Kn.fused_ffn(x.to(DEV), pw1, bias=b1.to(DEV), residual=r.to(DEV), return_row_stats=True)
    yn, sn = Kn.fused_ffn(x[:rows].to(DEV), pw1, bias=b1.to(DEV), residual=r[:rows].contiguous().to(DEV), return_row_stats=True)
    assert torch.equal(yn.cpu(), yw[:rows].cpu())
    assert (sn.mean.cpu() - sw.mean[:rows].cpu()).abs().max().item() < 1e-5
    assert ((sn.rstd.cpu() - sw.rstd[:rows].cpu()).abs() / sw.rstd[:rows].cpu()).max().item() < 1e-5
    # consumer fed the SAME statistics on both sides: bit-identical outputs
    zw = Kn.fused_ffn(yw, fw2, add_gelu=True, ln_stats=sw)
    zn = Kn.fused_ffn(yw[:rows].contiguous(), fw2, add_gelu=True, ln_stats=Kn.RowStats(sw.data[:rows].contiguous(), H, sw.ext[:rows].contiguous()))
    assert Kn.device_status() == 0
    assert torch.equal(zn.cpu(), zw[:rows].cpu())
    # and the pair against the oracle's operator sequence
    yo = orc.fused_ffn(x[:rows], w1, b1, r[:rows])
    zo = orc.fused_ffn(orc.fused_layer_norm(yo, gamma, beta), w2, b2, add_gelu=True).float()
    tol = 3e-2 if dtype == torch.float16 else 2e-1
    zn2 = Kn.fused_ffn(yn, fw2, add_gelu=True, ln_stats=sn)
    assert (zn2.cpu().float() - zo).abs().max().item() < tol
