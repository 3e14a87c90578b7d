"""CPU: pins the oracle (oracle/gpt2_oracle.py) to the golden vectors produced by the
unmodified reference under Triton's interpreter (tests/golden/make_golden.py).

Tolerances: fp32 outputs max-abs 1e-4 per kernel (the hot path's stated fp32 tolerance; the
measured gaps are 1e-7..6e-5, summation order only); fp16/bf16 outputs within one unit in the
last place (a 1-ulp flip when an fp32 value sits on a rounding boundary) or 1e-4 absolute,
whichever is larger (results that cancel to near zero carry the absolute error of their terms)."""

import numpy as np
import pytest
import torch

from conftest import TINY, golden_names, load_golden, ulp_tolerance
from oracle import gpt2_oracle as orc

FP32_TOL = 1e-4


def _close(z, ref, rel_for_big=True):
    assert z.dtype == ref.dtype and z.shape == ref.shape
    d = (z.float() - ref.float()).abs()
    if ref.dtype == torch.float32:
        # 1e-4 absolute, relaxed relatively for the reference tests' O(10..80) GEMM outputs
        tol = FP32_TOL * torch.clamp(ref.abs(), min=1.0) if rel_for_big else torch.full_like(d, FP32_TOL)
    else:
        tol = ulp_tolerance(torch.maximum(ref.float().abs(), z.float().abs()), ref.dtype, 1.0, floor=FP32_TOL)
    bad = d > tol
    assert not bad.any(), f"max|d|={d.max().item():.3e} at {int(bad.sum())} elements"


@pytest.mark.parametrize("name", golden_names("emb_"))
def test_embeddings_bit_exact(name):
    g = load_golden(name)
    z = orc.fused_embeddings(g["x"], g["wte"], g["wpe"])
    assert torch.equal(z, g["z"])


@pytest.mark.parametrize("name", golden_names("ln_"))
def test_layer_norm(name):
    g = load_golden(name)
    _close(orc.fused_layer_norm(g["x"], g["w"], g["b"]), g["z"], rel_for_big=False)


@pytest.mark.parametrize("name", golden_names("ffn_"))
def test_ffn(name):
    g = load_golden(name)
    gelu = "_g1" in name or name.endswith("_gelu")
    bias = None if "_b0" in name else g["b"]
    res = g.get("r") if not name.endswith("_gelu") else None
    _close(orc.fused_ffn(g["x"], g["w"], bias, res, gelu), g["z"])


@pytest.mark.parametrize("name", golden_names("attn_"))
def test_attention(name):
    g = load_golden(name)
    _close(orc.flash_attention_v1(g["q"], g["k"], g["v"]), g["z"], rel_for_big=False)


def test_qkv_split():
    g = load_golden("qkv_f32")
    q, k, v = orc.matmul_and_split_qkv(g["x"], g["w"], g["b"], 4)
    for a, b in ((q, g["q"]), (k, g["k"]), (v, g["v"])):
        assert a.is_contiguous()
        _close(a, b, rel_for_big=False)


def _tiny(name, dtype, affine):
    g = load_golden(name)
    cfg = orc.OracleConfig(**TINY)
    sd32 = orc.seeded_state_dict(cfg, seed=0, random_affine=affine)
    sums = np.array([float(v.double().sum()) for v in sd32.values()])
    assert np.array_equal(sums, g["weight_sums"].numpy()), "seeded weights differ from the ones the fixture was made with"
    sd = {k: v.to(dtype) for k, v in sd32.items()}
    return g, cfg, sd


@pytest.mark.parametrize("name,affine", [("tiny_f32", False), ("tiny_f32_affine", True)])
def test_tiny_model_fp32_teacher_forced(name, affine):
    """Each sub-block fed the reference's own input reproduces the reference's output to 1e-4."""
    g, cfg, sd = _tiny(name, torch.float32, affine)
    emb = orc.fused_embeddings(g["ids"], sd["wte_weight"], sd["wpe_weight"])
    assert torch.equal(emb, g["emb"])
    x = g["emb"]
    for i in range(cfg.n_layer):
        a = orc.attention_block(sd, f"blocks.{i}.0.", x, cfg.n_head)
        assert (a - g[f"attn{i}"]).abs().max() < FP32_TOL
        m = orc.mlp_block(sd, f"blocks.{i}.1.", g[f"attn{i}"])
        assert (m - g[f"mlp{i}"]).abs().max() < FP32_TOL
        x = g[f"mlp{i}"]
    hid = orc.fused_layer_norm(x, sd["layer_norm_weight"], sd["layer_norm_bias"])
    assert (hid - g["hidden"]).abs().max() < FP32_TOL
    logits = orc.lm_head(sd, g["hidden"])
    assert (logits - g["logits"]).abs().max() < FP32_TOL


@pytest.mark.parametrize("name,affine", [("tiny_f32", False), ("tiny_f32_affine", True)])
def test_tiny_model_fp32_end_to_end(name, affine):
    """Free-running: argmax identical; logits within 2e-3.  (1e-4 end to end is out of reach of
    any implementation whose fp32 summation order differs from numpy's: one-ulp differences flip
    fp16 operand roundings and the final LayerNorm amplifies them; see the teacher-forced test
    for the per-op 1e-4 bound.)"""
    g, cfg, sd = _tiny(name, torch.float32, affine)
    hid = orc.gpt_forward(sd, cfg, g["ids"])
    logits = orc.lm_head(sd, hid)
    assert (logits - g["logits"]).abs().max() < 2e-3
    assert torch.equal(logits.argmax(-1), g["logits"].argmax(-1))


def test_tiny_model_fp16_end_to_end():
    g, cfg, sd = _tiny("tiny_f16_affine", torch.float16, True)
    hid = orc.gpt_forward(sd, cfg, g["ids"])
    logits = orc.lm_head(sd, hid)
    assert (logits.float() - g["logits"].float()).abs().max() < 2e-2
    ref = g["logits"].float()
    top2 = ref.topk(2, dim=-1).values
    clear = (top2[..., 0] - top2[..., 1]) > 2e-2  # argmax must agree wherever the reference's own margin is clear
    assert torch.equal(logits.float().argmax(-1)[clear], ref.argmax(-1)[clear])


def test_accounting_known_answers():
    g = load_golden("accounting")
    cfg = orc.OracleConfig()
    assert orc.get_fwd_flops(cfg, 1024) == int(g["fwd_flops_1024"][0])
    assert orc.get_num_parameters(cfg) == int(g["num_parameters"][0])
    assert orc.estimate_days(6 * (405 * 10**9) * (15 * 10**12), mfu=0.45, gpu="h100", num_gpus=16_000) == float(g["estimate_days"][0])
    assert orc.estimate_days(6 * (405 * 10**9) * (15 * 10**12), mfu=0.45, gpu="h100", num_gpus=16_000) == 59.24544994944388  # test.py:150-152
    assert orc.compute_mfu(1e14, "a100") == float(g["mfu"][0])
    assert sorted(orc.state_dict_keys(cfg).keys()) == sorted(str(s) for s in g["state_dict_keys"])
    assert 3 * orc.get_fwd_flops(cfg, 1024) / (6 * orc.get_num_parameters(cfg) * 1024) >= 0.9995  # test.py:136-144
