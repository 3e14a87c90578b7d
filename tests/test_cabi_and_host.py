"""CPU tests: the C-ABI library builds, loads and exports every symbol the header declares (no
compute without a GPU); the module surface mirrors the reference's; accounting known answers."""

import ctypes
import os
import re

import pytest
import torch

from conftest import ROOT, TINY, load_golden

HEADER = os.path.join(ROOT, "include", "b200_gpt.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_and_exports_every_declared_symbol():
    from gpt_triton_b200 import _lib
    from gpt_triton_b200.build import build

    path = build()
    assert os.path.exists(path)
    lib = ctypes.CDLL(path)
    names = declared_functions()
    assert len(names) >= 10
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/b200_gpt.h but not exported"
    assert sorted(_lib.SIGNATURES) == names, "ctypes signature table and header disagree"
    bound = _lib.load()
    assert bound.b200_abi_version() == 6
    assert bound.b200_status_string(0) == b"ok"
    assert bound.b200_status_string(6) == b"a kernel abandoned a bounded wait"


def test_argument_checks_need_no_gpu():
    """Entry points validate sizes/dtypes before touching the device."""
    from gpt_triton_b200 import _lib

    lib = _lib.load()
    assert lib.b200_ffn_workspace_bytes(128, 256, 64, 0, _lib.F16) == 256 * 64 * 2  # [K,N] weight needs repacking
    assert lib.b200_ffn_workspace_bytes(128, 256, 64, 1, _lib.F16) == 0  # both operands usable in place
    assert lib.b200_ffn_workspace_bytes(128, 256, 64, 1, _lib.F32) == (128 + 256) * 64 * 2
    assert lib.b200_ffn_workspace_bytes(61, 31, 23, 0, _lib.F32) == (61 * 24 * 2 + 255) // 256 * 256 + (31 * 24 * 2 + 255) // 256 * 256
    assert lib.b200_layernorm(None, None, None, None, 4, 8, 1e-5, 7, 0, None) == 1  # bad dtype
    assert lib.b200_layernorm(None, None, None, None, 0, 8, 1e-5, 0, 0, None) == 0  # empty input is a no-op
    assert lib.b200_embedding(None, None, None, None, 2, 9, 10, 8, 4, 0, None, None) == 1  # L > P
    strides = (ctypes.c_int64 * 3)(1, 1, 1)
    assert lib.b200_attention(None, None, None, None, 1, 1, 4, 24, strides, strides, strides, strides, 1.0, 0, 0, None, None) == 1
    assert lib.b200_gemm(None, None, None, None, None, 4, 4, 0, 8, 8, 4, 4, 1, 1, 0, None, None) == 1  # K = 0
    assert lib.b200_ffn(None, None, None, None, None, 0, 4, 4, 4, 0, 0, 1, None, 0, None, None) == 0  # M = 0
    assert lib.b200_layernorm(ctypes.c_void_p(256), ctypes.c_void_p(256), ctypes.c_void_p(256), ctypes.c_void_p(256), 4, 8, 1e-5, 1, 2, None) == 4  # fp16 -> bf16 is not built
    # LayerNorm-aware GEMM: exactly one role per call, 16-bit data only; the fold is not offered for fp32 weights
    p256 = ctypes.c_void_p(256)
    shape = (8, 8, 8, 8, 8, 8, 8)
    assert lib.b200_gemm_ln(p256, p256, None, None, p256, *shape, 1, 1, 0, None, None, None, None, None, 1e-5, None, 0, None, None) == 1
    assert lib.b200_gemm_ln(p256, p256, None, None, p256, *shape, 1, 0, 0, None, None, None, p256, p256, 1e-5, p256, 1 << 20, None, None) == 4
    assert lib.b200_gemm_ln(p256, p256, None, None, p256, *shape, 1, 1, 0, None, None, None, p256, p256, 1e-5, None, 0, None, None) == 5  # producer needs its workspace
    assert lib.b200_gemm_ln(p256, p256, None, None, p256, *shape, 1, 1, 0, p256, None, p256, None, None, 1e-5, None, 0, None, None) == 1  # consumer needs the row extensions
    assert lib.b200_gemm_ln(p256, p256, None, None, p256, *shape, 1, 2, 0, p256, p256, p256, None, None, 1e-5, None, 0, None, None) == 4  # operand and storage type must agree
    assert lib.b200_gemm_ln_workspace_bytes(100, 768) == 12 * 128 * 8 and lib.b200_gemm_ln_workspace_bytes(100, 1600) == 25 * 128 * 8  # 64-column slices
    assert lib.b200_fold_layernorm(p256, p256, p256, None, p256, p256, p256, p256, 8, 8, 8, 0, None) == 4
    assert lib.b200_fold_layernorm(p256, p256, p256, None, p256, p256, p256, p256, 8, 8, 4, 1, None) == 1  # ld_packed < K
    assert lib.b200_row_ln_stats(None, None, None, 0, 8, 1e-5, 1, None) == 0 and lib.b200_row_ln_stats(None, None, None, 4, 8, 1e-5, 1, None) == 1
    # sizes beyond what the GEMM indexes are refused before any arithmetic on them
    assert lib.b200_ffn(p256, p256, None, None, p256, 1 << 40, 8, 8, 8, 0, 0, 1, None, 0, None, None) == 1
    assert lib.b200_ffn_static_scratch(p256, p256, None, None, p256, 1 << 40, 8, 1 << 40, 8, 0, 0, 0, None, None) == 1
    assert lib.b200_selftest_bounded_wait(None, 1000, None) == 1  # needs a status word
    assert lib.b200_selftest_bounded_wait(ctypes.c_void_p(256), 0, None) == 1  # and a positive cycle limit
    # row statistics without the product: argmax_out is mandatory, targets and target_logit_out come together,
    # the rounding type is 16-bit, and the workspace is checked before any launch
    assert lib.b200_gemm_argmax_workspace_bytes(100, 1000) == 8 * 128 * 12  # 4 tiles of 256 columns x 2 slices, rows padded to 64
    one = ctypes.c_void_p(256)
    assert lib.b200_gemm_rowstats(one, one, None, 4, 4, 8, 8, 8, 1, 1, None, None, None, None, None, 0, None, None) == 1
    assert lib.b200_gemm_rowstats(one, one, None, 4, 4, 8, 8, 8, 1, 1, one, one, None, None, None, 0, None, None) == 1
    assert lib.b200_gemm_rowstats(one, one, None, 4, 4, 8, 8, 8, 1, 0, None, one, None, None, None, 0, None, None) == 4  # fp32 rounding: unsupported
    assert lib.b200_gemm_rowstats(one, one, None, 4, 4, 8, 8, 8, 1, 1, None, one, None, None, None, 0, None, None) == 5  # no workspace
    assert lib.b200_gemm_rowstats(one, one, None, 0, 4, 8, 8, 8, 1, 1, None, one, None, None, None, 0, None, None) == 0  # M = 0
    # token-by-token generation: the position lives in device memory and is mandatory; sizes are checked first
    assert lib.b200_embedding_at(one, one, one, one, 2, 1, 10, 8, 4, 1, None, 1e-5, None, None, None, None) == 1  # no position
    assert lib.b200_embedding_at(one, one, one, one, 2, 9, 10, 8, 4, 1, None, 1e-5, None, None, one, None) == 1  # L > P
    assert lib.b200_embedding_at(one, one, one, one, 0, 1, 10, 8, 4, 1, None, 1e-5, None, None, one, None) == 0  # empty batch
    assert lib.b200_kv_cache_fill(one, one, 2, 9, 64, 8, 1, None) == 1  # more positions than the cache holds
    assert lib.b200_kv_cache_fill(one, one, 0, 9, 64, 16, 1, None) == 0
    assert lib.b200_attention_decode(one, one, one, 2, 4, 48, 16, 1.0, 1, one, None, None) == 4  # head size not built
    assert lib.b200_attention_decode(one, one, one, 2, 4, 64, 16, 1.0, 1, None, None, None) == 1  # no position
    assert lib.b200_attention_decode(one, one, one, 0, 4, 64, 16, 1.0, 1, one, None, None) == 0
    assert lib.b200_decode_append(one, one, 4, 8, 2, one, 1, None, None, None) == 1  # row pitch below the column count
    assert lib.b200_decode_append(one, one, 8, 8, 2, None, 1, None, None, None) == 1
    assert lib.b200_sample_logits(one, 16, 2, 16, 1, 0.0, 0, 0, None, one, None) == 1  # temperature must be positive
    assert lib.b200_sample_logits(one, 8, 2, 16, 1, 1.0, 0, 0, None, one, None) == 1  # row pitch below the vocabulary
    assert lib.b200_sample_logits(one, 16, 0, 16, 1, 1.0, 0, 0, None, one, None) == 0


def test_operators_refuse_cpu_tensors():
    from gpt_triton_b200 import kernels as K

    with pytest.raises(RuntimeError, match="CUDA"):
        K.fused_layer_norm(torch.rand(2, 8), torch.ones(8), torch.zeros(8))
    with pytest.raises(RuntimeError, match="CUDA"):
        K.fused_embeddings(torch.zeros((1, 2), dtype=torch.long), torch.rand(4, 8), torch.rand(4, 8))
    with pytest.raises(RuntimeError, match="CUDA"):
        K.flash_attention_v1(*(torch.rand(1, 1, 4, 16) for _ in range(3)))


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from gpt_triton_b200 import _lib

    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "libb200gpt.so"))
    with pytest.raises(ImportError, match="no CPU or PyTorch fallback"):
        _lib.load()


def test_module_surface_and_state_dict_layout():
    from gpt_triton_b200.gpt import FusedGPT, GPTConfig, get_num_parameters

    g = load_golden("accounting")
    assert GPTConfig() == GPTConfig(vocab_size=50304, block_size=512, n_layer=12, n_head=12, n_embd=768, dropout=0.1)
    model = FusedGPT(GPTConfig()).eval()
    assert list(model.state_dict().keys()) == [str(s) for s in g["state_dict_keys"]]
    assert get_num_parameters(model) == int(g["num_parameters"][0])
    assert model.get_fwd_flops(1024) == int(g["fwd_flops_1024"][0])
    r = (model.get_fwd_flops(1024) * 3) / (6 * get_num_parameters(model) * 1024)
    assert r >= 0.9995  # the reference's test_flops (test.py:136-144)
    blk = model.blocks[0]
    assert blk[0].c_attn_weight.shape == (768, 2304) and blk[1].ffn2_weight.shape == (3072, 768)


def test_accounting_known_answers():
    from gpt_triton_b200.gpt import GPU_TO_FLOPS, GPTConfig, compute_mfu, estimate_days, executed_fwd_flops

    g = load_golden("accounting")
    t = estimate_days(6 * (405 * 10**9) * (15 * 10**12), mfu=0.45, gpu="h100", num_gpus=16_000)
    assert t == 59.24544994944388 == float(g["estimate_days"][0])  # the reference's test_estimate_days (test.py:147-152)
    assert compute_mfu(1e14, "a100") == float(g["mfu"][0])
    assert GPU_TO_FLOPS["b200"] == 2250 * 10**12
    with pytest.raises(AssertionError):
        compute_mfu(1.0, "tpu")
    cfg = GPTConfig(vocab_size=50257, block_size=1024)
    assert abs(executed_fwd_flops(cfg, 512, 300) / 3.8801e13 - 1) < 1e-3
    assert abs(executed_fwd_flops(cfg, 512, 300, with_lm_head=False) / 2.6944e13 - 1) < 1e-3


def test_huggingface_state_dict_conversion():
    """A GPT2Model built from a config (no download) converts key for key and loads."""
    from transformers import GPT2Config, GPT2Model

    from gpt_triton_b200.gpt import FusedGPT, convert_huggingface_to_triton

    hf_cfg = GPT2Config(vocab_size=1024, n_positions=128, n_embd=128, n_layer=2, n_head=4)
    hf = GPT2Model(hf_cfg)
    sd, cfg = convert_huggingface_to_triton(hf.state_dict(), hf_cfg)
    assert (cfg.vocab_size, cfg.block_size, cfg.n_layer, cfg.n_head, cfg.n_embd) == (1024, 128, 2, 4, 128)
    model = FusedGPT(cfg)
    missing, unexpected = model.load_state_dict(sd)
    assert not missing and not unexpected
    assert torch.equal(model.blocks[1][1].ffn1_weight, hf.h[1].mlp.c_fc.weight)
    assert torch.equal(model.blocks[0][0].c_attn_bias, hf.h[0].attn.c_attn.bias)
    hf_cfg.n_ctx = 64
    assert convert_huggingface_to_triton(hf.state_dict(), hf_cfg)[1].block_size == 64


def test_convert_hf_and_load_model_reads_a_checkpoint_directory(tmp_path):
    """convert_hf_and_load_model (gpt.py:240-247 of the reference) with a save_pretrained directory in place of
    the hub id: returns (FusedGPT, GPT2Model), both in eval mode, parameters equal tensor for tensor."""
    from transformers import GPT2Config, GPT2Model

    from gpt_triton_b200.gpt import convert_hf_and_load_model

    GPT2Model(GPT2Config(vocab_size=512, n_positions=64, n_embd=64, n_layer=2, n_head=2)).save_pretrained(str(tmp_path))
    model, hf = convert_hf_and_load_model(str(tmp_path), "cpu")
    assert not model.training and not hf.training
    assert (model.config.vocab_size, model.config.block_size, model.config.n_layer) == (512, 64, 2)
    assert torch.equal(model.wte_weight, hf.wte.weight) and torch.equal(model.layer_norm_bias, hf.ln_f.bias)
    assert torch.equal(model.blocks[1][0].c_proj_weight, hf.h[1].attn.c_proj.weight)
