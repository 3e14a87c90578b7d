"""CPU oracle for the GPT-2 forward path (TEST INFRASTRUCTURE, not product code).

This file restates, in plain PyTorch-on-CPU arithmetic, what the reference's
Triton kernels compute, with the reference's rounding points kept:

* ``fused_embeddings``   follows kernels.py:37-101
* ``fused_layer_norm``   follows kernels.py:104-164
* ``gelu_new``/``tanh``  follow  kernels.py:15-26
* ``fused_ffn``          follows kernels.py:169-315
* ``matmul_and_split_qkv`` follows kernels.py:347-367
* ``flash_attention_v1`` follows kernels.py:375-525
* ``gpt_forward``/``lm_head`` follow gpt.py:38-60, 90-111, 163-180 and the
  commented-out tied lm_head at gpt.py:159-161, 172-179
* ``get_fwd_flops``/``estimate_days``/``compute_mfu`` follow gpt.py:62-67,
  113-119, 182-196, 250-263

Parity is PINNED: ``tests/golden/make_golden.py`` runs the unmodified
reference under ``TRITON_INTERPRET=1`` and stores its outputs; the CPU test
suite checks every function here against those vectors.  The exception is the
"generation" section (``generate_by_recompute``, ``sample_logits``): the
reference has no inference loop, so those are "parity unpinned" -- defined on
top of the pinned forward, see the comment there.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of
``bench.py`` may import this module.  The product package never does.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch

KEY_BLOCK = 64  # kernels.py:509 -- BLOCK_SIZE_L of the reference attention kernel


def _f16_operand(t: torch.Tensor) -> torch.Tensor:
    """Round to fp16 (the reference casts every tl.dot operand, kernels.py:229, 234,
    414, 428, 465-466) and widen to fp32 so the product/accumulate is fp32."""
    return t.to(torch.float16).to(torch.float32)


# --------------------------------------------------------------------------- embeddings
@torch.no_grad()
def fused_embeddings(x, wte, wpe):
    """z[b,l,:] = wte[x[b,l],:] + wpe[l,:]   (kernels.py:59-72; position is pid % L).

    The add happens in the storage dtype (both loads have wte's dtype), so a
    same-dtype add reproduces it bit for bit.
    """
    assert wte.shape[1] == wpe.shape[1]
    B, L = x.shape
    assert L <= wpe.shape[0], "sequence longer than the position table"
    pos = torch.arange(L)
    if wte.dtype in (torch.float16, torch.bfloat16):
        # one rounding of the exact sum == the native half add
        z = (wte[x].float() + wpe[pos][None].float()).to(wte.dtype)
    else:
        z = wte[x] + wpe[pos][None]
    return z


# --------------------------------------------------------------------------- layer norm
@torch.no_grad()
def fused_layer_norm(x, weight, bias, eps: float = 1e-5):
    """Row LayerNorm with fp32 statistics, two-pass variance (kernels.py:116-145)."""
    assert weight.shape == bias.shape and x.shape[-1] == weight.shape[0]
    H = x.shape[-1]
    xf = x.reshape(-1, H).float()
    mean = xf.sum(dim=1, keepdim=True) / H
    d = xf - mean
    var = (d * d).sum(dim=1, keepdim=True) / H
    rstd = 1.0 / torch.sqrt(var + eps)
    z = d * rstd
    z = z * weight.float() + bias.float()
    return z.to(x.dtype).reshape(x.shape)


# --------------------------------------------------------------------------- GEMM
def _tanh_via_sigmoid(x):
    return 2 * torch.sigmoid(2 * x) - 1  # kernels.py:17-18


def gelu_new(x):
    a = math.sqrt(2.0 / math.pi)  # kernels.py:23-26
    b = x + 0.044715 * x * x * x
    return 0.5 * x * (1.0 + _tanh_via_sigmoid(a * b))


@torch.no_grad()
def fused_ffn(x, weight, bias=None, residual=None, add_gelu=False):
    """z = [gelu](x16 @ w16 + b) + r ; fp32 accumulate; order bias -> gelu -> residual
    (kernels.py:224-257); result cast to x.dtype (kernels.py:281)."""
    out_shape_0 = x.shape[:-1]
    K = x.shape[-1]
    assert weight.shape[0] == K
    N = weight.shape[1]
    z = _f16_operand(x.reshape(-1, K)) @ _f16_operand(weight)
    if bias is not None:
        z = z + bias.float()
    if add_gelu:
        z = gelu_new(z)
    if residual is not None:
        z = z + residual.reshape(-1, N).float()
    return z.to(x.dtype).reshape(*out_shape_0, N)


@torch.no_grad()
def matmul_and_split_qkv(x, weight, bias, num_heads):
    """kernels.py:348-367: GEMM, split in three, each to [B, nh, L, d] contiguous."""
    y = fused_ffn(x, weight, bias=bias)
    B, L, H3 = y.shape
    assert H3 % 3 == 0
    h = H3 // 3
    assert h % num_heads == 0
    d = h // num_heads
    q, k, v = y.split(h, dim=2)
    return tuple(t.reshape(B, L, num_heads, d).transpose(1, 2).contiguous() for t in (q, k, v))


# --------------------------------------------------------------------------- attention
@torch.no_grad()
def flash_attention_v1(q, k, v, key_block: int = KEY_BLOCK):
    """Causal attention with the reference's online softmax over 64-key blocks
    (kernels.py:417-474): P = exp(s - running_max) is rounded to fp16 per block
    before the PV product, the running max/denominator are fp32."""
    assert q.shape[:2] == k.shape[:2] and q.shape[-1] == k.shape[-1] and k.shape == v.shape
    B, N, Lq, H = q.shape
    Lk = k.shape[2]
    scale = 1 / math.sqrt(H)  # kernels.py:507
    qf = _f16_operand(q.reshape(B * N, Lq, H))
    kf = _f16_operand(k.reshape(B * N, Lk, H))
    vf = _f16_operand(v.reshape(B * N, Lk, H))
    z = torch.zeros((B * N, Lq, H), dtype=torch.float32)
    m = torch.full((B * N, Lq, 1), float("-inf"), dtype=torch.float32)
    l = torch.zeros((B * N, Lq, 1), dtype=torch.float32)
    iq = torch.arange(Lq)[:, None]
    for s in range(0, Lk, key_block):
        e = min(s + key_block, Lk)
        ik = torch.arange(s, e)[None, :]
        qk = torch.bmm(qf, kf[:, s:e].transpose(1, 2)) * scale  # kernels.py:429
        qk = torch.where(iq >= ik, qk, torch.tensor(float("-inf")))  # kernels.py:438
        bm = qk.max(dim=2, keepdim=True).values
        new_m = torch.where(bm > m, bm, m)  # kernels.py:442-444
        p = torch.exp(qk - new_m)
        mult = torch.exp(m - new_m)
        # rows whose running max is still -inf would give nan here; with Lq == Lk and a
        # causal mask the first block always holds key 0, so this never happens.
        l = l * mult + p.sum(dim=2, keepdim=True)
        z = z * mult
        m = new_m
        z = z + torch.bmm(_f16_operand(p), vf[:, s:e])  # kernels.py:465-468
    z = z / l  # kernels.py:471
    return z.to(q.dtype).reshape(B, N, Lq, H)


# --------------------------------------------------------------------------- model
@dataclass
class OracleConfig:
    """Field names follow gpt.py:122-129."""

    vocab_size: int = 50304
    block_size: int = 512
    n_layer: int = 12
    n_head: int = 12
    n_embd: int = 768
    dropout: float = 0.1


def state_dict_keys(cfg):
    """The reference's state-dict layout (gpt.py:29-36, 76-85, 137-157): name -> shape."""
    h = cfg.n_embd
    keys = {"wte_weight": (cfg.vocab_size, h), "wpe_weight": (cfg.block_size, h)}
    for i in range(cfg.n_layer):
        a, m = f"blocks.{i}.0.", f"blocks.{i}.1."
        keys[a + "layer_norm_weight"] = (h,)
        keys[a + "layer_norm_bias"] = (h,)
        keys[a + "c_attn_weight"] = (h, 3 * h)
        keys[a + "c_attn_bias"] = (3 * h,)
        keys[a + "c_proj_weight"] = (h, h)
        keys[a + "c_proj_bias"] = (h,)
        keys[m + "layer_norm_weight"] = (h,)
        keys[m + "layer_norm_bias"] = (h,)
        keys[m + "ffn1_weight"] = (h, 4 * h)
        keys[m + "ffn1_bias"] = (4 * h,)
        keys[m + "ffn2_weight"] = (4 * h, h)
        keys[m + "ffn2_bias"] = (h,)
    keys["layer_norm_weight"] = (h,)
    keys["layer_norm_bias"] = (h,)
    return keys


def seeded_state_dict(cfg, seed=0, dtype=torch.float32, scale_residual_proj=False, random_affine=False):
    """Random-init weights of the benchmark configs: matrices/embeddings N(0, 0.02) from a
    CPU generator, biases 0, LayerNorm gamma 1 / beta 0; optionally the two output
    projections scaled by 1/sqrt(2*n_layer).  ``random_affine`` instead draws non-trivial
    biases and LayerNorm parameters so that tests exercise those code paths."""
    g = torch.Generator().manual_seed(seed)
    sd = {}
    for name, shape in state_dict_keys(cfg).items():
        if len(shape) == 2:
            w = torch.randn(shape, generator=g) * 0.02
            if scale_residual_proj and (name.endswith("c_proj_weight") or name.endswith("ffn2_weight")):
                w = w / math.sqrt(2 * cfg.n_layer)
        elif name.endswith("layer_norm_weight"):
            w = torch.ones(shape)
            if random_affine:
                w = w + 0.1 * torch.randn(shape, generator=g)
        else:
            w = torch.zeros(shape)
            if random_affine:
                w = 0.05 * torch.randn(shape, generator=g)
        sd[name] = w.to(dtype)
    return sd


@torch.no_grad()
def attention_block(sd, prefix, x, n_head):
    """gpt.py:38-60."""
    residual = x
    x = fused_layer_norm(x, sd[prefix + "layer_norm_weight"], sd[prefix + "layer_norm_bias"])
    q, k, v = matmul_and_split_qkv(x, sd[prefix + "c_attn_weight"], sd[prefix + "c_attn_bias"], n_head)
    x = flash_attention_v1(q, k, v)
    x = x.transpose(1, 2).contiguous().view(residual.shape)
    return fused_ffn(x, sd[prefix + "c_proj_weight"], bias=sd[prefix + "c_proj_bias"], residual=residual)


@torch.no_grad()
def mlp_block(sd, prefix, x):
    """gpt.py:90-111."""
    residual = x
    x = fused_layer_norm(x, sd[prefix + "layer_norm_weight"], sd[prefix + "layer_norm_bias"])
    x = fused_ffn(x, sd[prefix + "ffn1_weight"], bias=sd[prefix + "ffn1_bias"], add_gelu=True)
    return fused_ffn(x, sd[prefix + "ffn2_weight"], bias=sd[prefix + "ffn2_bias"], residual=residual)


@torch.no_grad()
def gpt_forward(sd, cfg, ids, return_intermediates=False):
    """gpt.py:163-180: embeddings -> blocks -> final LayerNorm; returns the hidden state."""
    inter = {}
    x = fused_embeddings(ids, sd["wte_weight"], sd["wpe_weight"])
    inter["emb"] = x
    for i in range(cfg.n_layer):
        x = attention_block(sd, f"blocks.{i}.0.", x, cfg.n_head)
        inter[f"attn{i}"] = x
        x = mlp_block(sd, f"blocks.{i}.1.", x)
        inter[f"mlp{i}"] = x
    x = fused_layer_norm(x, sd["layer_norm_weight"], sd["layer_norm_bias"])
    return (x, inter) if return_intermediates else x


@torch.no_grad()
def lm_head(sd, hidden):
    """The tied head the reference leaves commented out (gpt.py:159-161, 172-179):
    fused_ffn(hidden, wte.T.contiguous(), bias=None)."""
    return fused_ffn(hidden, sd["wte_weight"].T.contiguous())


# --------------------------------------------------------------------------- generation (parity unpinned)
# The reference never built an inference loop (README.md:55 lists "KV cache + sampling" as to do), so nothing below
# is pinned by reference outputs.  The definition used instead: generating a token means running the reference's
# whole forward (restated above, pinned) over the sequence so far and picking from the last position's logits; a
# key/value cache must not change the result beyond rounding.
@torch.no_grad()
def generate_by_recompute(sd, cfg, ids, max_new_tokens, pick=None):
    """ids (batch, prompt_len) -> (tokens (batch, max_new_tokens), last-position logits of every step): every step
    re-runs gpt_forward + lm_head over the whole sequence; `pick(logits (batch, vocab), position)` chooses the next
    ids (default: argmax, lowest index on ties)."""
    seq = ids.clone()
    tokens, step_logits = [], []
    for _ in range(max_new_tokens):
        logits = lm_head(sd, gpt_forward(sd, cfg, seq)[:, -1:, :])[:, 0, :]
        nxt = logits.float().argmax(dim=-1) if pick is None else pick(logits, seq.shape[1])
        step_logits.append(logits)
        tokens.append(nxt)
        seq = torch.cat([seq, nxt[:, None]], dim=1)
    return torch.stack(tokens, dim=1), step_logits


_M64 = (1 << 64) - 1


def _mix64(z: int) -> int:
    """Finaliser of SplitMix64 (Steele, Lea, Flood 2014) on Python integers, modulo 2^64."""
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    return z ^ (z >> 31)


def sampling_uniform(seed: int, step: int, row: int, col: int) -> float:
    """u in (0, 1) of the library's counter-based generator: 23 bits of mix64(mix64(seed + golden * (step + 1)) ^ (row, col))."""
    key = _mix64((seed + 0x9E3779B97F4A7C15 * ((step & 0xFFFFFFFF) + 1)) & _M64)
    x = _mix64(key ^ ((row << 32) | col))
    return ((x >> 41) + 0.5) / 8388608.0


def sample_logits(logits, temperature, top_k, seed, step):
    """Top-k filter + Gumbel-max draw, in float64: returns (ids (rows,), scores (rows, vocab) with -inf where filtered
    out), scores[r, j] = logits[r, j] / temperature - log(-log(u(seed, step, r, j))).  Columns tied with the k-th
    largest logit all stay in; the id is the lowest index of the maximum score."""
    import numpy as np

    x = logits.to(torch.float64).numpy()
    rows, vocab = x.shape
    scores = np.full((rows, vocab), -np.inf)
    for r in range(rows):
        keep = np.ones(vocab, dtype=bool)
        if 0 < top_k < vocab:
            kth = np.sort(x[r])[vocab - top_k]
            keep = x[r] >= kth
        u = np.array([sampling_uniform(seed, step, r, j) for j in range(vocab)])
        sc = x[r] / temperature - np.log(-np.log(u))
        scores[r, keep] = sc[keep]
    return torch.from_numpy(scores.argmax(axis=1)), torch.from_numpy(scores)


# --------------------------------------------------------------------------- accounting
GPU_TO_FLOPS = {"v100": 130 * 10**12, "a100": 312 * 10**12, "h100": 989 * 10**12}  # gpt.py:14-18


def get_fwd_flops(cfg, num_tokens):
    """gpt.py:62-67, 113-119, 182-196."""
    h, v, p, mid = cfg.n_embd, cfg.vocab_size, cfg.block_size, 4 * cfg.n_embd
    ln = 2 * num_tokens * h
    attn = ln + num_tokens * (3 * h) * (2 * h) + num_tokens * (3 * h) + num_tokens * h * (2 * h) + num_tokens * h
    mlp = ln + num_tokens * mid * (2 * h) + num_tokens * mid + num_tokens * h * (2 * mid) + num_tokens * h
    return cfg.n_layer * (attn + mlp) + ln + num_tokens * h * (2 * v) + num_tokens * h * (2 * p)


def get_num_parameters(cfg):
    return sum(math.prod(s) for s in state_dict_keys(cfg).values())


def estimate_days(flops, mfu=0.45, gpu="h100", num_gpus=1):
    assert gpu in GPU_TO_FLOPS  # gpt.py:250-254
    return flops / (mfu * GPU_TO_FLOPS[gpu] * 3600 * 24 * num_gpus)


def compute_mfu(flops_per_second, gpu="h100"):
    assert gpu in GPU_TO_FLOPS  # gpt.py:261-263
    return flops_per_second / GPU_TO_FLOPS[gpu]
