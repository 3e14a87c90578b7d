"""GPU tests of token-by-token generation (key/value cache, one-query attention, sampling, FusedGPT.generate).

The reference has no inference loop (its README.md:55 lists "KV cache + sampling" as not built), so the checks are:
the one-query attention against the last row of the oracle's flash_attention_v1 (pinned); the cached generation
against re-running the whole sequence (teacher-forced: every generated token must be an argmax of the full forward's
logits at its position, to rounding) and against the CPU oracle's recompute loop on the tiny configuration; the
sampler against its float64 restatement and against the softmax probabilities it is meant to draw from."""

import math

import pytest
import torch

from conftest import TINY
from oracle import gpt2_oracle as orc
from test_gpu_model import build_model

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL = {torch.float32: 1e-4, torch.float16: 2e-3, torch.bfloat16: 1.6e-2}


def _status():
    from gpt_triton_b200 import kernels as K

    return K.device_status()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("D,L,B,NH", [(64, 1, 3, 5), (64, 2, 3, 5), (64, 64, 3, 5), (64, 65, 3, 5), (64, 300, 3, 5), (32, 129, 3, 5), (128, 70, 3, 5),
                                      # enough (batch, head) pairs for one warp each (the large-batch variant of the kernel)
                                      (64, 70, 200, 12), (32, 33, 100, 25), (64, 193, 100, 25)])
def test_attention_decode_matches_last_row_of_full_attention(dtype, D, L, B, NH):
    from gpt_triton_b200 import kernels as K

    cap = L + 3
    H = NH * D
    g = torch.Generator().manual_seed(L * 7 + D)
    q, k, v = (torch.randn((B, NH, L, D), generator=g).to(dtype) for _ in range(3))
    ref = orc.flash_attention_v1(q, k, v)[:, :, -1, :].reshape(B, H).float()
    merged = lambda t: t.transpose(1, 2).reshape(B, L, H)  # (B, L, NH*D)
    cache = torch.full((B, cap, 2 * H), float("nan"), dtype=dtype)
    cache[:, :L - 1, :H] = merged(k)[:, :L - 1]
    cache[:, :L - 1, H:] = merged(v)[:, :L - 1]
    qkv_new = torch.cat([merged(q)[:, -1], merged(k)[:, -1], merged(v)[:, -1]], dim=1).contiguous()
    cache_d = cache.to(DEV)
    pos = torch.tensor([L - 1, 0], dtype=torch.int32, device=DEV)
    out = K.attention_decode(qkv_new.to(DEV), cache_d, pos, NH).cpu().float()
    assert _status() == 0
    # (over the 10^5 outputs of the large cases one fp16 rounding of P flips on a last-bit difference of an fp32 score: the
    # bound on arbitrary inputs is about 5e-4 for any implementation, as for the full attention kernel)
    assert (out - ref).abs().max().item() < (TOL[dtype] if B * NH < 100 else max(TOL[dtype], 5e-4))
    # the new token's keys and values joined the cache, nothing else was written
    got = cache_d.cpu()
    assert torch.equal(got[:, L - 1], qkv_new[:, H:])
    assert torch.equal(got[:, :L - 1], cache[:, :L - 1]) and torch.isnan(got[:, L:].float()).all()


def test_attention_decode_refuses_a_full_cache():
    """A position outside the cache is reported through the status word (code 41); nothing is read or written."""
    from gpt_triton_b200 import kernels as K

    B, NH, D, cap = 2, 4, 64, 8
    cache = torch.zeros((B, cap, 2 * NH * D), dtype=torch.float16, device=DEV)
    qkv = torch.ones((B, 3 * NH * D), dtype=torch.float16, device=DEV)
    assert _status() == 0
    K.attention_decode(qkv, cache, torch.tensor([cap, 0], dtype=torch.int32, device=DEV), NH)
    assert _status() == 41
    assert cache.abs().sum().item() == 0
    K.attention_decode(qkv, cache, torch.tensor([cap - 1, 0], dtype=torch.int32, device=DEV), NH)
    assert _status() == 0 and cache[:, cap - 1].eq(1).all()


def test_decode_append_columns_feedback_and_overflow():
    """tokens[:, pos[0] - pos[1] + advance] = ids, the same ids into the feedback buffer, pos[0] += 1 when advancing; a
    column outside the token buffer writes nothing and is reported through the status word (code 42)."""
    from gpt_triton_b200 import kernels as K

    B = 700  # more rows than the single block has threads
    tokens = torch.full((B, 3), -1, dtype=torch.int64, device=DEV)
    feedback = torch.full((B,), -1, dtype=torch.int64, device=DEV)
    pos = torch.tensor([9, 9], dtype=torch.int32, device=DEV)
    ids = [torch.arange(B, device=DEV) * 10 + k for k in range(4)]
    K.decode_append(ids[0], tokens, pos, advance=False, feedback=feedback)  # the prompt's prediction: column 0, position stays
    assert pos.tolist() == [9, 9] and torch.equal(tokens[:, 0], ids[0]) and torch.equal(feedback, ids[0]) and (tokens[:, 1:] == -1).all()
    K.decode_append(ids[1], tokens, pos, advance=True, feedback=feedback)
    K.decode_append(ids[2], tokens, pos, advance=True)
    assert pos.tolist() == [11, 9] and torch.equal(tokens[:, 1], ids[1]) and torch.equal(tokens[:, 2], ids[2]) and torch.equal(feedback, ids[1])
    assert _status() == 0
    before = tokens.clone()
    K.decode_append(ids[3], tokens, pos, advance=True, feedback=feedback)  # column 3 does not exist
    assert _status() == 42
    assert pos.tolist() == [11, 9] and torch.equal(tokens, before) and torch.equal(feedback, ids[1])


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_kv_cache_fill_copies_keys_and_values(dtype):
    from gpt_triton_b200 import kernels as K

    B, L, H, cap = 3, 37, 96, 50
    qkv = torch.randn((B, L, 3 * H), generator=torch.Generator().manual_seed(1)).to(dtype)
    cache = torch.zeros((B, cap, 2 * H), dtype=dtype, device=DEV)
    K.kv_cache_fill(qkv.to(DEV), cache)
    got = cache.cpu()
    assert torch.equal(got[:, :L], qkv[:, :, H:]) and got[:, L:].abs().sum().item() == 0


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_embedding_at_a_device_side_position(dtype):
    from gpt_triton_b200 import kernels as K

    V, P, H, B = 100, 40, 64, 5
    g = torch.Generator().manual_seed(3)
    wte, wpe = torch.randn((V, H), generator=g).to(dtype), torch.randn((P, H), generator=g).to(dtype)
    ids = torch.randint(0, V, (B, 1), generator=g)
    for p in (0, 17, P - 1):
        pos = torch.tensor([p, 0], dtype=torch.int32, device=DEV)
        z, stats = K.fused_embeddings(ids.to(DEV), wte.to(DEV), wpe.to(DEV), return_row_stats=True, position=pos)
        ref = wte[ids[:, 0]] + wpe[p]  # same-dtype add, as kernels.py:68-69 of the reference
        assert torch.equal(z.cpu()[:, 0], ref)
        mean = ref.float().mean(dim=1)
        assert (stats.mean.cpu() - mean).abs().max().item() < 1e-5
    # two positions starting at p: rows p and p + 1
    ids2 = torch.randint(0, V, (B, 2), generator=g)
    z = K.fused_embeddings(ids2.to(DEV), wte.to(DEV), wpe.to(DEV), position=torch.tensor([7], dtype=torch.int32, device=DEV))
    assert torch.equal(z.cpu(), wte[ids2] + wpe[7:9][None])


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("top_k", [0, 1, 5, 200])
def test_sample_logits_matches_the_float64_restatement(dtype, top_k):
    """Same generator, same filter, same Gumbel-max: the ids agree wherever the restatement's best two scores are not
    within float32 rounding of each other."""
    from gpt_triton_b200 import kernels as K

    rows, V, temperature, seed, step = 6, 1000, 0.7, 12345, 9
    logits = (torch.randn((rows, V), generator=torch.Generator().manual_seed(top_k)) * 3).to(dtype)
    logits[0, 10:14] = logits[0].max()  # ties at the top: all of them stay in for top_k = 1
    ids_ref, scores = orc.sample_logits(logits, temperature, top_k, seed, step)
    ids = K.sample_logits(logits.to(DEV), temperature=temperature, top_k=top_k, seed=seed,
                          step=torch.tensor([step], dtype=torch.int32, device=DEV)).cpu()
    top2 = scores.topk(2, dim=1).values
    for r in range(rows):
        assert scores[r, ids[r]] > -math.inf, "a filtered-out column was drawn"
        assert ids[r] == ids_ref[r] or (top2[r, 0] - scores[r, ids[r]]).item() < 1e-4
    if top_k == 1:  # only the row maximum (and what ties with it) can be drawn
        assert 10 <= ids[0].item() < 14
        assert torch.equal(logits.float().gather(1, ids[:, None])[:, 0], logits.float().max(dim=1).values)
    # a step or seed change moves the draws; the same pair repeats them
    again = K.sample_logits(logits.to(DEV), temperature=temperature, top_k=top_k, seed=seed,
                            step=torch.tensor([step], dtype=torch.int32, device=DEV)).cpu()
    assert torch.equal(again, ids)


def test_sample_logits_full_vocabulary_row():
    from gpt_triton_b200 import kernels as K

    V = 50257
    logits = (torch.randn((2, V), generator=torch.Generator().manual_seed(8)) * 2).half()
    ids_ref, scores = orc.sample_logits(logits, 1.0, 40, 3, 0)
    pitch = (V + 63) // 64 * 64
    buf = torch.zeros((2, pitch), dtype=torch.float16, device=DEV)
    buf[:, :V] = logits.to(DEV)
    ids = K.sample_logits(buf[:, :V], temperature=1.0, top_k=40, seed=3).cpu()
    assert (scores > -math.inf).sum(dim=1).min().item() >= 40  # (more than 40 only through ties at the threshold)
    for r in range(2):
        assert ids[r] == ids_ref[r] or (scores[r].max() - scores[r, ids[r]]).item() < 1e-4


def test_sample_logits_draws_from_the_softmax():
    """20000 rows with the same 8 logits: the frequencies of the drawn ids follow softmax(logits / temperature)
    (top_k = 5 removes the three smallest) within 4.5 standard deviations."""
    from gpt_triton_b200 import kernels as K

    n, temperature = 20000, 1.3
    row = torch.tensor([1.0, -0.5, 2.0, 0.3, -3.0, 0.9, 1.7, -1.2])
    logits = row.repeat(n, 1).to(DEV)
    for top_k in (0, 5):
        ids = K.sample_logits(logits, temperature=temperature, top_k=top_k, seed=77).cpu()
        x = row.double() / temperature
        if top_k:
            x[row < row.sort().values[-top_k]] = -math.inf
        p = torch.softmax(x, dim=0)
        freq = torch.bincount(ids, minlength=8).double() / n
        sigma = (p * (1 - p) / n).sqrt()
        assert ((freq - p).abs() <= 4.5 * sigma + 1e-12).all(), (freq, p)


def _teacher_forced_check(model, prompt, tokens, tol):
    """Every generated token must be an argmax, to `tol`, of the logits the full forward over prompt + tokens gives at
    the position before it."""
    L0 = prompt.shape[1]
    seq = torch.cat([prompt, tokens[:, :-1]], dim=1)
    logits = model.logits(seq).float()[:, L0 - 1:, :]  # (B, new, V): position L0-1+s predicts token s
    best = logits.max(dim=-1).values
    chosen = logits.gather(-1, tokens.unsqueeze(-1)).squeeze(-1)
    gap = (best - chosen).max().item()
    assert gap <= tol, f"a generated token trails the recomputed argmax by {gap}"
    return (logits.argmax(dim=-1) == tokens).float().mean().item()


@pytest.mark.parametrize("name,cfg,dtype,tol,B,L0,new", [
    ("tiny_f32", TINY, torch.float32, 2e-3, 3, 20, 24),
    ("small_width_f16", dict(vocab_size=2048, block_size=256, n_layer=2, n_head=12, n_embd=768), torch.float16, 2e-2, 4, 70, 40),
    ("small_width_bf16", dict(vocab_size=2048, block_size=256, n_layer=2, n_head=12, n_embd=768), torch.bfloat16, 1.3e-1, 4, 65, 30),
    ("prompt_of_one_f16", dict(vocab_size=512, block_size=128, n_layer=2, n_head=4, n_embd=256), torch.float16, 2e-2, 2, 1, 100),
])
def test_greedy_generation_matches_recomputation(name, cfg, dtype, tol, B, L0, new):
    model, _, _ = build_model(cfg, dtype, random_affine=True)
    prompt = torch.randint(0, cfg["vocab_size"], (B, L0), generator=torch.Generator().manual_seed(4)).to(DEV)
    tokens = model.generate(prompt, new)
    assert tokens.shape == (B, new) and tokens.dtype == torch.int64
    agree = _teacher_forced_check(model, prompt, tokens, tol)
    assert agree > 0.6, agree  # (ties and one-ulp near-ties of 16-bit logits are common; the gap check above is the bound)
    # eager steps only (no captured graph): the same kernels, the same ids
    assert torch.equal(model.generate(prompt, new, use_cuda_graph=False), tokens)
    # the session and its captured step serve another prompt length and a shorter continuation
    prompt2 = prompt[:, : max(1, L0 // 2)].contiguous()
    t2 = model.generate(prompt2, new // 2)
    assert torch.equal(t2, model.generate(prompt2, new // 2, use_cuda_graph=False))
    _teacher_forced_check(model, prompt2, t2, tol)


def test_tiny_generation_matches_the_cpu_oracle():
    """Tiny fp32 configuration: cached generation on the GPU against the oracle's recompute-everything loop on the CPU;
    ids equal, or the oracle's own top-two gap at the first difference of a sequence is within the forward's
    end-to-end tolerance."""
    model, ocfg, sd = build_model(TINY, torch.float32, random_affine=True)
    prompt = torch.randint(0, TINY["vocab_size"], (2, 12), generator=torch.Generator().manual_seed(9))
    new = 10
    tokens = model.generate(prompt.to(DEV), new).cpu()
    ref, step_logits = orc.generate_by_recompute(sd, ocfg, prompt, new)
    for b in range(2):
        diff = (tokens[b] != ref[b]).nonzero()
        if len(diff):
            s = diff[0].item()
            top2 = step_logits[s][b].float().topk(2).values
            assert (top2[0] - top2[1]).item() < 2e-3, (b, s, tokens[b], ref[b])


def test_sampled_generation_is_reproducible_and_seeded():
    cfg = dict(vocab_size=512, block_size=128, n_layer=2, n_head=4, n_embd=256)
    model, _, _ = build_model(cfg, torch.float16, random_affine=True)
    prompt = torch.randint(0, 512, (8, 10), generator=torch.Generator().manual_seed(1)).to(DEV)
    a = model.generate(prompt, 30, temperature=0.9, top_k=50, seed=1)
    b = model.generate(prompt, 30, temperature=0.9, top_k=50, seed=1)
    c = model.generate(prompt, 30, temperature=0.9, top_k=50, seed=2)
    assert torch.equal(a, b) and not torch.equal(a, c)
    assert (a >= 0).all() and (a < 512).all()
    # top_k = 1 is greedy whatever the temperature (fp32 logits: no ties at the top)
    tiny, _, _ = build_model(TINY, torch.float32, random_affine=True)
    p32 = torch.randint(0, TINY["vocab_size"], (4, 9), generator=torch.Generator().manual_seed(2)).to(DEV)
    assert torch.equal(tiny.generate(p32, 12, temperature=0.9, top_k=1, seed=5), tiny.generate(p32, 12))


def test_generation_refuses_what_does_not_fit():
    cfg = dict(vocab_size=512, block_size=64, n_layer=1, n_head=4, n_embd=128)
    model, _, _ = build_model(cfg, torch.float16)
    prompt = torch.zeros((1, 60), dtype=torch.long, device=DEV)
    assert model.generate(prompt, 5).shape == (1, 5)  # positions 0..63
    with pytest.raises(AssertionError):
        model.generate(prompt, 6)


def test_generation_at_the_benchmark_size():
    """GPT-2 124M shapes, fp16, the benchmark's weights and ids: 512 prompts of 300 tokens, 8 tokens generated with the
    key/value cache (the one-warp-per-head attention variant, the narrow-tile GEMMs at 512 rows, the captured step).
    Size-independent properties: every generated token is an argmax, to rounding, of the full forward's logits over
    prompt + tokens at its position; and the continuations of sequences 0, 1, 510, 511 are bit-identical when those
    four are generated as a batch of their own (rows are independent of their batch)."""
    from test_gpu_model import GPT2_SMALL

    model, _, _ = build_model(GPT2_SMALL, torch.float16, scale_residual_proj=True)
    prompt = torch.randint(0, 50257, (512, 300), generator=torch.Generator().manual_seed(0)).to(DEV)
    new = 8
    tokens = model.generate(prompt, new)
    assert tokens.shape == (512, new) and (tokens >= 0).all() and (tokens < 50257).all()
    seq = torch.cat([prompt, tokens[:, :-1]], dim=1)
    hidden = model(seq)[:, 299:, :].contiguous()  # positions 299 .. 306 predict tokens 0 .. 7
    logits = model.lm_head(hidden).float()
    gap = (logits.max(dim=-1).values - logits.gather(-1, tokens.unsqueeze(-1)).squeeze(-1)).max().item()
    assert gap <= 2e-2, f"a generated token trails the recomputed argmax by {gap}"
    sel = torch.tensor([0, 1, 510, 511], device=DEV)
    assert torch.equal(model.generate(prompt[sel].contiguous(), new), tokens[sel])
