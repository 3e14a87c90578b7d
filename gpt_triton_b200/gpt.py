"""GPT-2 forward modules on top of the sm_100a operators, with the reference's module surface.

Class names, constructor arguments, parameter names and therefore the state-dict layout are
those of the reference (``FusedAttention`` gpt.py:21-67, ``FusedMLP`` gpt.py:70-119,
``GPTConfig`` gpt.py:122-129, ``FusedGPT`` gpt.py:132-196), so a converted Hugging Face GPT-2
state dict loads unchanged (gpt.py:199-247).  What is new:

* ``FusedGPT.forward`` still returns the final hidden state (gpt.py:180); ``FusedGPT.logits`` /
  ``FusedGPT.lm_head`` add the tied head that the reference leaves commented out
  (gpt.py:159-161, 172-179) and use ``wte`` itself as a K-major operand, not its transpose;
* every GEMM weight is packed once per parameter version into the tensor-core operand layout;
* in 16-bit models ``FusedGPT.forward`` folds the two LayerNorms of every block into the GEMMs that follow them
  (the fusion the reference leaves as a TODO, kernels.py:132-133): row statistics come out of the kernel that wrote
  the rows (embedding, c_proj, ffn2), the normalised activations are never written, and 24 of the 25 LayerNorm
  launches of a 12-layer forward disappear.  ``FusedGPT.fold_layer_norm = False`` (or calling a block module on its
  own) gives the operator-by-operator sequence of the reference; the two differ by roundings only;
* attention reads q/k/v as views of the c_attn output and writes merged heads, so the four
  per-layer copies of the reference (kernels.py:359-365, gpt.py:51) do not exist;
* ``GPU_TO_FLOPS`` has a ``"b200"`` entry, and ``executed_fwd_flops`` counts what the tensor
  cores really execute.

Forward/eval only: in the reference the training branch cannot run either (gpt.py:165 reads a
config field that gpt.py:129 does not define).
"""

import os
from dataclasses import dataclass

import torch
from torch import nn

from . import kernels as K

GPU_TO_FLOPS = {"v100": 130e12, "a100": 312e12, "h100": 989e12, "b200": 2250e12}
GPU_TO_FLOPS = {k: int(v) for k, v in GPU_TO_FLOPS.items()}


def _uniform(*shape):
    # the reference initialises every matrix and bias with torch.rand; real use loads a state dict
    return nn.Parameter(torch.rand(*shape))


def _ln_params(module, h):
    module.layer_norm_weight = nn.Parameter(torch.ones(h))
    module.layer_norm_bias = nn.Parameter(torch.zeros(h))


def _linear_flops(tokens, fan_in, fan_out):
    """Multiply-adds plus the bias add, the way the reference counts a projection."""
    return tokens * fan_out * 2 * fan_in + tokens * fan_out


def _ln_flops(tokens, h):
    return 2 * tokens * h


class _OperandCache:
    """Derived operands (PackedWeight and friends) per parameter; rebuilt when the parameter is replaced, cast,
    moved or written in place.  The tag uses the Parameter's own ``_version``, which ``load_state_dict``,
    ``param.copy_`` and optimizer steps bump (``param.data`` is a fresh tensor object whose counter always reads 0,
    so it cannot serve).  Writes made *through* ``param.data`` (``param.data.mul_(2)``) bump no counter torch
    exposes: after such a write call ``refresh_operands()`` on the model."""

    def __init__(self):
        self._slots = {}

    def clear(self):
        self._slots.clear()

    @staticmethod
    def _tag(param):
        return (param.data_ptr(), param._version, param.dtype, param.device, tuple(param.shape))

    def derived(self, key, params, make):
        """`make()` cached under `key` until one of `params` changes."""
        tag = tuple(self._tag(p) for p in params)
        slot = self._slots.get(key)
        if slot is None or slot[0] != tag:
            slot = (tag, make())
            self._slots[key] = slot
        return slot[1]

    def __call__(self, param, weight_is_nk=False):
        return self.derived(("packed", id(param), weight_is_nk), (param,),
                            lambda: K.pack_weight(param.data.contiguous(), weight_is_nk=weight_is_nk))

    def folded(self, weight, ln_weight, ln_bias, bias):
        """FoldedWeight of `weight` with the LayerNorm (ln_weight, ln_bias) in front of it and `bias` behind."""
        return self.derived(("folded", id(weight)), (weight, ln_weight, ln_bias, bias),
                            lambda: K.fold_layer_norm(weight.data.contiguous(), ln_weight.data.contiguous(), ln_bias.data.contiguous(),
                                                      bias.data.contiguous()))


class _EvalOnly(nn.Module):
    def _check_eval(self):
        if self.training:
            raise NotImplementedError("libb200gpt implements the forward/eval path only: call .eval() first")

    def refresh_operands(self):
        """Drop every cached derived operand (packed weights) of this module and its children; the next forward
        rebuilds them from the parameters.  Needed only after writes through ``param.data``, which torch's version
        counters do not see; ``load_state_dict``, ``copy_``, casts and moves are noticed without it."""
        for m in self.modules():
            cache = getattr(m, "_operand", None)
            if isinstance(cache, _OperandCache):
                cache.clear()


class FusedAttention(_EvalOnly):
    def __init__(self, hidden_size, num_heads, dropout_prob=0.0):
        super().__init__()
        self.hidden_size, self.num_heads, self.dropout_prob = hidden_size, num_heads, dropout_prob
        _ln_params(self, hidden_size)
        self.c_attn_weight = _uniform(hidden_size, 3 * hidden_size)
        self.c_attn_bias = _uniform(3 * hidden_size)
        self.c_proj_weight = _uniform(hidden_size, hidden_size)
        self.c_proj_bias = _uniform(hidden_size)
        self._operand = _OperandCache()

    def forward(self, x, kv_cache=None):
        """``kv_cache`` (batch, capacity, 2 * hidden), optional: receives the keys and values of these positions
        (the prompt of a generation)."""
        self._check_eval()
        skip = x
        y = K.fused_layer_norm(x, self.layer_norm_weight.data, self.layer_norm_bias.data)
        qkv = K.fused_ffn(y, self._operand(self.c_attn_weight), bias=self.c_attn_bias.data)
        if kv_cache is not None:
            K.kv_cache_fill(qkv, kv_cache)
        q, k, v = K.split_qkv(qkv, self.num_heads)
        y = K.flash_attention_v1(q, k, v, merged_heads=True).view(skip.shape)
        return K.fused_ffn(y, self._operand(self.c_proj_weight), bias=self.c_proj_bias.data, residual=skip)

    def forward_folded(self, x, stats, return_row_stats=True, kv_cache=None):
        """The same block with its LayerNorm folded into c_attn: x (batch, seqlen, hidden) are the raw rows,
        `stats` their RowStats.  Returns (output, RowStats of the output) for the block that follows."""
        self._check_eval()
        w = self._operand.folded(self.c_attn_weight, self.layer_norm_weight, self.layer_norm_bias, self.c_attn_bias)
        qkv = K.fused_ffn(x, w, ln_stats=stats)
        if kv_cache is not None:
            K.kv_cache_fill(qkv, kv_cache)
        q, k, v = K.split_qkv(qkv, self.num_heads)
        y = K.flash_attention_v1(q, k, v, merged_heads=True).view(x.shape)
        if not return_row_stats:
            return K.fused_ffn(y, self._operand(self.c_proj_weight), bias=self.c_proj_bias.data, residual=x), None
        return K.fused_ffn(y, self._operand(self.c_proj_weight), bias=self.c_proj_bias.data, residual=x, return_row_stats=True)

    def decode(self, x, stats, kv_cache, pos):
        """One generated token per sequence: x (batch, hidden) are the raw rows of the token at position pos[0],
        `stats` their RowStats (None: unfolded LayerNorm, as in forward()).  Its keys and values join `kv_cache` and
        its query attends over positions 0..pos[0].  Returns (output (batch, hidden), RowStats or None)."""
        self._check_eval()
        if stats is not None:
            w = self._operand.folded(self.c_attn_weight, self.layer_norm_weight, self.layer_norm_bias, self.c_attn_bias)
            qkv = K.fused_ffn(x, w, ln_stats=stats)
        else:
            y = K.fused_layer_norm(x, self.layer_norm_weight.data, self.layer_norm_bias.data)
            qkv = K.fused_ffn(y, self._operand(self.c_attn_weight), bias=self.c_attn_bias.data)
        y = K.attention_decode(qkv, kv_cache, pos, self.num_heads)
        if stats is None:
            return K.fused_ffn(y, self._operand(self.c_proj_weight), bias=self.c_proj_bias.data, residual=x), None
        return K.fused_ffn(y, self._operand(self.c_proj_weight), bias=self.c_proj_bias.data, residual=x, return_row_stats=True)

    def get_fwd_flops(self, num_tokens):
        h = self.hidden_size
        return _ln_flops(num_tokens, h) + _linear_flops(num_tokens, h, 3 * h) + _linear_flops(num_tokens, h, h)


class FusedMLP(_EvalOnly):
    def __init__(self, hidden_size, dropout_prob=0.0):
        super().__init__()
        self.hidden_size, self.intermediate_size, self.dropout_prob = hidden_size, 4 * hidden_size, dropout_prob
        _ln_params(self, hidden_size)
        self.ffn1_weight = _uniform(hidden_size, self.intermediate_size)
        self.ffn1_bias = _uniform(self.intermediate_size)
        self.ffn2_weight = _uniform(self.intermediate_size, hidden_size)
        self.ffn2_bias = _uniform(hidden_size)
        self._operand = _OperandCache()

    def forward(self, x):
        self._check_eval()
        y = K.fused_layer_norm(x, self.layer_norm_weight.data, self.layer_norm_bias.data)
        y = K.fused_ffn(y, self._operand(self.ffn1_weight), bias=self.ffn1_bias.data, add_gelu=True)
        return K.fused_ffn(y, self._operand(self.ffn2_weight), bias=self.ffn2_bias.data, residual=x)

    def forward_folded(self, x, stats, return_row_stats=True):
        """The same block with its LayerNorm folded into ffn1 (see FusedAttention.forward_folded)."""
        self._check_eval()
        w = self._operand.folded(self.ffn1_weight, self.layer_norm_weight, self.layer_norm_bias, self.ffn1_bias)
        y = K.fused_ffn(x, w, add_gelu=True, ln_stats=stats)
        if not return_row_stats:
            return K.fused_ffn(y, self._operand(self.ffn2_weight), bias=self.ffn2_bias.data, residual=x), None
        return K.fused_ffn(y, self._operand(self.ffn2_weight), bias=self.ffn2_bias.data, residual=x, return_row_stats=True)

    def get_fwd_flops(self, num_tokens):
        h, mid = self.hidden_size, self.intermediate_size
        return _ln_flops(num_tokens, h) + _linear_flops(num_tokens, h, mid) + _linear_flops(num_tokens, mid, h)


@dataclass
class GPTConfig:
    vocab_size: int = 50304
    block_size: int = 512
    n_layer: int = 12
    n_head: int = 12
    n_embd: int = 768
    dropout: float = 0.1


class FusedGPT(_EvalOnly):
    # Fold the LayerNorms of the blocks into the GEMMs behind them (16-bit models; see the module docstring).  The
    # environment variable B200GPT_FOLD_LAYERNORM=0 changes the default for the process; the attribute can also be set
    # per model.
    fold_layer_norm = os.environ.get("B200GPT_FOLD_LAYERNORM", "1") != "0"

    def __init__(self, config):
        super().__init__()
        self.config = config
        h = config.n_embd
        self.wte_weight = _uniform(config.vocab_size, h)
        self.wpe_weight = _uniform(config.block_size, h)
        layers = []
        for _ in range(config.n_layer):
            layers.append(nn.Sequential(FusedAttention(h, config.n_head, dropout_prob=config.dropout),
                                        FusedMLP(h, dropout_prob=config.dropout)))
        self.blocks = nn.ModuleList(layers)
        _ln_params(self, h)
        self._operand = _OperandCache()

    def _folds(self):
        return self.fold_layer_norm and self.wte_weight.dtype in (torch.float16, torch.bfloat16) and self.config.n_embd % 8 == 0

    def _body(self, x, kv_caches=None):
        """ids (batch, seqlen) -> residual stream before the final LayerNorm; kv_caches: one tensor per layer that
        receives the layer's keys and values (the prompt of a generation)."""
        self._check_eval()
        cache = (lambda i: None) if kv_caches is None else (lambda i: kv_caches[i])
        if self._folds():
            y, stats = K.fused_embeddings(x, self.wte_weight.data, self.wpe_weight.data, return_row_stats=True)
            last = len(self.blocks) - 1
            for i, (attention, mlp) in enumerate(self.blocks):
                y, stats = attention.forward_folded(y, stats, kv_cache=cache(i))
                y, stats = mlp.forward_folded(y, stats, return_row_stats=i != last)  # the final LayerNorm stays a kernel
        else:
            y = K.fused_embeddings(x, self.wte_weight.data, self.wpe_weight.data)
            for i, (attention, mlp) in enumerate(self.blocks):
                y = mlp(attention(y, kv_cache=cache(i)))
        return y

    def forward(self, x):
        """ids (batch, seqlen) -> final hidden state (batch, seqlen, n_embd)."""
        return K.fused_layer_norm(self._body(x), self.layer_norm_weight.data, self.layer_norm_bias.data)

    def _decode_body(self, ids, kv_caches, pos):
        """ids (batch,) of the tokens at position pos[0] -> their final hidden state (batch, n_embd); their keys and
        values join the caches."""
        self._check_eval()
        B = ids.shape[0]
        if self._folds():
            y, stats = K.fused_embeddings(ids.view(B, 1), self.wte_weight.data, self.wpe_weight.data, return_row_stats=True, position=pos)
            y = y.view(B, -1)
            last = len(self.blocks) - 1
            for i, (attention, mlp) in enumerate(self.blocks):
                y, stats = attention.decode(y, stats, kv_caches[i], pos)
                y, stats = mlp.forward_folded(y, stats, return_row_stats=i != last)
        else:
            y = K.fused_embeddings(ids.view(B, 1), self.wte_weight.data, self.wpe_weight.data, position=pos).view(B, -1)
            for i, (attention, mlp) in enumerate(self.blocks):
                y = mlp(attention.decode(y, None, kv_caches[i], pos)[0])
        return K.fused_layer_norm(y, self.layer_norm_weight.data, self.layer_norm_bias.data)

    def _pick(self, hidden, temperature, top_k, seed, pos):
        """hidden (batch, n_embd), final LayerNorm applied -> next ids (batch,) int64: greedy (temperature 0: row
        argmax in the lm_head's epilogue, logits not written for 16-bit models) or sampled."""
        B, h = hidden.shape
        w = self._operand(self.wte_weight, weight_is_nk=True)
        if temperature == 0.0 and hidden.dtype != torch.float32:
            return K.ffn_row_statistics(hidden, w, want_lse=False)[0]
        V = self.config.vocab_size
        pitch = (V + 63) // 64 * 64
        buf = torch.empty((B, pitch), device=hidden.device, dtype=hidden.dtype)
        logits = K.fused_ffn(hidden, w, out=buf[:, :V])
        if temperature == 0.0:
            return logits.argmax(dim=-1)
        return K.sample_logits(logits, temperature=temperature, top_k=top_k, seed=seed, step=pos)

    @torch.no_grad()
    def generate(self, ids, max_new_tokens, temperature=0.0, top_k=0, seed=0, use_cuda_graph=True):
        """ids (batch, prompt_len) -> (batch, max_new_tokens) int64 continuation, one token per step with a key/value
        cache (the inference loop the reference's README.md:55 lists as not built).  temperature 0: greedy; > 0:
        draws from softmax(logits / temperature) over the top_k largest logits (0 = all), reproducible for a given
        seed.  The sessions (cache, captured decode step) are kept on the model per
        (batch, capacity, temperature, top_k, seed) and re-used by later calls of the same shape."""
        B, L0 = ids.shape
        need = L0 + max_new_tokens - 1
        key = (B, temperature, top_k, seed, use_cuda_graph, self.wte_weight.dtype, self.wte_weight.device)
        sessions = self.__dict__.setdefault("_sessions", {})
        session = sessions.get(key)
        if session is None or session.capacity < need or session.tokens.shape[1] < max_new_tokens or session.stale():
            sessions.pop(key, None)
            while len(sessions) >= 4:  # every session holds a cache: keep a few
                sessions.pop(next(iter(sessions)))
            sessions[key] = session = GenerationSession(self, B, capacity=need, max_new_tokens=max_new_tokens, temperature=temperature,
                                                        top_k=top_k, seed=seed, use_cuda_graph=use_cuda_graph)
        return session.generate(ids, max_new_tokens)

    @torch.no_grad()
    def lm_head(self, hidden, return_argmax=False, return_lse=False):
        """hidden (batch, seqlen, n_embd) -> logits (batch, seqlen, vocab_size) with the tied
        embedding matrix.  The logits buffer's row pitch is padded to a multiple of 64 elements so
        every row starts 128-byte aligned (wide stores); the result is the [..., :vocab_size] view
        of it.  ``return_argmax=True`` also returns the greedy next-token ids (batch, seqlen), taken
        in the GEMM's epilogue (16-bit models); ``return_lse=True`` additionally the row log-sum-exp
        (batch, seqlen) float32, so that a token's cross-entropy is lse - logits[target]."""
        B, L, h = hidden.shape
        V = self.config.vocab_size
        pitch = (V + 63) // 64 * 64
        buf = torch.empty((B * L, pitch), device=hidden.device, dtype=hidden.dtype)
        w = self._operand(self.wte_weight, weight_is_nk=True)
        if (return_argmax or return_lse) and hidden.dtype != torch.float32:
            res = K.fused_ffn(hidden.reshape(B * L, h), w, out=buf[:, :V], return_argmax=True, return_lse=return_lse)
            logits = buf.view(B, L, pitch)[:, :, :V]
            return (logits, res[1].view(B, L), res[2].view(B, L)) if return_lse else (logits, res[1].view(B, L))
        K.fused_ffn(hidden.reshape(B * L, h), w, out=buf[:, :V])
        logits = buf.view(B, L, pitch)[:, :, :V]
        if return_lse:
            return logits, logits.argmax(dim=-1), torch.logsumexp(logits.float(), dim=-1)
        return (logits, logits.argmax(dim=-1)) if return_argmax else logits

    @torch.no_grad()
    def logits(self, x):
        """ids -> logits: forward() followed by the tied lm_head."""
        return self.lm_head(self.forward(x))

    @torch.no_grad()
    def logits_and_next_ids(self, x):
        """ids -> (logits, greedy next-token ids): forward(), then the tied lm_head with the argmax fused
        into its epilogue."""
        return self.lm_head(self.forward(x), return_argmax=True)

    @torch.no_grad()
    def next_ids(self, x):
        """ids (batch, seqlen) -> greedy next-token ids (batch, seqlen): forward(), then the tied lm_head reduced to its
        row argmax inside the GEMM's epilogue; the (tokens, vocab) logits are never written (16-bit models; fp32 models
        go through the logits)."""
        hidden = self.forward(x)
        if hidden.dtype == torch.float32:
            return self.lm_head(hidden, return_argmax=True)[1]
        B, L, h = hidden.shape
        w = self._operand(self.wte_weight, weight_is_nk=True)
        return K.ffn_row_statistics(hidden.reshape(B * L, h), w, want_lse=False)[0].view(B, L)

    @torch.no_grad()
    def token_nll(self, x, targets):
        """ids, targets (batch, seqlen) -> per-token cross-entropy (batch, seqlen) float32 =
        lse(logits) - logits[target], over the logits as the lm_head would round them.  16-bit models take both terms
        out of the lm_head GEMM's epilogue without writing the logits; fp32 models go through the logits."""
        hidden = self.forward(x)
        if hidden.dtype == torch.float32:
            logits, _, lse = self.lm_head(hidden, return_argmax=True, return_lse=True)
            return lse - logits.gather(-1, targets.unsqueeze(-1)).squeeze(-1)
        B, L, h = hidden.shape
        w = self._operand(self.wte_weight, weight_is_nk=True)
        _, lse, picked = K.ffn_row_statistics(hidden.reshape(B * L, h), w, targets=targets.reshape(B * L).contiguous())
        return (lse - picked).view(B, L)

    def get_fwd_flops(self, num_tokens):
        """The reference's analytic count (gpt.py:182-196): embeddings counted as matmuls,
        attention score/value products not counted."""
        c = self.config
        total = sum(m.get_fwd_flops(num_tokens) for pair in self.blocks for m in pair)
        total += _ln_flops(num_tokens, c.n_embd)
        total += num_tokens * c.n_embd * 2 * (c.vocab_size + c.block_size)
        return total


class GraphedForward:
    """One forward of a FusedGPT for a fixed (batch, seqlen), captured in a CUDA graph and replayed.

    The 87 kernel launches of a 12-layer forward cost the host a few milliseconds; at small batches that is
    more than the GPU needs (8 x 300 tokens: 2.9 ms eager, 1.4 ms replayed on a B200).  ``what`` selects the
    captured method: "forward" (hidden state), "logits", "logits_and_next_ids" or "next_ids".  The results are static
    buffers that every call overwrites; clone them to keep them."""

    def __init__(self, model, example_ids, what="logits", warmup=3):
        assert what in ("forward", "logits", "logits_and_next_ids", "next_ids")
        self._model, self._warmup = model, warmup
        self._fn = getattr(model, what)
        self.static_ids = example_ids.clone()
        self._capture()

    def _signature(self):
        return tuple(_OperandCache._tag(p) for p in self._model.parameters())

    def _capture(self):
        dev = self.static_ids.device
        # warm-up on a side stream: first calls set kernel attributes, pack weights and fill the allocator's pool
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side), torch.no_grad():
            for _ in range(max(1, self._warmup)):
                self._fn(self.static_ids)
        torch.cuda.current_stream(dev).wait_stream(side)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph), torch.no_grad():
            self.outputs = self._fn(self.static_ids)
        self._sig = self._signature()

    def __call__(self, ids):
        assert ids.shape == self.static_ids.shape, "a captured forward serves one (batch, seqlen) only"
        if self._signature() != self._sig:
            # a parameter was reloaded, cast or replaced since the capture: the graph holds the old packed operands
            self._capture()
        self.static_ids.copy_(ids)
        self.graph.replay()
        return self.outputs


class GenerationSession:
    """Token-by-token generation for a fixed batch size: the key/value cache of every layer
    ((batch, capacity, 2 * n_embd) each), the device-side position counter and, after the first two decode steps,
    a CUDA graph of one decode step that is replayed for every further token of this and later generations (any
    prompt length: the position lives in device memory).  Prompt + generated tokens - 1 must fit both `capacity`
    and the model's position table.  No counterpart in the reference (README.md:55)."""

    EAGER_STEPS = 2  # decode steps run eagerly before the capture (kernel attributes, allocator pools)

    def __init__(self, model, batch, capacity, max_new_tokens, temperature=0.0, top_k=0, seed=0, use_cuda_graph=True):
        cfg = model.config
        assert capacity <= cfg.block_size, f"{capacity} positions exceed the position table ({cfg.block_size} rows)"
        assert temperature >= 0.0 and top_k >= 0 and max_new_tokens >= 1
        dev, dtype = model.wte_weight.device, model.wte_weight.dtype
        self.model, self.batch, self.capacity = model, batch, max(int(capacity), 1)
        self.temperature, self.top_k, self.seed, self.use_cuda_graph = float(temperature), int(top_k), int(seed), use_cuda_graph
        self.kv = [torch.empty((batch, self.capacity, 2 * cfg.n_embd), device=dev, dtype=dtype) for _ in range(cfg.n_layer)]
        self.pos = torch.zeros(2, device=dev, dtype=torch.int32)  # {tokens in the cache, prompt length}
        self.tokens = torch.zeros((batch, max_new_tokens), device=dev, dtype=torch.int64)
        self.feedback = torch.zeros((batch,), device=dev, dtype=torch.int64)  # the ids the next decode step embeds
        self.graph = None
        self._sig = self._signature()

    def _signature(self):
        return tuple(_OperandCache._tag(p) for p in self.model.parameters())

    def stale(self):
        """True once a parameter has been reloaded, cast or moved: a captured step holds the old operands."""
        return self._signature() != self._sig

    def _step(self):
        m = self.model
        hidden = m._decode_body(self.feedback, self.kv, self.pos)
        ids = m._pick(hidden, self.temperature, self.top_k, self.seed, self.pos)
        K.decode_append(ids, self.tokens, self.pos, advance=True, feedback=self.feedback)

    @torch.no_grad()
    def generate(self, ids, max_new_tokens):
        m = self.model
        B, L0 = ids.shape
        assert B == self.batch and L0 >= 1 and 1 <= max_new_tokens <= self.tokens.shape[1]
        assert L0 + max_new_tokens - 1 <= self.capacity, "prompt + generated tokens do not fit this session's cache"
        assert not self.stale(), "the model's parameters changed: make a new session"
        dev = self.pos.device
        # prompt: the usual forward, its keys/values copied into the caches; next id from the last position
        y = m._body(ids, kv_caches=self.kv)
        last = K.fused_layer_norm(y[:, -1, :].contiguous(), m.layer_norm_weight.data, m.layer_norm_bias.data)
        self.pos.copy_(torch.tensor([L0, L0], dtype=torch.int32), non_blocking=False)
        first = m._pick(last, self.temperature, self.top_k, self.seed, self.pos)
        K.decode_append(first, self.tokens, self.pos, advance=False, feedback=self.feedback)
        steps = max_new_tokens - 1
        done = 0
        if self.graph is None:
            while done < min(steps, self.EAGER_STEPS):
                self._step()
                done += 1
            if self.use_cuda_graph and done < steps:
                torch.cuda.synchronize(dev)
                self.graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(self.graph):
                    self._step()
        for _ in range(steps - done):
            if self.graph is not None:
                self.graph.replay()
            else:
                self._step()
        code = K.device_status(dev)
        if code:
            raise RuntimeError(f"generation stopped by a device-side check (code {code}): cache or token buffer out of room")
        return self.tokens[:, :max_new_tokens].clone()


def executed_fwd_flops(config, batch, seqlen, with_lm_head=True):
    """Tensor-core flop one forward really executes: the four projections of every layer,
    causal attention (QK^T and PV over the lower triangle) and optionally the tied lm_head."""
    T, h, d = batch * seqlen, config.n_embd, config.n_embd // config.n_head
    gemm = 2 * T * 12 * h * h * config.n_layer
    attn = 4 * batch * config.n_head * d * (seqlen * (seqlen + 1) // 2) * config.n_layer
    head = 2 * T * h * config.vocab_size if with_lm_head else 0
    return gemm + attn + head


_HF_TOP = {"wte.weight": "wte_weight", "wpe.weight": "wpe_weight", "ln_f.weight": "layer_norm_weight", "ln_f.bias": "layer_norm_bias"}
# (HF sub-key, slot in the nn.Sequential pair, our parameter stem)
_HF_BLOCK = [("ln_1", 0, "layer_norm"), ("attn.c_attn", 0, "c_attn"), ("attn.c_proj", 0, "c_proj"),
             ("ln_2", 1, "layer_norm"), ("mlp.c_fc", 1, "ffn1"), ("mlp.c_proj", 1, "ffn2")]
_HF_DROPPED = ("attn.bias", "attn.masked_bias")  # causal-mask buffers of older HF versions


def convert_huggingface_to_triton(hf_sd, hf_config):
    """Hugging Face ``GPT2Model`` state dict -> (``FusedGPT`` state dict, ``GPTConfig``).

    Pure key renaming as in gpt.py:199-237 (HF Conv1D weights are already [in, out]); mask
    buffers are dropped; ``n_positions`` stands in when the config carries no ``n_ctx``."""
    config = GPTConfig(vocab_size=hf_config.vocab_size, block_size=getattr(hf_config, "n_ctx", None) or hf_config.n_positions,
                       n_layer=hf_config.n_layer, n_head=hf_config.n_head, n_embd=hf_config.n_embd, dropout=0.1)
    rename = dict(_HF_TOP)
    for i in range(config.n_layer):
        for hf_stem, slot, stem in _HF_BLOCK:
            for kind in ("weight", "bias"):
                rename[f"h.{i}.{hf_stem}.{kind}"] = f"blocks.{i}.{slot}.{stem}_{kind}"
        for dropped in _HF_DROPPED:
            rename[f"h.{i}.{dropped}"] = None
    out = {}
    for name, tensor in hf_sd.items():
        target = rename[name]  # KeyError on an unknown key, like the reference
        if target is not None:
            out[target] = tensor
    return out, config


def convert_hf_and_load_model(model_id, device):
    """As gpt.py:240-247; needs the Hugging Face checkpoint to be reachable."""
    from transformers import GPT2Model

    hf_model = GPT2Model.from_pretrained(model_id)
    state_dict, config = convert_huggingface_to_triton(hf_model.state_dict(), hf_model.config)
    model = FusedGPT(config)
    model.load_state_dict(state_dict)
    return model.to(device).eval(), hf_model.to(device).eval()


def estimate_days(flops, mfu=0.45, gpu="h100", num_gpus=1):
    assert gpu in GPU_TO_FLOPS
    per_day = mfu * GPU_TO_FLOPS[gpu] * 3600 * 24 * num_gpus
    return flops / per_day


def get_num_parameters(model):
    return sum(p.numel() for p in model.parameters())


def compute_mfu(flops_per_second, gpu="h100"):
    assert gpu in GPU_TO_FLOPS
    return flops_per_second / GPU_TO_FLOPS[gpu]
