"""Generate the golden vectors under tests/golden/ by running the UNMODIFIED reference.

Run where the reference checkout is available (it is not needed, nor read, by any
test at run time):

    python tests/golden/make_golden.py --reference /path/to/gpt-triton

The reference's Triton kernels are executed by Triton's numpy interpreter
(TRITON_INTERPRET=1, CPU only).  One shim is applied, outside the reference's
files: triton 3.6's interpreter refuses a Python ``bool`` for the non-constexpr
``apply_gelu`` argument (kernels.py:179, 306), so ``bool`` launch arguments are
passed on as ``int``.  Inputs are drawn exactly as the tests draw them again
(seeded CPU generators); every fixture also stores its inputs so that the tests do
not depend on generator reproducibility.
"""

import argparse
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"
os.environ.setdefault("PYTHONDONTWRITEBYTECODE", "1")
sys.dont_write_bytecode = True

import numpy as np  # noqa: E402
import torch  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import gpt2_oracle as orc  # noqa: E402  (only for the seeded weight generator)


def install_bool_shim():
    import triton.runtime.interpreter as interp

    orig = interp._implicit_cvt

    def cvt(arg):
        if isinstance(arg, bool):
            arg = int(arg)
        return orig(arg)

    interp._implicit_cvt = cvt


def to_np(t):
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().copy()  # raw bits; tests view them back
    return t.numpy().copy()


def save(name, **arrays):
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **{k: (to_np(v) if isinstance(v, torch.Tensor) else np.asarray(v)) for k, v in arrays.items()})
    print("wrote", path, os.path.getsize(path) // 1024, "KiB")


def ref_test_inputs(M, K, N):
    """test.py:17-25."""
    torch.manual_seed(1337)
    x = torch.rand((M, K), dtype=torch.float32)
    w = torch.rand((K, N), dtype=torch.float32)
    b = torch.rand((N,), dtype=torch.float32)
    r = torch.rand_like(x, dtype=torch.float32)
    if K != N:
        r = None
    return x, w, b, r


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of a checkout of thevasudevgupta/gpt-triton")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    install_bool_shim()
    import gpt as ref_gpt
    import kernels as ref_k

    # ---------------------------------------------------------------- embeddings (test.py:28-44)
    # No bf16 case: Triton 3.6's numpy interpreter keeps bf16 values as raw 16-bit integers and the
    # kernel's same-dtype `z += ...` (kernels.py:68-69) then adds the bit patterns, so a bf16
    # embedding (and with it a whole bf16 model) is garbage under the interpreter.  bf16 vectors
    # exist only for the kernels that widen their loads first (LayerNorm, GEMM, attention).
    g = torch.Generator().manual_seed(11)
    for tag, (V, B, H, L, P, dt) in {
        "emb_f32": (32, 8, 128, 10, 20, torch.float32),
        "emb_f32_full": (2, 8, 256, 20, 20, torch.float32),
        "emb_f16": (32, 4, 96, 7, 9, torch.float16),
    }.items():
        x = torch.randint(0, V, (B, L), generator=g)
        wte = torch.rand((V, H), generator=g).to(dt)
        wpe = torch.rand((P, H), generator=g).to(dt)
        z = ref_k.fused_embeddings(x, wte, wpe)
        save(tag, x=x, wte=wte, wpe=wpe, z=z)

    # ---------------------------------------------------------------- layer norm (test.py:47-59)
    for M, K in [(249, 123), (32, 128), (32, 64)]:
        x, *_ = ref_test_inputs(M, K, 32)
        w = torch.ones(K)
        b = torch.zeros(K)
        z = ref_k.fused_layer_norm(x, w, b)
        save(f"ln_f32_{M}x{K}", x=x, w=w, b=b, z=z)
    g = torch.Generator().manual_seed(12)
    for tag, (M, K, dt) in {"ln_f16": (37, 768, torch.float16), "ln_bf16": (19, 1600, torch.bfloat16), "ln_f32_affine": (21, 200, torch.float32)}.items():
        x = (torch.randn((M, K), generator=g) * 1.7 + 0.3).to(dt)
        w = (1 + 0.2 * torch.randn(K, generator=g)).to(dt)
        b = (0.1 * torch.randn(K, generator=g)).to(dt)
        z = ref_k.fused_layer_norm(x, w, b)
        save(tag, x=x, w=w, b=b, z=z)

    # ---------------------------------------------------------------- GEMM (test.py:62-87)
    for M, N, K in [(128, 128, 256), (199, 129, 129), (61, 31, 23)]:
        x, w, b, r = ref_test_inputs(M, K, N)
        for gelu in (True, False):
            for use_b in (True, False):
                z = ref_k.fused_ffn(x, w, bias=b if use_b else None, residual=r, add_gelu=gelu)
                extra = {} if r is None else {"r": r}
                save(f"ffn_f32_{M}x{N}x{K}_g{int(gelu)}_b{int(use_b)}", x=x, w=w, b=b, z=z, **extra)
    g = torch.Generator().manual_seed(13)
    for tag, (M, N, K, dt) in {"ffn_f16": (70, 96, 64, torch.float16), "ffn_bf16": (33, 72, 40, torch.bfloat16)}.items():
        x = torch.randn((M, K), generator=g).to(dt)
        w = (0.05 * torch.randn((K, N), generator=g)).to(dt)
        b = (0.1 * torch.randn(N, generator=g)).to(dt)
        r = torch.randn((M, N), generator=g).to(dt)
        save(tag + "_gelu", x=x, w=w, b=b, z=ref_k.fused_ffn(x, w, bias=b, add_gelu=True))
        save(tag + "_res", x=x, w=w, b=b, r=r, z=ref_k.fused_ffn(x, w, bias=b, residual=r))

    # ---------------------------------------------------------------- attention (test.py:90-117)
    def attn_inputs(B, N, L, H):  # test.py:90-95
        torch.manual_seed(1337)
        q = torch.rand((B, N, L, H))
        return q, torch.rand_like(q), torch.rand_like(q)

    for B, N, L, H in [(2, 3, 199, 64), (1, 2, 128, 128), (1, 2, 63, 256), (2, 2, 70, 32), (1, 3, 65, 16)]:
        q, k, v = attn_inputs(B, N, L, H)
        save(f"attn_f32_{B}x{N}x{L}x{H}", q=q, k=k, v=v, z=ref_k.flash_attention_v1(q, k, v))
    g = torch.Generator().manual_seed(14)
    for tag, (B, N, L, H, dt) in {"attn_f16": (1, 2, 150, 64, torch.float16), "attn_bf16": (1, 2, 100, 64, torch.bfloat16), "attn_f32_randn": (1, 2, 200, 64, torch.float32)}.items():
        q, k, v = (torch.randn((B, N, L, H), generator=g).to(dt) for _ in range(3))
        save(tag, q=q, k=k, v=v, z=ref_k.flash_attention_v1(q, k, v))

    # ---------------------------------------------------------------- qkv split (kernels.py:348-367)
    g = torch.Generator().manual_seed(15)
    x = torch.randn((2, 9, 48), generator=g)
    w = 0.1 * torch.randn((48, 144), generator=g)
    b = 0.1 * torch.randn(144, generator=g)
    q, k, v = ref_k.matmul_and_split_qkv(x, w, b, 4)
    save("qkv_f32", x=x, w=w, b=b, q=q, k=k, v=v)

    # ---------------------------------------------------------------- tiny GPT-2 end to end
    # n_layer=2, n_embd=128, n_head=4, vocab=1024, n_positions=128, batch 2 x seq 64
    def run_model(tag, dtype, random_affine, B=2, L=64):
        cfg = ref_gpt.GPTConfig(vocab_size=1024, block_size=128, n_layer=2, n_head=4, n_embd=128, dropout=0.1)
        ocfg = orc.OracleConfig(**cfg.__dict__)
        sd = orc.seeded_state_dict(ocfg, seed=0, dtype=torch.float32, random_affine=random_affine)
        model = ref_gpt.FusedGPT(cfg)
        model.load_state_dict(sd)
        model = model.to(dtype).eval()
        ids = torch.randint(0, 1024, (B, L), generator=torch.Generator().manual_seed(0))
        inter = {}
        with torch.no_grad():
            x = ref_k.fused_embeddings(ids, model.wte_weight.data, model.wpe_weight.data)
            inter["emb"] = x
            for i, block in enumerate(model.blocks):
                x = block[0](x)
                inter[f"attn{i}"] = x
                x = block[1](x)
                inter[f"mlp{i}"] = x
            hidden_manual = ref_k.fused_layer_norm(x, model.layer_norm_weight.data, model.layer_norm_bias.data)
            hidden = model(ids)
            assert torch.equal(hidden, hidden_manual)
            logits = ref_k.fused_ffn(hidden, model.wte_weight.data.T.contiguous())
        wsum = np.array([float(v.double().sum()) for v in sd.values()])
        save(tag, ids=ids, hidden=hidden, logits=logits, weight_sums=wsum, **inter)

    run_model("tiny_f32", torch.float32, False)
    run_model("tiny_f32_affine", torch.float32, True)
    run_model("tiny_f16_affine", torch.float16, True, B=2, L=40)

    # ---------------------------------------------------------------- accounting known answers
    cfg = ref_gpt.GPTConfig()
    model = ref_gpt.FusedGPT(cfg).eval()
    save(
        "accounting",
        fwd_flops_1024=np.array([model.get_fwd_flops(1024)], dtype=np.int64),
        num_parameters=np.array([ref_gpt.get_num_parameters(model)], dtype=np.int64),
        estimate_days=np.array([ref_gpt.estimate_days(6 * (405 * 10**9) * (15 * 10**12), mfu=0.45, gpu="h100", num_gpus=16_000)]),
        mfu=np.array([ref_gpt.compute_mfu(1e14, "a100")]),
        state_dict_keys=np.array(list(model.state_dict().keys())),
    )


if __name__ == "__main__":
    main()
