"""Failure detection without a GPU fault: the bounded wait every tensor-core kernel uses runs out on a barrier that
nothing completes, the kernel reports a status code and returns, and the context stays usable."""

import time

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def test_bounded_wait_runs_out_and_reports():
    from gpt_triton_b200 import _lib
    from gpt_triton_b200 import kernels as K

    t0 = time.perf_counter()
    code = K.bounded_wait_selftest(limit_cycles=200_000_000)  # about 0.1 s of SM clock
    elapsed = time.perf_counter() - t0
    assert code == 6 and _lib.load().b200_status_string(code) == b"a kernel abandoned a bounded wait"
    assert 0.02 < elapsed < 5.0
    # the context is alive and the library still computes
    x = torch.randn((64, 64), device=DEV).half()
    w = torch.randn((64, 32), device=DEV).half()
    z = K.fused_ffn(x, w)
    torch.cuda.synchronize()
    assert torch.isfinite(z.float()).all()
    assert (z.float() - x.float() @ w.float()).abs().max().item() < 0.1


def test_status_word_stays_zero_on_healthy_runs():
    from gpt_triton_b200 import kernels as K

    x = torch.randn((300, 768), device=DEV).half()
    pw = K.pack_weight(torch.randn((768, 768), device=DEV).half() * 0.02)
    K.fused_ffn(x, pw, residual=x)
    qkv = (torch.randn((2, 130, 2304), device=DEV) / 8).half()
    q, k, v = (t.view(2, 130, 12, 64).transpose(1, 2) for t in qkv.split(768, dim=2))
    K.flash_attention_v1(q, k, v)
    assert K.device_status() == 0
