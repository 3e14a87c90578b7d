"""GPU: b200_ffn_static_scratch, the fused_ffn entry point for callers that may not allocate device
memory (its packing scratch is a fixed array inside the library).  Collected last on purpose.

Called through the C ABI twice in a row with different problems and compared, bit for bit (the same
kernels run on both sides), with b200_ffn given a caller-allocated workspace."""

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _run_both(lib, _lib, x, w, b, r, gelu, w_is_nk):
    M, K = x.shape
    N = w.shape[0] if w_is_nk else w.shape[1]
    dt = _lib.dtype_code(x.dtype)
    stream = _lib.stream_ptr(x.device)
    need = lib.b200_ffn_workspace_bytes(M, N, K, int(w_is_nk), dt)
    ws = torch.empty(max(need, 1), dtype=torch.uint8, device=DEV)
    ref = torch.full((M, N), float("nan"), dtype=x.dtype, device=DEV)
    st = lib.b200_ffn(x.data_ptr(), w.data_ptr(), b.data_ptr(), None if r is None else r.data_ptr(), ref.data_ptr(), M, N, K, N,
                      int(w_is_nk), int(gelu), dt, ws.data_ptr(), need, None, stream)
    assert st == 0, lib.b200_status_string(st)
    out = torch.full((M, N), float("nan"), dtype=x.dtype, device=DEV)
    st = lib.b200_ffn_static_scratch(x.data_ptr(), w.data_ptr(), b.data_ptr(), None if r is None else r.data_ptr(), out.data_ptr(), M, N,
                                     K, N, int(w_is_nk), int(gelu), dt, None, stream)
    assert st == 0, lib.b200_status_string(st)
    torch.cuda.synchronize()
    assert torch.isfinite(ref.float()).all()
    assert torch.equal(out, ref), (out.float() - ref.float()).abs().max().item()
    return out


def test_static_scratch_matches_workspace_entry_point_on_two_calls_in_a_row():
    from gpt_triton_b200 import _lib

    lib = _lib.load()
    g = torch.Generator().manual_seed(7)
    # call 1: fp32 storage, ragged K -> x and w are both packed into the scratch
    x1 = torch.randn((300, 72), generator=g).to(DEV)
    w1 = (torch.randn((72, 520), generator=g) * 0.1).to(DEV)
    b1 = torch.randn(520, generator=g).to(DEV)
    o1 = _run_both(lib, _lib, x1, w1, b1, None, True, False)
    # call 2, straight after: smaller fp16 problem with residual -> only w is packed, over call 1's leftovers
    x2 = torch.randn((130, 64), generator=g).half().to(DEV)
    w2 = (torch.randn((64, 200), generator=g) * 0.1).half().to(DEV)
    b2 = torch.randn(200, generator=g).half().to(DEV)
    r2 = torch.randn((130, 200), generator=g).half().to(DEV)
    _run_both(lib, _lib, x2, w2, b2, r2, False, False)
    # and call 1 again: the shared array must not remember call 2
    assert torch.equal(_run_both(lib, _lib, x1, w1, b1, None, True, False), o1)


def test_static_scratch_rejects_problems_beyond_its_capacity():
    from gpt_triton_b200 import _lib

    lib = _lib.load()
    x = torch.zeros((8, 8), device=DEV)
    # 2^20 x 4096 fp32: the packed x alone would be 8 GiB
    st = lib.b200_ffn_static_scratch(x.data_ptr(), x.data_ptr(), None, None, x.data_ptr(), 1 << 20, 4096, 4096, 4096, 0, 0, _lib.F32, None,
                                     _lib.stream_ptr(x.device))
    assert st == 5 and lib.b200_status_string(st) == b"workspace missing or too small"
    torch.cuda.synchronize()
