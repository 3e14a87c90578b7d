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


def test_static_scratch_capacity_boundary_with_honestly_sized_buffers():
    """The 32 MiB array holds exactly an fp32 problem with M = N = 8192, K = 1024 (2 x 16 MiB of packed operands): that
    call is served; 8 more rows of x are refused with B200_ERR_WORKSPACE before anything is launched.  Every pointer
    handed in covers the sizes it claims, so a regression of the size check would show as a wrong status or result,
    not as an out-of-bounds access."""
    from gpt_triton_b200 import _lib

    lib = _lib.load()
    g = torch.Generator().manual_seed(11)
    K, N = 1024, 8192
    w = (torch.randn((K, N), generator=g) * 0.05).to(DEV)
    x_big = torch.randn((8200, K), generator=g).to(DEV)
    out = torch.empty((8200, N), device=DEV)
    stream = _lib.stream_ptr(x_big.device)
    assert lib.b200_ffn_workspace_bytes(8192, N, K, 0, _lib.F32) == 32 << 20
    st = lib.b200_ffn_static_scratch(x_big.data_ptr(), w.data_ptr(), None, None, out.data_ptr(), 8192, N, K, N, 0, 0, _lib.F32, None, stream)
    assert st == 0, lib.b200_status_string(st)
    torch.cuda.synchronize()
    rows = torch.tensor([0, 1, 4095, 8191], device=DEV)
    ref = x_big[rows].cpu().half().float() @ w.cpu().half().float()  # operands rounded to fp16 as the operator rounds them
    assert (out[rows].cpu() - ref).abs().max().item() < 2e-3
    out.fill_(float("nan"))
    st = lib.b200_ffn_static_scratch(x_big.data_ptr(), w.data_ptr(), None, None, out.data_ptr(), 8200, N, K, N, 0, 0, _lib.F32, None, stream)
    assert st == 5 and lib.b200_status_string(st) == b"workspace missing or too small"
    torch.cuda.synchronize()
    assert torch.isnan(out).all()  # nothing was launched


def test_static_scratch_allocates_nothing_and_serves_in_place_operands_of_any_size():
    """The entry point's promise: no device allocation.  After a warm-up call (the first call on a device looks the
    array's address up), free device memory and torch's own allocation counter are the same before and after a
    call.  A call that has nothing to pack (fp16, [N, K] weight, K % 8 == 0: the tied lm_head's layout) is served
    whatever its size, and the w_is_nk layout with packing (fp32) works too."""
    from gpt_triton_b200 import _lib

    lib = _lib.load()
    g = torch.Generator().manual_seed(12)
    x = torch.randn((4096, 768), generator=g).half().to(DEV)
    wte = (torch.randn((50257, 768), generator=g) * 0.02).half().to(DEV)  # 77 MB: far beyond 32 MiB if it had to be packed
    pitch = 50304
    out = torch.empty((4096, pitch), dtype=torch.float16, device=DEV)
    stream = _lib.stream_ptr(x.device)

    def call():
        return lib.b200_ffn_static_scratch(x.data_ptr(), wte.data_ptr(), None, None, out.data_ptr(), 4096, 50257, 768, pitch, 1, 0, _lib.F16, None, stream)

    assert call() == 0
    torch.cuda.synchronize()
    free0, alloc0 = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated()
    assert call() == 0
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free0 and torch.cuda.memory_allocated() == alloc0
    rows = torch.tensor([0, 77, 4095], device=DEV)
    ref = x[rows].cpu().float() @ wte.cpu().float().T
    assert (out[rows, :50257].cpu().float() - ref).abs().max().item() < 5e-3
    # [N, K] weights in fp32: both operands are packed into the array
    x32 = torch.randn((200, 72), generator=g).to(DEV)
    w_nk = (torch.randn((136, 72), generator=g) * 0.1).to(DEV)
    b = torch.randn(136, generator=g).to(DEV)
    _run_both(lib, _lib, x32, w_nk, b, None, True, True)


def test_static_scratch_rejects_sizes_it_cannot_index():
    from gpt_triton_b200 import _lib

    lib = _lib.load()
    # sizes whose byte counts overflow 64 bits, and sizes beyond what the kernels index: refused as bad arguments
    # before any arithmetic is done on them (no pointer is ever dereferenced: NULL pointers are given)
    for m, n, k in ((1 << 62, 8, 1 << 62), (1 << 33, 8, 8), (8, 1 << 33, 8)):
        assert lib.b200_ffn_static_scratch(None, None, None, None, None, m, n, k, n, 0, 0, _lib.F32, None, None) == 1
    torch.cuda.synchronize()
