"""CPU, world_size 2 over gloo: the batch-sharding host logic (no GPU, no CUDA kernels)."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from gpt_triton_b200.sharding import shard_bounds


def test_shard_bounds_cover_exactly_once():
    for n in (0, 1, 5, 8, 511, 512):
        for w in (1, 2, 3, 4, 8):
            spans = [shard_bounds(n, r, w) for r in range(w)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_bounds(4, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _fake_logits(ids):
    # deterministic stand-in for FusedGPT.logits: depends only on the row's own ids
    v = torch.arange(11, dtype=torch.float32)
    return torch.sin(ids[..., None].float() * 0.37 + v)


def _worker(rank, world, port, n_rows, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from gpt_triton_b200.sharding import shard_batch, sharded_forward

        ids = torch.randint(0, 100, (n_rows, 6), generator=torch.Generator().manual_seed(0))
        lo, hi = shard_bounds(n_rows, rank, world)
        assert torch.equal(shard_batch(ids), ids[lo:hi])
        full = _fake_logits(ids)
        got = sharded_forward(_fake_logits, ids, gather="argmax")
        assert torch.equal(got, full.argmax(-1))
        got = sharded_forward(_fake_logits, ids, gather="logits")
        assert torch.equal(got, full)
        got = sharded_forward(_fake_logits, ids, gather="none")
        assert torch.equal(got, full[lo:hi])
        # a callable that already returns ids (the fused lm_head epilogue on a GPU): gathered as they are
        got = sharded_forward(lambda x: _fake_logits(x).argmax(-1), ids, gather="argmax", fn_returns="ids")
        assert torch.equal(got, full.argmax(-1))
        with pytest.raises(ValueError):
            sharded_forward(_fake_logits, ids, gather="logits", fn_returns="ids")
        if n_rows % world == 0:
            from gpt_triton_b200.sharding import gather_equal_rows

            out = torch.empty((n_rows, 6), dtype=ids.dtype)
            assert gather_equal_rows(ids[lo:hi], out=out) is out and torch.equal(out, ids)
            with pytest.raises(ValueError):
                gather_equal_rows(ids[lo:hi], out=torch.empty((n_rows + 1, 6), dtype=ids.dtype))
        open(os.path.join(out_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n_rows", [8, 5])
def test_sharded_forward_world_size_2(tmp_path, n_rows):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, n_rows, str(tmp_path)), nprocs=2, join=True)
    assert sorted(os.listdir(tmp_path)) == ["ok0", "ok1"]
