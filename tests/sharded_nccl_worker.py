"""Worker of tests/test_gpu_multi.py: run as `python -m torch.distributed.run --nproc-per-node N` on N GPUs of one
box.  Every rank builds the same seeded GPT-2 (124M shapes, fp16, 3 layers to keep it quick), runs its slice of one
global batch through `sharding.sharded_forward` over NCCL and checks that the gathered next-token ids are
bit-identical to the single-GPU `FusedGPT.next_ids` of the whole batch, for an evenly and an unevenly divided
batch, through the fused-epilogue ids and through materialised logits; and that a generation (key/value cache)
split the same way returns the single-GPU continuations."""

import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def main():
    from gpt_triton_b200 import kernels as K
    from gpt_triton_b200.gpt import FusedGPT, GPTConfig
    from gpt_triton_b200.sharding import shard_bounds, sharded_forward
    from oracle import gpt2_oracle as orc  # seeded weight generator only

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=dev)
    try:
        kw = dict(vocab_size=50257, block_size=1024, n_layer=3, n_head=12, n_embd=768, dropout=0.1)
        sd = orc.seeded_state_dict(orc.OracleConfig(**kw), seed=0, scale_residual_proj=True)
        model = FusedGPT(GPTConfig(**kw))
        model.load_state_dict(sd)
        model = model.half().to(dev).eval()
        for n_rows in (16, 13):
            ids = torch.randint(0, 50257, (n_rows, 300), generator=torch.Generator().manual_seed(0)).to(dev)
            whole = model.next_ids(ids)  # every rank computes the single-GPU answer for itself
            got = sharded_forward(model.next_ids, ids, gather="argmax", fn_returns="ids")
            assert got.shape == whole.shape and torch.equal(got, whole), f"rank {rank}: fused ids differ ({n_rows} rows)"
            via_logits = sharded_forward(model.logits, ids, gather="argmax")
            lo, hi = shard_bounds(n_rows, rank, world)
            logits = model.logits(ids[lo:hi])
            # torch.argmax may pick another of several equal maxima than the epilogue (lowest column): compare values
            picked = logits.gather(-1, via_logits[lo:hi, :, None])[..., 0]
            assert torch.equal(picked, logits.max(-1).values), f"rank {rank}: logits-path ids are not row maxima"
            assert torch.equal(logits.gather(-1, whole[lo:hi, :, None])[..., 0], picked)
        # generation with the key/value cache, batch split over the ranks: the gathered continuations equal the
        # single-GPU ones (a row's arithmetic does not depend on how many rows share its launch)
        prompts = torch.randint(0, 50257, (10, 40), generator=torch.Generator().manual_seed(1)).to(dev)
        whole = model.generate(prompts, 6)
        got = sharded_forward(lambda x: model.generate(x, 6), prompts, gather="argmax", fn_returns="ids")
        assert got.shape == whole.shape and torch.equal(got, whole), f"rank {rank}: sharded generation differs"
        assert K.device_status() == 0
        dist.barrier()
        if rank == 0:
            print(f"sharded_nccl_worker ok: world {world}")
    finally:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
