"""Benchmark of the GPT-2 forward hot path: tokens/s of a GPT-2 124M forward (tied lm_head
included) on ONE synthetic 512 x 300 fp16 batch, split by rows over the GPUs of one node (strong scaling:
rank r of N runs rows [r * 512 / N, (r + 1) * 512 / N) on a full replica of the weights).

    python bench.py [--gpus N] [--steps K] [--warmup W]          # this engine (sm_100a kernels)
    python bench.py --impl reference [...]                       # the plain PyTorch forward on the host cores

One "step" is one forward pass (embedding -> 12 blocks -> final LayerNorm -> lm_head logits) over
the batch.  Rank 0 prints one JSON line.  `value` is device-timed with the ids resident in HBM;
`e2e` is the same pass driven from pinned host ids with the argmax ids (all-gathered over NCCL when N > 1)
read back each step.  Weights are random-init N(0, 0.02) (output projections scaled by 1/sqrt(24)), ids
uniform: no dataset or checkpoint is involved.
"""

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GPT2_SMALL = dict(vocab_size=50257, block_size=1024, n_layer=12, n_head=12, n_embd=768, dropout=0.1)
BATCH, SEQ = 512, 300
# the larger, attention-heavier configurations (not the headline; `--model` times them on one GPU)
OTHER_MODELS = {
    "355m": (dict(vocab_size=50257, block_size=1024, n_layer=24, n_head=16, n_embd=1024, dropout=0.1), 256, 1024, torch.bfloat16),
    "1.5b": (dict(vocab_size=50257, block_size=1024, n_layer=48, n_head=25, n_embd=1600, dropout=0.1), 128, 1024, torch.bfloat16),
}
CPU_SAMPLE_BATCH = 32  # sequences per CPU-baseline step (the full batch would take minutes per step)
# One-pass ncu capture (DRAM bytes read + written, duration) of the full-size c_fc launch; bench.py only reads it.
TRAFFIC_FILE = os.path.join("profiles", "gemm_tn_kernel_c_fc_153600x3072x768_fp16_dram.md")
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


def make_state_dict(dtype):
    from oracle import gpt2_oracle as orc  # seeded weight generator only (shared with the tests)

    cfg = orc.OracleConfig(**GPT2_SMALL)
    sd = orc.seeded_state_dict(cfg, seed=0, scale_residual_proj=True)
    return cfg, {k: v.to(dtype) for k, v in sd.items()}


def measured_traffic():
    """(bytes per launch, source) of the dominant kernel's launch from the tracked one-pass ncu summary: the line
    `traffic_bytes_per_launch: <read> + <write>` of TRAFFIC_FILE; (None, reason) if the summary is not there."""
    path = os.path.join(ROOT, TRAFFIC_FILE)
    try:
        with open(path) as f:
            for line in f:
                if line.startswith("traffic_bytes_per_launch:"):
                    read, write = (float(t) for t in line.split(":", 1)[1].split("+"))
                    return read + write, TRAFFIC_FILE
    except (OSError, ValueError):
        pass
    return None, "no ncu summary of the full-size launch in this tree"


def make_ids(batch, seed):
    return torch.randint(0, GPT2_SMALL["vocab_size"], (batch, SEQ), generator=torch.Generator().manual_seed(seed))


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi.  It is started before the warm-up passes
    (nvidia-smi needs a second or more to come up on a multi-GPU box) and keeps only the samples that arrived
    between mark_begin() and mark_end(), the timed region; if the region was too short to catch one, the samples of
    the warm-up passes (same kernels, same load) stand in and the record says so."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.rows, self.proc, self.thread = [], None, None
        self.t_begin = self.t_end = None
        self.cmd = ["nvidia-smi", f"--id={gpu_index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"]

    def start(self):
        try:
            self.proc = subprocess.Popen(self.cmd, stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return

        def pump():
            for line in self.proc.stdout:
                self.rows.append((time.monotonic(), line))

        self.thread = threading.Thread(target=pump, daemon=True)
        self.thread.start()

    def mark_begin(self):
        self.t_begin = time.monotonic()

    def mark_end(self):
        self.t_end = time.monotonic()

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"], "samples": 0}
        time.sleep(0.12)  # one more sampling period: a sample describes the 100 ms before it
        self.proc.terminate()
        self.thread.join(timeout=5)
        inside = [line for t, line in self.rows if self.t_begin is not None and self.t_begin <= t <= (self.t_end or t) + 0.12]
        window = "timed region"
        if not inside:
            inside = [line for _, line in self.rows]
            window = "warm-up passes and timed region (the timed region was shorter than one sampling period)"
        sm, mx, reasons = [], [], set()
        for line in inside:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                clock, top = float(parts[0]), float(parts[1])
            except ValueError:
                continue
            sm.append(clock)
            mx.append(top)
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        busy = [c for c in sm if c > 0]
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(busy), "window": window}


# ----------------------------------------------------------------------------- CPU arm
def use_all_host_threads():
    """Every host core this process may use: torchrun exports OMP_NUM_THREADS=1 to its workers, which would leave the
    CPU arm on a single thread."""
    try:
        torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    except (AttributeError, OSError):
        torch.set_num_threads(max(1, os.cpu_count() or 1))


def cpu_forward_tokens_per_s(steps, warmup):
    """The oracle (CPU restatement of the reference's forward + tied lm_head, all host threads)
    on CPU_SAMPLE_BATCH x 300 tokens of the benchmark batch per step."""
    from oracle import gpt2_oracle as orc

    use_all_host_threads()
    cfg, sd = make_state_dict(torch.float16)
    ids = make_ids(BATCH, 0)[:CPU_SAMPLE_BATCH]
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        logits = orc.lm_head(sd, orc.gpt_forward(sd, cfg, ids))
        _ = logits.argmax(-1)
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    mean = sum(times) / len(times)
    return ids.numel() / mean, mean, torch.get_num_threads()


def cpu_hf_forward_tokens_per_s(steps, warmup):
    """transformers' GPT2Model built from a config (no download) with the benchmark's weights, fp32, plus hidden @ wte.T:
    the plain PyTorch forward the reference compares itself with (bench.py:26-52 of the reference), on the same
    CPU_SAMPLE_BATCH x 300 tokens and host threads as the oracle arm.  None when transformers is not importable."""
    try:
        from transformers import GPT2Config, GPT2Model
    except Exception:
        return None
    use_all_host_threads()
    kw = GPT2_SMALL
    hf_cfg = GPT2Config(vocab_size=kw["vocab_size"], n_positions=kw["block_size"], n_embd=kw["n_embd"], n_layer=kw["n_layer"],
                        n_head=kw["n_head"], resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0)
    hf = GPT2Model(hf_cfg).eval()
    _, sd = make_state_dict(torch.float32)
    top = {"wte.weight": "wte_weight", "wpe.weight": "wpe_weight", "ln_f.weight": "layer_norm_weight", "ln_f.bias": "layer_norm_bias"}
    blk = [("ln_1", 0, "layer_norm"), ("attn.c_attn", 0, "c_attn"), ("attn.c_proj", 0, "c_proj"), ("ln_2", 1, "layer_norm"),
           ("mlp.c_fc", 1, "ffn1"), ("mlp.c_proj", 1, "ffn2")]
    hf_sd = {k: sd[v] for k, v in top.items()}
    for i in range(kw["n_layer"]):
        for stem, slot, ours in blk:
            for kind in ("weight", "bias"):
                hf_sd[f"h.{i}.{stem}.{kind}"] = sd[f"blocks.{i}.{slot}.{ours}_{kind}"]
    missing, unexpected = hf.load_state_dict(hf_sd, strict=False)
    assert not unexpected and all(".attn.bias" in m or ".attn.masked_bias" in m for m in missing), (missing, unexpected)
    ids = make_ids(BATCH, 0)[:CPU_SAMPLE_BATCH]
    times = []
    with torch.no_grad():
        for i in range(warmup + steps):
            t0 = time.perf_counter()
            logits = hf(ids).last_hidden_state @ hf.wte.weight.T
            _ = logits.argmax(-1)
            if i >= warmup:
                times.append(time.perf_counter() - t0)
    mean = sum(times) / len(times)
    return ids.numel() / mean, mean, torch.get_num_threads()


def cpu_baseline_record(steps, warmup, port_steps):
    """The CPU figures of this workload on the host cores: the plain PyTorch forward the reference measures itself
    against (transformers' GPT2Model fp32 + hidden @ wte.T; bench.py:26-52 of the reference) as the value, and the
    rounding-faithful oracle port of the reference's kernels (slower: it emulates fp16 operand rounding) next to it."""
    sample = f"{CPU_SAMPLE_BATCH} x {SEQ} tokens of the 512 x 300 batch per step"
    hf = cpu_hf_forward_tokens_per_s(steps=steps, warmup=warmup)
    port = cpu_forward_tokens_per_s(steps=port_steps, warmup=1) if port_steps > 0 else None
    if hf is None:  # transformers missing: the port is all there is
        port = port or cpu_forward_tokens_per_s(steps=steps, warmup=warmup)
        return {"value": port[0], "unit": "tokens/s", "cores": port[2], "kind": "port", "mean_s_per_step": port[1],
                "sample": sample + ", oracle port (fp16-rounded operands, fp32 accumulate)"}
    rec = {"value": hf[0], "unit": "tokens/s", "cores": hf[2], "kind": "port", "mean_s_per_step": hf[1],
           "sample": sample + f", fp32, {steps} timed passes after {warmup} warm-up",
           "what": "transformers GPT2Model built from a config with the benchmark's weights, fp32, + hidden @ wte.T + argmax: the plain "
                   "PyTorch forward the reference benchmarks itself against"}
    if port is not None:
        rec["oracle_port"] = {"value": port[0], "unit": "tokens/s", "cores": port[2],
                              "what": "CPU restatement of the reference's kernels with their rounding points, same sample"}
    return rec


def run_reference_arm(args, rank):
    if rank != 0:
        return
    cpu = cpu_baseline_record(steps=args.steps, warmup=args.warmup, port_steps=1)
    tps = cpu["value"]
    print(json.dumps({
        "impl": "reference", "metric": "gpt2_124m_fwd_tokens_per_s", "value": tps, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": cpu["mean_s_per_step"] * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
        "config": {"workload": "GPT-2 124M forward + tied lm_head, 512 x 300 (CPU arm: bounded sample per step)",
                   "batch": CPU_SAMPLE_BATCH, "seq_len": SEQ},
        "cpu_baseline": cpu,
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


# ----------------------------------------------------------------------------- GPU arm
def run_gpu_arm(args, rank, world, local_rank):
    import torch.distributed as dist

    from gpt_triton_b200 import _lib
    from gpt_triton_b200 import kernels as K
    from gpt_triton_b200.gpt import FusedGPT, GPTConfig, GraphedForward, executed_fwd_flops
    from gpt_triton_b200.sharding import gather_equal_rows, gather_rows, shard_bounds

    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    lib = _lib.load()
    peaks, peak_kind = load_peaks()

    _, sd = make_state_dict(torch.float16)
    gcfg = GPTConfig(**GPT2_SMALL)
    model = FusedGPT(gcfg)
    model.load_state_dict(sd)
    model = model.half().to(dev).eval()
    del sd

    # ONE global 512 x 300 batch (the same seeded ids on every rank); rank r runs its contiguous rows of it
    BATCH = args.global_batch
    ids_global = make_ids(512, 0)[:BATCH]
    lo, hi = shard_bounds(BATCH, rank, world)
    local_batch = hi - lo
    ids_host = ids_global[lo:hi].contiguous().pin_memory()
    ids_dev = ids_host.to(dev)
    tokens_per_step = BATCH * SEQ  # whole job

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    status = {"code": 0}

    def check_device_status(where):
        """A kernel that gave up a bounded on-chip wait returns early: its time would be a fast wrong number."""
        code = K.device_status(dev)
        if code:
            status["code"] = code
            raise RuntimeError(f"{where}: a kernel abandoned a bounded wait (device status {code}); the timing is void")

    def timed_replays(graph, steps):
        barrier()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            graph.replay()
        end.record()
        barrier()
        return max_over_ranks(start.elapsed_time(end)) / steps

    # ---- device-resident throughput ("value"): the forward + lm_head captured once in a CUDA graph (the library's
    # GraphedForward) and replayed, so that host-side launch jitter on a shared box cannot starve the GPU
    sampler = ClockSampler(local_rank if "CUDA_VISIBLE_DEVICES" not in os.environ else os.environ["CUDA_VISIBLE_DEVICES"].split(",")[local_rank])
    if rank == 0:
        sampler.start()  # only rank 0's GPU is reported; eight nvidia-smi processes at once slow each other down
    for _ in range(args.warmup):
        model.logits(ids_dev)
    launches_before_capture = lib.b200_launch_count()
    fwd = GraphedForward(model, ids_dev, what="logits", warmup=1)
    torch.cuda.synchronize()
    launches_per_forward = (lib.b200_launch_count() - launches_before_capture) // 2  # one warm-up pass + the captured pass
    for _ in range(max(1, args.warmup)):
        fwd.graph.replay()
    sampler.mark_begin()
    ms_per_step = timed_replays(fwd.graph, args.steps)
    sampler.mark_end()
    clocks = sampler.stop() if rank == 0 else None
    check_device_status("timed forward")
    launches = launches_per_forward * args.steps
    value = tokens_per_step / (ms_per_step * 1e-3)
    del fwd

    # ---- end to end: pinned host ids in, argmax ids (from the lm_head epilogue, all ranks' rows gathered) out, every step
    out_host = torch.empty((BATCH, SEQ), dtype=torch.int64).pin_memory()
    e2e_fwd = GraphedForward(model, ids_dev, what="logits_and_next_ids", warmup=1)
    gathered = torch.empty((BATCH, SEQ), device=dev, dtype=torch.int64) if world > 1 else None
    even = BATCH % world == 0

    def e2e_step():
        nonlocal gathered
        e2e_fwd.static_ids.copy_(ids_host, non_blocking=True)
        e2e_fwd.graph.replay()
        am = e2e_fwd.outputs[1]
        if world > 1:
            # 8 bytes per token cross NVLink: one NCCL all-gather of the ids, straight into the result buffer
            if even:
                gather_equal_rows(am, out=gathered)
            else:
                gathered = gather_rows(am, BATCH)
            out_host.copy_(gathered, non_blocking=True)
        else:
            out_host.copy_(am, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for _ in range(max(1, args.warmup // 2)):
        e2e_step()
    barrier()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        e2e_step()
    end.record()
    barrier()
    e2e_ms = max_over_ranks(start.elapsed_time(end)) / args.steps
    e2e_value = tokens_per_step / (e2e_ms * 1e-3)
    check_device_status("end-to-end steps")
    # every rank holds the whole batch's ids; its own rows are what its own forward produced
    assert torch.equal(out_host[lo:hi], e2e_fwd.outputs[1].cpu()), "gathered ids do not contain this rank's rows"
    ids_checksum = int(out_host.sum().item())
    if world > 1:
        t = torch.tensor([ids_checksum, -ids_checksum], device=dev, dtype=torch.int64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        assert t[0].item() == -t[1].item(), "ranks disagree on the gathered ids"
    del e2e_fwd

    # ---- for information: the same forward with the lm_head reduced to its row argmax inside the GEMM epilogue
    # (FusedGPT.next_ids: the [tokens, vocab] logits are never written); not the headline workload
    ids_fwd = GraphedForward(model, ids_dev, what="next_ids", warmup=1)
    ids_fwd.graph.replay()
    ids_only_ms = timed_replays(ids_fwd.graph, args.steps)
    del ids_fwd

    # ---- for information at N > 1: the replica figure (every rank a whole 512 x 300 batch of its own, no split)
    weak = None
    if world > 1:
        full_ids = make_ids(512, rank)[:BATCH].to(dev)
        wfwd = GraphedForward(model, full_ids, what="logits", warmup=1)
        wfwd.graph.replay()
        weak_ms = timed_replays(wfwd.graph, max(2, args.steps // 2))
        weak = {"value": world * BATCH * SEQ / (weak_ms * 1e-3), "unit": "tokens/s", "ms_per_step": weak_ms,
                "what": "weak scaling: every GPU runs its own 512 x 300 batch (N times the work of the headline)"}
        del wfwd, full_ids

    # ---- roofline of the dominant kernel (the tcgen05 GEMM): CUDA events around every GEMM launch
    # of further forward passes, on the stream the kernels are launched on.  The other operators are
    # bracketed the same way to give the per-step breakdown.
    records = []
    other = {"attention": [], "layernorm": [], "embedding": []}
    orig = {"fused_ffn": K.fused_ffn, "flash_attention_v1": K.flash_attention_v1, "fused_layer_norm": K.fused_layer_norm,
            "fused_embeddings": K.fused_embeddings}

    def timed_ffn(x, weight, *a, **kw):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        z = orig["fused_ffn"](x, weight, *a, **kw)
        e.record()
        m = x.numel() // x.shape[-1]
        records.append((m, weight.N, weight.K, s, e))
        return z

    def timed(kind, name):
        def fn(*a, **kw):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            z = orig[name](*a, **kw)
            e.record()
            other[kind].append((s, e))
            return z
        return fn

    K.fused_ffn = timed_ffn
    K.flash_attention_v1 = timed("attention", "flash_attention_v1")
    K.fused_layer_norm = timed("layernorm", "fused_layer_norm")
    K.fused_embeddings = timed("embedding", "fused_embeddings")
    probe_steps = min(3, args.steps)
    try:
        for _ in range(probe_steps):
            model.logits(ids_dev)
        torch.cuda.synchronize()
    finally:
        for name, fn in orig.items():
            setattr(K, name, fn)
    check_device_status("per-operator probe passes")
    # Per shape, the MEDIAN launch duration (a host stall on a shared box can leave the GPU idle inside one bracket)
    by_shape = {}
    for m, n, k, s, e in records:
        by_shape.setdefault((m, n, k), []).append(s.elapsed_time(e))
    gemm_ms = sum(statistics.median(v) * len(v) for v in by_shape.values())
    gemm_flop = sum(2.0 * m * n * k * len(v) for (m, n, k), v in by_shape.items())
    achieved_tflops = gemm_flop / (gemm_ms * 1e-3) / 1e12
    peak_tflops = float(peaks.get("bf16_tflops_sustained", FALLBACK_PEAKS["bf16_tflops_sustained"]))
    detail = {f"{m}x{n}x{k}": {"launches_per_step": len(v) // probe_steps, "median_ms": statistics.median(v),
                              "tflops": 2.0 * m * n * k / (statistics.median(v) * 1e-3) / 1e12}
              for (m, n, k), v in by_shape.items()}

    breakdown = {"gemm": gemm_ms / probe_steps}
    for kind, evs in other.items():
        times = [s.elapsed_time(e) for s, e in evs]
        breakdown[kind] = statistics.median(times) * len(times) / probe_steps
    breakdown["unattributed"] = ms_per_step - sum(breakdown.values())

    flops = executed_fwd_flops(gcfg, local_batch, SEQ)  # per GPU
    per_gpu_flops_s = flops / (ms_per_step * 1e-3)

    cpu = None
    if rank == 0 and world == 1 and not args.skip_cpu_baseline:
        cpu = cpu_baseline_record(steps=2, warmup=1, port_steps=1)

    if rank == 0:
        traffic, traffic_source = measured_traffic()
        sm_mhz = clocks.get("sm_mhz") if clocks else None
        print(json.dumps({
            "metric": "gpt2_124m_fwd_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "fp16", "data": "synthetic",
            "config": {"workload": f"GPT-2 124M forward + tied lm_head (logits written), ONE {BATCH} x 300 batch split by rows over the GPUs, "
                                   "fp16 storage, fp32 accumulate",
                       "global_batch": BATCH, "batch_per_gpu": local_batch, "seq_len": SEQ,
                       "parallelism": f"batch rows sharded x{world}, full weight replica per GPU",
                       "layer_norm": "folded into c_attn / c_fc (statistics from the producing kernel); final LayerNorm is a kernel",
                       "l2": "no flush: each step streams several GB of activations and logits per GPU, far beyond the 126 MB L2",
                       "flop_per_step_per_gpu": flops},
            "breakdown_ms_per_step": breakdown,
            "ms_per_step_x_sm_mhz": ms_per_step * sm_mhz if sm_mhz else None,
            "mfu": {"of_spec_2250": per_gpu_flops_s / 2250e12, f"of_{peak_kind}_sustained": per_gpu_flops_s / (peak_tflops * 1e12)},
            "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": e2e_ms, "h2d_bytes_per_step": ids_host.numel() * 8,
                    "d2h_bytes_per_step": out_host.numel() * 8,
                    "collective": "NCCL all_gather_into_tensor of the argmax ids (8 B/token)" if world > 1 else None,
                    "ids_checksum": ids_checksum},
            "next_ids_only": {"value": tokens_per_step / (ids_only_ms * 1e-3), "unit": "tokens/s", "ms_per_step": ids_only_ms,
                              "note": "same forward, greedy ids out of the lm_head epilogue, logits not written; informational"},
            "weak_per_gpu": weak,
            "device_status": status["code"],
            "gpu_launches": int(launches), "launch_mode": f"CUDA graph replay, {launches_per_forward} library kernels per forward, "
                                                          f"programmatic dependent launch {'on' if os.environ.get('B200GPT_PDL', '0') == '1' else 'off'}",
            "roofline": {"kernel": "gemm_tn_kernel (tcgen05, all GEMM shapes of the forward)", "bound": "tensor",
                         "achieved": achieved_tflops, "peak": peak_tflops, "unit": "TFLOP/s", "frac": achieved_tflops / peak_tflops,
                         "peak_source": f"{peak_kind}: cuBLAS bf16 sustained",
                         "note": "the times of the LayerNorm-aware GEMMs include their share of the folded LayerNorms (statistics in the epilogue, "
                                 "merge kernel, extension k-block); measured in eager passes after the timed loops",
                         # the whole replayed step (every kernel, tensor-core flop only) against the same peak
                         "whole_step": {"achieved": per_gpu_flops_s / 1e12, "frac": per_gpu_flops_s / (peak_tflops * 1e12)},
                         # DRAM bytes of one full-size c_fc launch (153600 x 3072 x 768) as ncu counted them
                         "traffic": traffic, "traffic_source": traffic_source,
                         "traffic_algorithmic": 2.0 * (153600 * 768 + 768 * 3072 + 153600 * 3072),
                         "per_shape": detail},
            "cpu_baseline": cpu,
            "clocks": clocks,
        }))


# ----------------------------------------------------------------------------- standalone kernel sweep
def run_sweep(args):
    """Single-kernel timings at the kernel-sweep shapes (fp16, seed 0): GEMM + bias + GELU with
    M=153600, K=768, N=3072; the tied lm_head (M=153600, K=768, N=50257: logits, logits + row argmax, row argmax
    without logits); LayerNorm and embedding on 153600 x 768; causal attention with B=512, H=12, D=64,
    S in {300, 1024, 2048}.  --rows / --batch shrink the problem (for profiler captures).
    One JSON line per kernel; not the headline metric."""
    from gpt_triton_b200 import kernels as K

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peaks, peak_kind = load_peaks()
    g = torch.Generator().manual_seed(0)
    M = args.rows or BATCH * SEQ
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # larger than the 126 MB L2

    def timed(fn):
        for _ in range(args.warmup):
            fn()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        total = 0.0
        for _ in range(args.steps):
            flush.zero_()
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            total += s.elapsed_time(e)
        return total / args.steps

    def report(name, ms, bound, work, unit_peak, extra):
        achieved = work / (ms * 1e-3) / (1e12 if bound == "tensor" else 1e9)
        print(json.dumps({"kernel": name, "ms": ms, "bound": bound, "achieved": achieved, "peak": unit_peak,
                          "unit": "TFLOP/s" if bound == "tensor" else "GB/s", "frac": achieved / unit_peak,
                          "peak_source": peak_kind, "l2": "flushed between timed launches", **extra}), flush=True)

    which = args.sweep
    if which in ("gemm", "all"):
        x = torch.randn((M, 768), generator=g).half().to(dev)
        w = (torch.randn((768, 3072), generator=g) * 0.02).half().to(dev)
        b = torch.randn(3072, generator=g).half().to(dev)
        pw = K.pack_weight(w)
        out = torch.empty((M, 3072), device=dev, dtype=torch.float16)
        ms = timed(lambda: K.fused_ffn(x, pw, bias=b, add_gelu=True, out=out))
        report("gemm_bias_gelu", ms, "tensor", 2.0 * M * 768 * 3072, float(peaks["bf16_tflops"]), {"M": M, "K": 768, "N": 3072})
        del x, out
    if which in ("gemm_ln", "all"):
        # the same shape as the forward runs it: LayerNorm folded in (raw rows + their statistics), bias + GELU
        x = torch.randn((M, 768), generator=g).half().to(dev)
        w = (torch.randn((768, 3072), generator=g) * 0.02).half().to(dev)
        b = torch.randn(3072, generator=g).half().to(dev)
        gamma = (1 + 0.1 * torch.randn(768, generator=g)).half().to(dev)
        beta = (0.1 * torch.randn(768, generator=g)).half().to(dev)
        fw = K.fold_layer_norm(w, gamma, beta, b)
        mom = K.row_stats(x)
        out = torch.empty((M, 3072), device=dev, dtype=torch.float16)
        ms = timed(lambda: K.fused_ffn(x, fw, add_gelu=True, ln_stats=mom, out=out))
        report("gemm_layernorm_bias_gelu", ms, "tensor", 2.0 * M * 768 * 3072, float(peaks["bf16_tflops"]), {"M": M, "K": 768, "N": 3072})
        del x, out, mom
    if which in ("gemm_res", "all"):
        # attention c_proj as the forward runs it: bias + residual, row statistics of the output emitted
        x = torch.randn((M, 768), generator=g).half().to(dev)
        w = (torch.randn((768, 768), generator=g) * 0.02).half().to(dev)
        b = torch.randn(768, generator=g).half().to(dev)
        r = torch.randn((M, 768), generator=g).half().to(dev)
        pw = K.pack_weight(w)
        out = torch.empty((M, 768), device=dev, dtype=torch.float16)
        for name, fn in (("gemm_bias_residual", lambda: K.fused_ffn(x, pw, bias=b, residual=r, out=out)),
                         ("gemm_bias_residual_row_stats", lambda: K.fused_ffn(x, pw, bias=b, residual=r, out=out, return_row_stats=True))):
            ms = timed(fn)
            report(name, ms, "tensor", 2.0 * M * 768 * 768, float(peaks["bf16_tflops"]),
                   {"M": M, "K": 768, "N": 768, "hbm_gbs": 3.0 * M * 768 * 2 / (ms * 1e-3) / 1e9})
        del x, out, r
    if which in ("lm_head", "all"):
        x = torch.randn((M, 768), generator=g).half().to(dev)
        wte = (torch.randn((50257, 768), generator=g) * 0.02).half().to(dev)
        pw = K.pack_weight(wte, weight_is_nk=True)
        pitch = (50257 + 63) // 64 * 64
        buf = torch.empty((M, pitch), device=dev, dtype=torch.float16)
        for name, fn in (("lm_head_logits", lambda: K.fused_ffn(x, pw, out=buf[:, :50257])),
                         ("lm_head_logits_argmax", lambda: K.fused_ffn(x, pw, out=buf[:, :50257], return_argmax=True)),
                         ("lm_head_argmax_only", lambda: K.ffn_row_statistics(x, pw, want_lse=False))):
            report(name, timed(fn), "tensor", 2.0 * M * 768 * 50257, float(peaks["bf16_tflops"]), {"M": M, "K": 768, "N": 50257})
        del x, buf, wte, pw
    if which in ("layernorm", "all"):
        x = torch.randn((M, 768), generator=g).half().to(dev)
        w, b = torch.ones(768, device=dev).half(), torch.zeros(768, device=dev).half()
        ms = timed(lambda: K.fused_layer_norm(x, w, b))
        report("layernorm", ms, "hbm", 2.0 * M * 768 * 2, float(peaks["hbm_gbs"]), {"M": M, "H": 768})
    if which in ("embedding", "all"):
        ids = torch.randint(0, 50257, (M // SEQ, SEQ), generator=g).to(dev)
        wte = (torch.randn((50257, 768), generator=g) * 0.02).half().to(dev)
        wpe = (torch.randn((1024, 768), generator=g) * 0.02).half().to(dev)
        ms = timed(lambda: K.fused_embeddings(ids, wte, wpe))
        report("embedding", ms, "hbm", 2.0 * ids.numel() * 768 * 2, float(peaks["hbm_gbs"]), {"tokens": ids.numel(), "H": 768})
    if which in ("attention", "all"):
        for S in (300, 1024, 2048):
            B = args.batch or BATCH
            qkv = (torch.randn((B, S, 3 * 768), generator=g) / 8).half().to(dev)
            q, k, v = (t.view(B, S, 12, 64).transpose(1, 2) for t in qkv.split(768, dim=2))
            ms = timed(lambda: K.flash_attention_v1(q, k, v, merged_heads=True))
            report(f"attention_S{S}", ms, "tensor", 4.0 * B * 12 * 64 * S * (S + 1) / 2, float(peaks["bf16_tflops"]),
                   {"B": B, "H": 12, "D": 64, "S": S, "hbm_gbs": 4.0 * B * S * 768 * 2 / (ms * 1e-3) / 1e9})
            del qkv, q, k, v


def kernel_trace(replay):
    """Kernel start/end records (torch.profiler's CUPTI activity records: no counters, nothing is serialised) of one
    call of `replay`, summed per kernel name, with the idle time between consecutive kernels."""
    from torch.profiler import ProfilerActivity, profile

    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        replay()
        torch.cuda.synchronize()
    recs = sorted(((ev.time_range.start, ev.time_range.end, ev.name) for ev in prof.events()
                   if ev.device_type == torch.autograd.DeviceType.CUDA and ev.time_range.end > ev.time_range.start), key=lambda r: r[0])
    span = recs[-1][1] - recs[0][0]
    busy = sum(r[1] - r[0] for r in recs)
    gaps = [(b[0] - a[1], a[2][:60], b[2][:60]) for a, b in zip(recs, recs[1:])]
    by_name = {}
    for st, en, name in recs:
        key = name.split("(")[0][:90]
        n, t = by_name.get(key, (0, 0.0))
        by_name[key] = (n + 1, t + (en - st))
    return {
        "kernels": len(recs), "span_ms": span / 1e3, "sum_of_kernel_durations_ms": busy / 1e3,
        "idle_between_kernels_ms": sum(g[0] for g in gaps if g[0] > 0) / 1e3, "overlap_ms": -sum(g[0] for g in gaps if g[0] < 0) / 1e3,
        "median_gap_us": statistics.median(g[0] for g in gaps),
        "per_kernel": {k: {"launches": n, "total_ms": t / 1e3} for k, (n, t) in sorted(by_name.items(), key=lambda kv: -kv[1][1])},
        "largest_gaps_us": [{"gap_us": g[0], "after": g[1], "before": g[2]} for g in sorted(gaps, key=lambda g: -g[0])[:5]],
    }


def run_gap_table(args):
    """Where one replayed forward spends its time between kernels: kernel start/end records of ONE CUDA-graph replay
    of the headline forward (torch.profiler's CUPTI activity records: no counters, no kernel is serialised or
    replayed), summed per kernel name, with the idle time between consecutive kernels (negative when programmatic
    dependent launch lets a kernel's set-up start under its predecessor's tail).  A diagnosis, not a benchmark value."""
    from gpt_triton_b200.gpt import FusedGPT, GPTConfig, GraphedForward

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    _, sd = make_state_dict(torch.float16)
    model = FusedGPT(GPTConfig(**GPT2_SMALL))
    model.load_state_dict(sd)
    model = model.half().to(dev).eval()
    batch = args.global_batch
    ids = make_ids(BATCH, 0)[:batch].to(dev)
    fwd = GraphedForward(model, ids, what="logits", warmup=3)
    for _ in range(5):
        fwd.graph.replay()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(10):
        fwd.graph.replay()
    e.record()
    torch.cuda.synchronize()
    plain_ms = s.elapsed_time(e) / 10
    rec = kernel_trace(fwd.graph.replay)
    rec.update({"what": "one CUDA-graph replay of the forward + lm_head under CUPTI activity tracing", "batch": batch, "seq_len": SEQ,
                "replay_ms_without_profiler": plain_ms})
    print(json.dumps(rec))


def run_other_model(args):
    """Forward + lm_head throughput of GPT-2 medium / XL (bf16, seq 1024) on one GPU: weights N(0, 0.02) drawn on
    the device, uniform ids.  Extra figure for the record, not the headline metric."""
    from gpt_triton_b200.gpt import FusedGPT, GPTConfig, executed_fwd_flops

    kw, batch, seq, dtype = OTHER_MODELS[args.model]
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    torch.manual_seed(0)
    with torch.device(dev):
        model = FusedGPT(GPTConfig(**kw))
    with torch.no_grad():
        for name, prm in model.named_parameters():
            if prm.dim() == 2:
                prm.normal_(0.0, 0.02)
            elif name.endswith("layer_norm_weight"):
                prm.fill_(1.0)
            else:
                prm.zero_()
    model = model.to(dtype).eval()
    ids = torch.randint(0, kw["vocab_size"], (batch, seq), device=dev)
    for _ in range(args.warmup):
        model.logits(ids)
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(args.steps):
        model.logits(ids)
    e.record()
    torch.cuda.synchronize()
    ms = s.elapsed_time(e) / args.steps
    flops = executed_fwd_flops(GPTConfig(**kw), batch, seq)
    print(json.dumps({"model": args.model, "batch": batch, "seq_len": seq, "dtype": str(dtype).replace("torch.", ""), "ms_per_step": ms,
                      "tokens_per_s": batch * seq / (ms * 1e-3), "flop_per_step": flops, "mfu_of_spec_2250": flops / (ms * 1e-3) / 2250e12}))


def run_decode(args):
    """Token-by-token generation of the 124M model (fp16, 512 sequences, 300-token prompts, `--new-tokens` generated
    greedily, one GPU): time of the prompt pass and of the replayed decode steps, and the HBM roofline of a decode
    step.  Extra figure for the record (the reference has no inference loop), not the headline metric.

    Algorithmic bytes of one decode step with n tokens already cached: every weight once (the 12 blocks + the tied
    embedding matrix as lm_head operand + the final LayerNorm) + keys and values of n positions read and of one
    position written per layer and sequence; activations of 512 rows are noise beside them."""
    from gpt_triton_b200 import kernels as K
    from gpt_triton_b200.gpt import FusedGPT, GenerationSession, GPTConfig

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peaks, peak_src = load_peaks()
    cfg, sd = make_state_dict(torch.float16)
    model = FusedGPT(GPTConfig(**GPT2_SMALL))
    model.load_state_dict(sd)
    model = model.to(torch.float16).to(dev).eval()
    B, L0, new = args.global_batch, SEQ, args.new_tokens
    prompt = make_ids(B, 0).to(dev)
    sess = GenerationSession(model, B, capacity=L0 + new - 1, max_new_tokens=new)
    tokens = sess.generate(prompt, new)  # prompt pass, two eager steps, capture, replays
    assert sess.graph is not None
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = max(args.steps, 3)
    # the prompt pass (forward + cache fill + first token), eager launches
    torch.cuda.synchronize()
    s.record()
    for _ in range(reps):
        model._body(prompt, kv_caches=sess.kv)
    e.record()
    torch.cuda.synchronize()
    prefill_ms = s.elapsed_time(e) / reps
    # the decode steps: rewind the device-side position to the end of the prompt (and the id that the first step
    # embeds to the first generated token) and replay the captured step
    def rewind():
        sess.pos.copy_(torch.tensor([L0, L0], dtype=torch.int32))
        sess.feedback.copy_(tokens[:, 0])
        torch.cuda.synchronize()

    rewind()
    lib = K._lib.load()
    n0 = lib.b200_launch_count()
    sess._step()  # one eager step, to count this library's launches
    launches = lib.b200_launch_count() - n0
    step_ms = []
    for _ in range(reps):
        rewind()
        s.record()
        for _ in range(new - 1):
            sess.graph.replay()
        e.record()
        torch.cuda.synchronize()
        step_ms.append(s.elapsed_time(e) / (new - 1))
    assert K.device_status(dev) == 0
    assert torch.equal(sess.tokens[:, :new], tokens), "replayed steps must regenerate the same ids"
    if args.gap_table:  # per-kernel times of ONE replayed decode step (the first after the prompt)
        rewind()
        rec = kernel_trace(sess.graph.replay)
        rec.update({"what": "one CUDA-graph replay of a decode step under CUPTI activity tracing", "batch": B, "cached_positions": L0})
        print(json.dumps(rec))
        return
    ms = sorted(step_ms)[len(step_ms) // 2]
    h, n_layer, V = GPT2_SMALL["n_embd"], GPT2_SMALL["n_layer"], GPT2_SMALL["vocab_size"]
    weight_bytes = 2 * (n_layer * 12 * h * h + V * h)
    mean_cached = L0 + (new - 2) / 2.0  # positions in the cache, averaged over the timed steps
    kv_bytes = n_layer * B * (mean_cached + 1) * 2 * h * 2
    alg = weight_bytes + kv_bytes
    print(json.dumps({
        "metric": "gpt2_124m_decode_tokens_per_s", "value": B / (ms * 1e-3), "unit": "tokens/s", "n_gpus": 1, "ms_per_decode_step": ms,
        "prompt_pass_ms": prefill_ms, "dtype": "fp16", "data": "synthetic",
        "config": {"workload": f"GPT-2 124M greedy generation, {B} sequences, {L0}-token prompts, {new} new tokens, key/value cache, "
                               "one CUDA-graph replay per token", "launches_per_decode_step": int(launches)},
        "roofline": {"bound": "hbm", "achieved": alg / (ms * 1e-3) / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": alg / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"], "peak_source": peak_src, "traffic": None,
                     "algorithmic_bytes_per_step": alg, "weights_bytes": weight_bytes, "kv_cache_bytes": kv_bytes},
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--skip-cpu-baseline", action="store_true")
    ap.add_argument("--sweep", default=None, choices=["gemm", "gemm_ln", "gemm_res", "lm_head", "layernorm", "embedding", "attention", "all"],
                    help="time single kernels at the kernel-sweep shapes instead of the forward")
    ap.add_argument("--rows", type=int, default=0, help="--sweep: rows (tokens) instead of 153600")
    ap.add_argument("--batch", type=int, default=0, help="--sweep attention: batch instead of 512")
    ap.add_argument("--model", default=None, choices=sorted(OTHER_MODELS), help="time a larger GPT-2 instead of the 124M headline")
    ap.add_argument("--global-batch", type=int, default=BATCH,
                    help="sequences in the global batch (default 512, the headline; 64 is what one of 8 GPUs runs)")
    ap.add_argument("--gap-table", action="store_true", help="per-kernel time and idle gaps of one replayed forward (diagnosis)")
    ap.add_argument("--decode", action="store_true", help="time token-by-token generation (key/value cache) instead of the forward")
    ap.add_argument("--new-tokens", type=int, default=64, help="--decode: tokens generated per sequence")
    args = ap.parse_args()
    if args.decode:  # (with --gap-table: the per-kernel trace of one decode step instead of the timing line)
        run_decode(args)
        return
    if args.gap_table:
        run_gap_table(args)
        return
    if args.sweep:
        run_sweep(args)
        return
    if args.model:
        run_other_model(args)
        return
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else max(args.warmup, 1)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference_arm(args, rank)
        return

    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # NCCL announces its version on stdout when the first communicator is built; keep stdout for the JSON line
        sys.stdout.flush()
        saved = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
            t = torch.zeros(1, device=torch.device("cuda", local_rank))
            dist.all_reduce(t)
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved, 1)
            os.close(saved)
    try:
        run_gpu_arm(args, rank, world, local_rank)
    finally:
        if world > 1:
            import torch.distributed as dist

            dist.destroy_process_group()


if __name__ == "__main__":
    main()
