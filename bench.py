"""Decode benchmark of the B200 megakernel (one JSON line on stdout).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl megakernel|reference]

Headline (``value``, ``e2e``, ``roofline``): a step is one decode call (one cooperative kernel
launch) for ``--batch`` sequences on the SmolLM-1.7B-shaped decoder with a KV cache of capacity
2048 pre-filled to 1024 positions (seeded synthetic weights and cache contents; every step reads
all 3.4 GB of weights, far more than the 126 MB L2, so no flush is needed between steps).  With
N > 1 (launched by torchrun, one rank per GPU) every GPU runs its own independent stream: data
parallel, no collective on the data path; the barrier and the max-over-ranks time use NCCL.

``value`` is tokens/s with inputs resident on the GPU.  ``e2e`` goes through the public API a
serving loop calls, ``DecoderKernel.decode_steps(..., steps=1)``: every step copies its token id
and position up from pinned host memory, launches, copies the sampled token back down and
synchronises.  ``roofline`` divides the algorithmic bytes of a step by the CUDA-event time of its
launch.  ``cpu_baseline`` times the CPU oracle (the reference's eager decode path, restated in
``oracle/``) on this host's cores over a bounded number of steps.

Further blocks in the same line (skipped with --no-extras):
``c4``       the data-parallel sweep as specified: 8 independent streams of batch 8 per GPU, 256 greedy
             steps from a 512-position prefix, through megabake_b200.dp with the device-side sampler;
``tp``       (N > 1) tensor-parallel decode of the Llama-3-8B shape over the N GPUs, batch 1 and 32,
             capacity 4096 pre-filled to 2048, all-reduce inside the kernel over NVLink peer buffers;
``prefill``  (N = 1) the prompt pass of the headline model at 64 and 512 tokens.
"""

from __future__ import annotations

import argparse
import gc
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

from megabake_b200.synth import CONFIGS, DecoderConfig, new_kv_state, synth_ids, synth_normal, synth_weights  # noqa: E402

FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1400.0
# dram__bytes_read.sum + dram__bytes_write.sum per launch from ncu captures, keyed by
# (config, batch, context); each entry names the summary under profiles/ that records the capture.
NCU_TRAFFIC = {
    # dram__bytes_read.sum + dram__bytes_write.sum per launch.  The multi-pass capture runs the first four layers
    # of the shape (read + write = 1.010 x that launch's algorithmic bytes); the figure below scales the
    # full launch's algorithmic bytes at context 1024 by the same ratio.
    ("smollm-1.7b", 1, 1024): (int(3_625_848_832 * 1.010), "profiles/megakernel_small_decode_smollm-1.7b_first-4-layers_sections.md"),
}


def parse_args():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=200)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="megakernel", choices=["megakernel", "reference"])
    parser.add_argument("--config", default="smollm-1.7b", choices=sorted(CONFIGS))
    parser.add_argument("--batch", type=int, default=1)
    parser.add_argument("--context", type=int, default=1024)
    parser.add_argument("--capacity", type=int, default=2048)
    parser.add_argument("--layers", type=int, default=0,
                        help="keep only the first N layers of the shape (profiler captures of a few hundred MB; never a bench value)")
    parser.add_argument("--cpu-steps", type=int, default=40, help="CPU baseline sample size")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--engine", default="auto", choices=["auto", "tcgen05", "fma"], help="kernel choice for the headline run")
    parser.add_argument("--no-extras", action="store_true", help="headline only: skip the c4 / tp / prefill blocks")
    parser.add_argument("--c4-steps", type=int, default=256)
    parser.add_argument("--tp-steps", type=int, default=128)
    return parser.parse_args()


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            data = json.loads(path.read_text())
            return float(data["hbm_gbs"]), float(data.get("bf16_tflops_sustained", FALLBACK_BF16_TFLOPS)), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, FALLBACK_BF16_TFLOPS, "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    REASONS = {
        0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
        0x80: "hw_power_brake_slowdown",
    }

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index = index
        self.samples: list[int] = []
        self.max_mhz = None
        self.reason_bits = 0
        self.stop_flag = threading.Event()
        self.error = None

    def run(self):
        try:
            import pynvml

            pynvml.nvmlInit()
            handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM)
            while not self.stop_flag.is_set():
                self.samples.append(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM))
                try:
                    self.reason_bits |= pynvml.nvmlDeviceGetCurrentClocksEventReasons(handle)
                except Exception:
                    self.reason_bits |= pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(handle)
                time.sleep(0.01)
        except Exception as error:  # NVML missing: report that instead of clocks
            self.error = repr(error)

    def summary(self) -> dict:
        if self.error or not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "error": self.error or "no samples"}
        reasons = [name for bit, name in self.REASONS.items() if self.reason_bits & bit]
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz, "reasons": reasons,
                "samples": len(self.samples)}


def build_state(config, batch, context, capacity, device):
    """Caches filled with seeded values for `context` positions, lengths set to it."""
    keys, values, lengths = new_kv_state(config, batch, capacity, device)
    for layer in range(config.layers):
        shape = (batch, context, config.kv_heads, config.head_dim)
        keys[layer][:, :context] = synth_normal(shape, seed=0, name=f"k{layer}", std=1.0, device=device)
        values[layer][:, :context] = synth_normal(shape, seed=0, name=f"v{layer}", std=1.0, device=device)
        lengths[layer].fill_(context)
    return keys, values, lengths


def reset_lengths(lengths, context):
    for length in lengths:
        length.fill_(context)


def cpu_baseline(config, weights, state, batch, context, capacity, steps):
    """The oracle's decode step on the host cores, same weights and cache contents."""
    from megabake_b200.synth import rope_tables
    from oracle import decoder_oracle as oracle

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    weights = {name: tensor.cpu() for name, tensor in weights.items()}
    keys = [tensor.cpu() for tensor in state[0]]
    values = [tensor.cpu() for tensor in state[1]]
    lengths = [torch.full((1,), context, dtype=torch.int32) for _ in range(config.layers)]
    tables = rope_tables(config, capacity)
    ids = synth_ids(batch, config.vocab, seed=1, name="bench").view(batch, 1)
    warmup = 3
    times = []
    with torch.no_grad():
        for step in range(warmup + steps):
            positions = torch.full((batch, 1), context + step, dtype=torch.int64)
            started = time.perf_counter()
            logits = oracle.decode_step(config, weights, tables, ids, positions, keys, values, lengths)
            elapsed = time.perf_counter() - started
            if step >= warmup:
                times.append(elapsed)
            ids = logits[:, 0].float().argmax(-1).view(batch, 1)
    median = statistics.median(times)
    return {
        "value": batch / median, "unit": "tokens/s", "cores": cores, "kind": "port",
        "us_per_call": median * 1e6,
        "sample": f"{steps} decode steps (after {warmup} warm-up) of the same workload from context {context}, "
                  f"median; oracle/decoder_oracle.py in eager PyTorch",
    }


class Group:
    """The torchrun group (or a single process): barrier, max over ranks."""

    def __init__(self, device, world):
        self.device, self.world = device, world

    def sync(self):
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            import torch.distributed as dist

            dist.barrier()
            torch.cuda.synchronize(self.device)

    def worst(self, value: float) -> float:
        if self.world == 1:
            return value
        import torch.distributed as dist

        cell = torch.tensor([value], dtype=torch.float64, device=self.device)
        dist.all_reduce(cell, op=dist.ReduceOp.MAX)
        return float(cell.item())


# --------------------------------------------------------------------------- C4: data-parallel sweep
def run_c4(args, config, weights, group: Group, rank: int, peak: float):
    """8 independent streams of batch 8 per GPU, 256 greedy steps each from a 512-position prefix
    (seeded cache contents stand in for the prompt pass), no collective on the data path."""
    from megabake_b200.dp import run_data_parallel
    from megabake_b200.runtime import DecoderKernel

    device = group.device
    streams_per_gpu, batch, prefix, steps = 8, 8, 512, args.c4_steps
    capacity = 1024
    n_streams = streams_per_gpu * group.world
    kernels, states = {}, {}
    first = [synth_ids(batch, config.vocab, seed=100 + s, name="c4") for s in range(n_streams)]
    stop = torch.cuda.Event(enable_timing=True)

    def make_runner(stream):
        kernel = DecoderKernel(config, weights, max_tokens=batch, max_positions=capacity, device=device)
        state = build_state(config, batch, prefix, capacity, device)
        kernels[stream], states[stream] = kernel, state

        def run(first_ids, start, count):
            ids = first_ids.view(batch, 1).to(device)
            positions = torch.full((batch, 1), start, dtype=torch.int64, device=device)
            tokens = kernel.decode_steps(ids, positions, *state, steps=count)
            stop.record()
            return tokens
        return run

    # build every stream's state first, then time only the decode loops
    mine = [s for s in range(n_streams) if s % group.world == rank]
    runners = {s: make_runner(s) for s in mine}
    for s in mine:  # warm-up: a few steps, then rewind
        runners[s](first[s], prefix, 3)
        reset_lengths(states[s][2], prefix)
    group.sync()
    launches_before = sum(k.launch_info()["launches"] for k in kernels.values())
    start = torch.cuda.Event(enable_timing=True)
    start.record()
    tokens = run_data_parallel(lambda s: runners[s], first, prefix, steps, on_device=True)
    group.sync()
    elapsed_ms = group.worst(start.elapsed_time(stop))
    for kernel in kernels.values():
        kernel.check()
    launches = sum(k.launch_info()["launches"] for k in kernels.values()) - launches_before
    per_gpu_bytes = streams_per_gpu * sum(config.decode_bytes(batch, prefix + s) for s in range(steps))
    achieved = per_gpu_bytes / (elapsed_ms / 1e3) / 1e9
    block = {
        "workload": f"{streams_per_gpu} streams x batch {batch} per GPU, {steps} greedy steps from a {prefix}-position prefix "
                    f"(seeded cache contents), device-side sampler, no collective",
        "value": n_streams * batch * steps / (elapsed_ms / 1e3), "unit": "tokens/s", "n_gpus": group.world,
        "ms_total": elapsed_ms, "us_per_stream_step": 1e3 * elapsed_ms / (steps * streams_per_gpu),
        "per_gpu_roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                             "kernel": "mk::megakernel (one launch per step of 8 sequences)"},
        "gpu_launches_per_gpu": launches,
        "tokens_checked": None if tokens is None else int(sum(t.numel() for t in tokens)),
    }
    del kernels, states, runners
    gc.collect()
    torch.cuda.empty_cache()
    return block


# --------------------------------------------------------------------------- C5: tensor parallel
def run_tp(args, group: Group, rank: int, peak: float):
    """Llama-3-8B shape over the N GPUs of the job: heads and MLP columns sharded, all-reduce after
    o_proj and down_proj inside the kernel, lm_head sharded by vocabulary."""
    from megabake_b200.tp import TensorParallelDecoder, shard_config, shard_weights

    device, size = group.device, group.world
    config = CONFIGS["llama3-8b"]
    capacity, context, steps = 4096, 2048, args.tp_steps
    full = synth_weights(config, seed=0, device=device)
    mine = shard_weights(config, full, rank, size)
    embed = full["model.embed_tokens.weight"]
    del full
    gc.collect()
    torch.cuda.empty_cache()
    decoder = TensorParallelDecoder(config, mine, rank=rank, size=size, max_tokens=32, max_positions=capacity, device=device)
    shard = shard_config(config, size)
    out = {"workload": f"llama3-8b-shaped bf16 decode over tp{size}, KV capacity {capacity} pre-filled to {context}, "
                       f"{steps} steps, in-kernel all-reduce (peer stores + stamped flags), vocabulary-sharded lm_head",
           "n_gpus": size}
    for batch in (1, 32):
        state = build_state(shard, batch, context, capacity, device)
        ids = synth_ids(batch, config.vocab, seed=3, name="tp").view(batch, 1).to(device)
        positions = [torch.full((batch, 1), context + s, dtype=torch.int64, device=device) for s in range(steps + 3)]
        for s in range(3):
            decoder.decode(ids, positions[s], *state)
        decoder.check()
        group.sync()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for s in range(steps):
            decoder.decode(ids, positions[3 + s], *state)
        end.record()
        group.sync()
        decoder.check()
        elapsed_ms = group.worst(begin.elapsed_time(end))
        rank_bytes = sum(shard.decode_bytes(batch, context + 3 + s) for s in range(steps))
        achieved = rank_bytes / (elapsed_ms / 1e3) / 1e9
        out[f"batch{batch}"] = {
            "value": batch * steps / (elapsed_ms / 1e3), "unit": "tokens/s", "us_per_step": 1e3 * elapsed_ms / steps,
            "per_gpu_roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                                 "algorithmic_bytes_per_step_per_gpu": rank_bytes // steps, "kernel": "mk::megakernel"},
            "allreduces_per_step": 2 * config.layers, "allreduce_payload_bytes": batch * config.hidden * 4,
        }
        del state
        gc.collect()
        torch.cuda.empty_cache()
    decoder.close()
    del decoder, mine, embed
    gc.collect()
    torch.cuda.empty_cache()
    return out


# --------------------------------------------------------------------------- prefill
def run_prefill(config, weights, device, hbm_peak: float, tensor_peak: float):
    from megabake_b200.runtime import DecoderKernel

    out = {}
    for tokens in (64, 512):
        kernel = DecoderKernel(config, weights, max_tokens=tokens, max_positions=max(tokens, 16), device=device)
        ids = synth_ids(tokens, config.vocab, seed=7, name=f"prompt{tokens}").view(1, tokens).to(device)
        for _ in range(3):
            kernel.prefill(ids)
        kernel.check()
        torch.cuda.synchronize(device)
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 5
        begin.record()
        for _ in range(reps):
            kernel.prefill(ids)
        end.record()
        torch.cuda.synchronize(device)
        kernel.check()
        ms = begin.elapsed_time(end) / reps
        linear = config.streamed_parameters() - config.layers * 2 * config.hidden - config.hidden
        flops = 2.0 * tokens * linear + 2.0 * 2.0 * tokens * tokens * config.q_size * config.layers / 2.0
        weight_bytes = 2 * config.streamed_parameters()
        hbm_ms, tensor_ms = weight_bytes / hbm_peak / 1e6, flops / tensor_peak / 1e9
        bound = "hbm" if hbm_ms >= tensor_ms else "tensor"
        out[f"tokens{tokens}"] = {
            "ms": ms, "tokens_per_s": tokens / (ms / 1e3), "bound": bound,
            "frac": max(hbm_ms, tensor_ms) / ms, "flops": flops, "weight_bytes": weight_bytes,
        }
        kernel.close()
    return out


def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    config = CONFIGS[args.config]
    if args.layers:
        values = config.to_dict()
        values.update(layers=args.layers, name=f"{config.name}-first-{args.layers}-layers")
        config = DecoderConfig(**values)
    workload = (f"{config.name}-shaped bf16 decode, batch {args.batch}, KV capacity {args.capacity} "
                f"pre-filled to {args.context}")
    base = {
        "metric": "decode tokens/s (us/call and roofline fraction alongside)", "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": workload, "parallelism": f"dp{args.gpus}" if args.gpus > 1 else "single",
                   "l2": "inputs larger than L2 (3.4 GB of weights streamed per step)"},
    }

    if args.impl == "reference":
        # The reference's own implementation of this path is eager PyTorch on the host
        # (its compiled kernels target sm_90a only); rank 0 alone times it, on the CPU only.
        if rank != 0:
            return
        weights = synth_weights(config, seed=0, device="cpu")
        state = build_state(config, args.batch, args.context, args.capacity, "cpu")
        steps = max(1, min(args.steps, args.cpu_steps))
        result = cpu_baseline(config, weights, state, args.batch, args.context, args.capacity, steps)
        line = dict(base)
        line.update({
            "impl": "reference", "value": result["value"], "ms_per_step": result["us_per_call"] / 1e3,
            "us_per_call": result["us_per_call"], "steps": steps, "n_gpus": args.gpus,
            "cpu_baseline": result,
            "e2e": {"value": result["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0,
        })
        print(json.dumps(line), flush=True)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the megakernel has no CPU path")
    from megabake_b200.runtime import DecoderKernel

    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=device)
    group = Group(device, world)
    weights = synth_weights(config, seed=0, device=device)
    kernel = DecoderKernel(config, weights, max_tokens=args.batch, max_positions=args.capacity, device=device,
                           engine=args.engine)
    keys, values, lengths = build_state(config, args.batch, args.context, args.capacity, device)
    ids = synth_ids(args.batch, config.vocab, seed=1 + rank, name="bench").view(args.batch, 1).to(device)
    if args.context + args.warmup + args.steps + 1 > args.capacity:
        raise SystemExit("context + steps exceeds the KV capacity")

    # ---- device-resident timing: one CUDA event pair per launch, on the launching stream
    position_list = [torch.full((args.batch, 1), args.context + step, dtype=torch.int64, device=device)
                     for step in range(args.warmup + args.steps)]
    for step in range(args.warmup):
        kernel.decode(ids, position_list[step], keys, values, lengths)
    kernel.check()
    group.sync()
    sampler = ClockSampler(local_rank)
    sampler.start()
    events = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    launches_before = kernel.launch_info()["launches"]
    events[0].record()
    for step in range(args.steps):
        kernel.decode(ids, position_list[args.warmup + step], keys, values, lengths)
        events[step + 1].record()
    group.sync()
    sampler.stop_flag.set()
    total_ms = group.worst(events[0].elapsed_time(events[-1]))
    per_launch_ms = [events[i].elapsed_time(events[i + 1]) for i in range(args.steps)]
    launches = kernel.launch_info()["launches"] - launches_before
    kernel.check()
    sampler.join(timeout=2)
    tokens = args.batch * args.steps * args.gpus
    value = tokens / (total_ms / 1e3)

    # ---- end to end through the public API from pinned host buffers: id and position up,
    # one launch with the device-side sampler, the sampled token down, synchronised every step
    reset_lengths(lengths, args.context)
    host_ids = torch.empty((args.batch, 1), dtype=torch.int64).pin_memory()
    host_ids.copy_(ids.cpu())
    host_pos = torch.empty((args.batch, 1), dtype=torch.int64).pin_memory()
    host_token = torch.empty((args.batch, 1), dtype=torch.int64).pin_memory()
    e2e_steps = args.steps

    def e2e_step(step):
        host_pos.fill_(args.context + step)
        kernel.step_from_host(host_ids, host_pos, keys, values, lengths, host_token)  # up, launch, down, synchronise
        host_ids.copy_(host_token)

    for step in range(args.warmup):
        e2e_step(step)
    group.sync()
    start_event, stop_event = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start_event.record()
    for step in range(e2e_steps):
        e2e_step(args.warmup + step)
    stop_event.record()
    group.sync()
    e2e_ms = group.worst(start_event.elapsed_time(stop_event))
    e2e_value = args.batch * e2e_steps * args.gpus / (e2e_ms / 1e3)
    kernel.check()

    peak, tensor_peak, peak_kind = measured_peaks()
    extras = {}
    if not args.no_extras:
        del keys, values, lengths
        gc.collect()
        torch.cuda.empty_cache()
        for name, runner in (("c4", lambda: run_c4(args, config, weights, group, rank, peak)),
                             ("tp", (lambda: run_tp(args, group, rank, peak)) if world > 1 else None),
                             ("prefill", (lambda: run_prefill(config, weights, device, peak, tensor_peak)) if world == 1 else None)):
            if runner is None:
                continue
            try:
                extras[name] = runner()
            except Exception as error:  # an extra block must never take the headline down
                extras[name] = {"error": f"{type(error).__name__}: {error}"[:400]}
            group.sync()
        keys, values, lengths = build_state(config, args.batch, args.context, args.capacity, device)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    mean_context = args.context + args.warmup + (args.steps - 1) / 2
    bytes_per_launch = config.decode_bytes(args.batch, int(round(mean_context)))
    launch_ms = statistics.mean(per_launch_ms)
    achieved = bytes_per_launch / (launch_ms / 1e3) / 1e9
    traffic, traffic_source = (None, None) if args.layers else NCU_TRAFFIC.get((args.config, args.batch, args.context), (None, None))
    line = dict(base)
    line.update({
        "value": value, "ms_per_step": total_ms / args.steps, "us_per_call": 1e3 * total_ms / args.steps,
        "tokens_per_s_per_gpu": value / args.gpus,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": traffic, "traffic_source": traffic_source, "peak_source": f"of {peak_kind}",
                     "algorithmic_bytes_per_launch": bytes_per_launch,
                     "kernel": ("mk::megakernel_small<%d, %s>" % (args.batch, "true" if args.batch == 1 else "false")
                                if args.batch <= 4 and args.engine != "tcgen05" else "mk::megakernel"),
                     "launch_us": launch_ms * 1e3, "frac_of_8TBps_nominal": achieved / 8000.0},
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": 16 * args.batch,
                "d2h_bytes_per_step": 8 * args.batch, "us_per_call": 1e3 * e2e_ms / e2e_steps,
                "call": "DecoderKernel.step_from_host (mk_decode_step_host): ids and positions copied from pinned host "
                        "memory, one launch with the device-side sampler, the token copied back, stream synchronised, "
                        "every step"},
        "gpu_launches": launches,
        "clocks": sampler.summary(),
    })
    line.update(extras)
    if not args.no_cpu_baseline and args.gpus == 1:
        line["cpu_baseline"] = cpu_baseline(config, weights, (keys, values, lengths), args.batch, args.context,
                                            args.capacity, args.cpu_steps)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
