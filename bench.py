"""Decode benchmark of the B200 megakernel (one JSON line on stdout).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl megakernel|reference]

A step is one decode call (one cooperative kernel launch) for ``--batch``
sequences on the SmolLM-1.7B-shaped decoder with a KV cache of capacity 2048
pre-filled to 1024 positions (seeded synthetic weights and cache contents; every
step reads all 3.4 GB of weights, far more than the 126 MB L2, so no flush is
needed between steps).  With N > 1 (launched by torchrun, one rank per GPU)
every GPU runs its own independent stream: data parallel, no collective on the
data path; the barrier and the max-over-ranks time use NCCL.

``value`` is tokens/s with inputs resident on the GPU; ``e2e`` goes through the
public API from pinned host buffers and back (ids/positions up, logits down,
synchronised every step, as a caller reading the logits would).  ``roofline``
divides the algorithmic bytes of a step by the CUDA-event time of its launch.
``cpu_baseline`` times the CPU oracle (the reference's eager decode path,
restated in ``oracle/``) on this host's cores over a bounded number of steps.
"""

from __future__ import annotations

import argparse
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

from megabake_b200.synth import CONFIGS, new_kv_state, synth_ids, synth_normal, synth_weights  # noqa: E402

FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of one launch, from the ncu capture summarised in
# profiles/megakernel_decode_smollm-1.7b_launch_list.md (mean of the two captured launches).
NCU_TRAFFIC = {("smollm-1.7b", 1, 1024): 3_640_695_296}


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
    parser.add_argument("--cpu-steps", type=int, default=40, help="CPU baseline sample size")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    return parser.parse_args()


def measured_peak():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


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


def cpu_baseline(config, weights_gpu, state_gpu, batch, context, capacity, steps):
    """The oracle's decode step on the host cores, same weights and cache contents."""
    from megabake_b200.synth import rope_tables
    from oracle import decoder_oracle as oracle

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    weights = {name: tensor.cpu() for name, tensor in weights_gpu.items()}
    keys = [tensor.cpu() for tensor in state_gpu[0]]
    values = [tensor.cpu() for tensor in state_gpu[1]]
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


def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    config = CONFIGS[args.config]
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
        # (its compiled kernels target sm_90a only); rank 0 alone times it.
        if rank != 0:
            return
        device = torch.device("cuda:0") if torch.cuda.is_available() else torch.device("cpu")
        weights = synth_weights(config, seed=0, device=device)
        state = build_state(config, args.batch, args.context, args.capacity, device)
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

        dist.init_process_group("nccl", device_id=device)
    weights = synth_weights(config, seed=0, device=device)
    kernel = DecoderKernel(config, weights, max_tokens=args.batch, max_positions=args.capacity, device=device)
    keys, values, lengths = build_state(config, args.batch, args.context, args.capacity, device)
    ids = synth_ids(args.batch, config.vocab, seed=1 + rank, name="bench").view(args.batch, 1).to(device)
    if args.context + args.warmup + args.steps + 1 > args.capacity:
        raise SystemExit("context + steps exceeds the KV capacity")

    def sync_all():
        torch.cuda.synchronize(device)
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize(device)

    # ---- device-resident timing: one CUDA event pair per launch, on the launching stream
    position_list = [torch.full((args.batch, 1), args.context + step, dtype=torch.int64, device=device)
                     for step in range(args.warmup + args.steps)]
    for step in range(args.warmup):
        kernel.decode(ids, position_list[step], keys, values, lengths)
    kernel.check()
    sync_all()
    sampler = ClockSampler(local_rank)
    sampler.start()
    events = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    launches_before = kernel.launch_info()["launches"]
    events[0].record()
    for step in range(args.steps):
        kernel.decode(ids, position_list[args.warmup + step], keys, values, lengths)
        events[step + 1].record()
    sync_all()
    sampler.stop_flag.set()
    total_ms = events[0].elapsed_time(events[-1])
    per_launch_ms = [events[i].elapsed_time(events[i + 1]) for i in range(args.steps)]
    launches = kernel.launch_info()["launches"] - launches_before
    kernel.check()
    sampler.join(timeout=2)
    if world > 1:
        worst = torch.tensor([total_ms], dtype=torch.float64, device=device)
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        total_ms = float(worst.item())
    tokens = args.batch * args.steps * args.gpus
    value = tokens / (total_ms / 1e3)

    # ---- end to end through the public API from pinned host buffers
    reset_lengths(lengths, args.context)
    host_ids = torch.empty((args.batch, 1), dtype=torch.int64).pin_memory()
    host_ids.copy_(ids.cpu())
    host_pos = torch.empty((args.batch, 1), dtype=torch.int64).pin_memory()
    host_logits = torch.empty((args.batch, 1, config.vocab), dtype=torch.bfloat16).pin_memory()
    dev_ids = torch.empty_like(host_ids, device=device)
    dev_pos = torch.empty_like(host_pos, device=device)
    e2e_steps = args.steps

    def e2e_step(step):
        host_pos.fill_(args.context + step)
        dev_ids.copy_(host_ids, non_blocking=True)
        dev_pos.copy_(host_pos, non_blocking=True)
        logits = kernel.decode(dev_ids, dev_pos, keys, values, lengths)
        host_logits.copy_(logits, non_blocking=True)
        torch.cuda.current_stream(device).synchronize()
        host_ids.copy_(host_logits[:, 0].float().argmax(-1).view(args.batch, 1))

    for step in range(args.warmup):
        e2e_step(step)
    sync_all()
    start_event, stop_event = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start_event.record()
    for step in range(e2e_steps):
        e2e_step(args.warmup + step)
    stop_event.record()
    sync_all()
    e2e_ms = start_event.elapsed_time(stop_event)
    if world > 1:
        worst = torch.tensor([e2e_ms], dtype=torch.float64, device=device)
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        e2e_ms = float(worst.item())
    e2e_value = args.batch * e2e_steps * args.gpus / (e2e_ms / 1e3)
    kernel.check()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak, peak_kind = measured_peak()
    mean_context = args.context + args.warmup + (args.steps - 1) / 2
    bytes_per_launch = config.decode_bytes(args.batch, int(round(mean_context)))
    launch_ms = statistics.mean(per_launch_ms)
    achieved = bytes_per_launch / (launch_ms / 1e3) / 1e9
    traffic = NCU_TRAFFIC.get((args.config, args.batch, args.context))
    line = dict(base)
    line.update({
        "value": value, "ms_per_step": total_ms / args.steps, "us_per_call": 1e3 * total_ms / args.steps,
        "tokens_per_s_per_gpu": value / args.gpus,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": traffic, "peak_source": f"of {peak_kind}",
                     "algorithmic_bytes_per_launch": bytes_per_launch,
                     "kernel": ("mk::megakernel_small<%d>" % args.batch if args.batch <= 4 else
                                "mk::megakernel_small<%d> + <%d> (two launches per step)" % ((args.batch + 1) // 2, args.batch // 2)
                                if args.batch <= 8 else "mk::megakernel"),
                     "launch_us": launch_ms * 1e3, "frac_of_8TBps_nominal": achieved / 8000.0},
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": 16 * args.batch,
                "d2h_bytes_per_step": 2 * config.vocab * args.batch, "us_per_call": 1e3 * e2e_ms / e2e_steps},
        "gpu_launches": launches,
        "clocks": sampler.summary(),
    })
    if not args.no_cpu_baseline and args.gpus == 1:
        line["cpu_baseline"] = cpu_baseline(config, weights, (keys, values, lengths), args.batch, args.context,
                                            args.capacity, args.cpu_steps)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
