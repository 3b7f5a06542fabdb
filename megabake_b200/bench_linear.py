"""Performance anchor of the projection engine (``mk_linear``: tcgen05 + TMA, swapAB):

    python -m megabake_b200.bench_linear

times y = x . W^T for M in {1, 4, 16, 64} tokens on the decoder's projection shapes against
``torch.matmul`` (cuBLAS) and against the algorithm of the reference's only sm_100 kernel
(``mk_baseline_mma_gemm``: the "blackwell_mma" body of src/megabake/bodies/blackwell.py:91-159
restated in CUDA C).  CUDA events around each launch, rotating weight copies larger than L2 so
that every launch streams from HBM; prints one markdown table and one JSON line.
"""

from __future__ import annotations

import ctypes
import json
import statistics

import torch

from . import _native
from .runtime import DecoderKernel
from .synth import synth_normal, synth_weights, tiny_config

SHAPES = [(2048, 2048), (8192, 2048), (2048, 8192), (49152, 2048)]  # (N, K): q/o, gate/up, down, lm_head of the 1.7B shape
TOKENS = [1, 4, 16, 64]


def _median_us(launch, reps: int) -> float:
    events = [torch.cuda.Event(enable_timing=True) for _ in range(reps + 1)]
    for i in range(3):
        launch(i)
    torch.cuda.synchronize()
    events[0].record()
    for i in range(reps):
        launch(i)
        events[i + 1].record()
    torch.cuda.synchronize()
    return statistics.median(events[i].elapsed_time(events[i + 1]) for i in range(reps)) * 1e3


def main() -> None:
    device = torch.device("cuda:0")
    torch.cuda.set_device(device)
    lib = _native.load()
    config = tiny_config()
    kernel = DecoderKernel(config, synth_weights(config, device=device), max_tokens=64, max_positions=16,
                           device=device, engine="tcgen05")
    stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
    rows = []
    for n, k in SHAPES:
        copies = max(2, (160 << 20) // (n * k * 2) + 1)  # rotate through more than the 126 MB L2
        weights = [synth_normal((n, k), seed=c, name=f"w{n}x{k}", std=0.02, device=device) for c in range(copies)]
        for m in TOKENS:
            x = synth_normal((m, k), seed=1, name=f"x{m}x{k}", std=1.0, device=device)
            out = torch.empty((m, n), dtype=torch.bfloat16, device=device)
            expected = (x.float() @ weights[0].float().T).to(torch.bfloat16)
            mine = kernel.linear(x, weights[0])
            lib.mk_baseline_mma_gemm(x.data_ptr(), weights[0].data_ptr(), out.data_ptr(), m, n, k, stream)
            torch.cuda.synchronize()
            kernel.check()
            for name, result in (("mk_linear", mine), ("baseline", out)):
                worst = float((result.float() - expected.float()).abs().max())
                assert worst <= 2e-2 + 1e-2 * float(expected.float().abs().max()), f"{name} {m}x{n}x{k}: off by {worst}"
            reps = 20
            t_mine = _median_us(lambda i: kernel.linear(x, weights[i % copies]), reps)
            t_torch = _median_us(lambda i: torch.matmul(x, weights[i % copies].T), reps)
            t_base = _median_us(lambda i: lib.mk_baseline_mma_gemm(
                x.data_ptr(), weights[i % copies].data_ptr(), out.data_ptr(), m, n, k, stream), reps)
            gbs = n * k * 2 / t_mine / 1e3
            rows.append(dict(tokens=m, n=n, k=k, mk_linear_us=t_mine, torch_matmul_us=t_torch, reference_mma_us=t_base,
                             mk_linear_gbs=gbs))
        del weights
        torch.cuda.empty_cache()
    print("| tokens | N x K | mk_linear us (GB/s) | torch.matmul us | reference mma.sync 16x32 us |")
    print("|---|---|---|---|---|")
    for r in rows:
        print(f"| {r['tokens']} | {r['n']} x {r['k']} | {r['mk_linear_us']:.1f} ({r['mk_linear_gbs']:.0f}) | "
              f"{r['torch_matmul_us']:.1f} | {r['reference_mma_us']:.1f} |")
    print(json.dumps({"linear_anchor": rows}))


if __name__ == "__main__":
    main()
