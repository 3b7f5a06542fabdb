"""Data-parallel decode: independent streams spread over one process per GPU.

Decode streams share nothing, so a rank replicates the weights, owns the KV caches of its
streams and runs them without any collective on the data path.  ``torch.distributed`` is used
only to agree on the partition and to collect the generated token ids at the end (control
plane).  The reference runs on one device only (src/megabake/compiler.py:1518-1528); this is
the partition its stream benchmark (benchmarks/full_model.py:463-467) would use per GPU.
"""

from __future__ import annotations

from typing import Callable, Sequence

import torch


def assign_streams(n_streams: int, world: int) -> list[list[int]]:
    """Round-robin partition: stream s runs on rank s % world."""
    if n_streams < 0 or world < 1:
        raise ValueError("n_streams must be >= 0 and world >= 1")
    return [list(range(rank, n_streams, world)) for rank in range(world)]


def greedy_stream(step: Callable[[torch.Tensor, torch.Tensor], torch.Tensor], first_ids: torch.Tensor,
                  start: int, steps: int) -> torch.Tensor:
    """Runs ``steps`` greedy decode steps of one stream.  ``step(ids[B,1], positions[B,1])``
    returns logits ``[B,1,V]`` and advances that stream's own KV state.  Returns ``[B, steps]`` ids."""
    ids = first_ids.view(-1, 1)
    out = []
    for offset in range(steps):
        positions = torch.full_like(ids, start + offset)
        logits = step(ids, positions)
        ids = logits[:, 0].float().argmax(-1).view(-1, 1)
        out.append(ids.view(-1).cpu())
    return torch.stack(out, dim=1) if out else torch.empty((ids.shape[0], 0), dtype=torch.int64)


def run_data_parallel(make_step: Callable[[int], Callable], first_ids: Sequence[torch.Tensor], start: int,
                      steps: int, *, rank: int | None = None, world: int | None = None,
                      on_device: bool = False) -> list[torch.Tensor] | None:
    """Every rank decodes its own streams; rank 0 returns the ids of all streams in stream
    order, the others return None.  ``make_step(stream)`` builds the step callable (and the KV
    state) of one stream on the calling rank's device.  With ``on_device`` the callable is
    ``run(first_ids, start, steps) -> ids [B, steps]`` instead and keeps the whole greedy loop on
    the GPU (``DecoderKernel.decode_steps``): the streams of a rank are then queued back to back
    with no host round trip between steps."""
    import torch.distributed as dist

    distributed = dist.is_available() and dist.is_initialized()
    rank = (dist.get_rank() if distributed else 0) if rank is None else rank
    world = (dist.get_world_size() if distributed else 1) if world is None else world
    mine = assign_streams(len(first_ids), world)[rank]
    if on_device:
        queued = {stream: make_step(stream)(first_ids[stream], start, steps) for stream in mine}
        local = {stream: tokens.cpu() for stream, tokens in queued.items()}  # one synchronisation, at the end
    else:
        local = {stream: greedy_stream(make_step(stream), first_ids[stream], start, steps) for stream in mine}
    if not distributed or world == 1:
        return [local[stream] for stream in range(len(first_ids))]
    gathered: list = [None] * world
    dist.all_gather_object(gathered, local)
    if rank != 0:
        return None
    merged: dict[int, torch.Tensor] = {}
    for part in gathered:
        merged.update(part)
    missing = [stream for stream in range(len(first_ids)) if stream not in merged]
    if missing:
        raise RuntimeError(f"streams {missing} were decoded by no rank")
    return [merged[stream] for stream in range(len(first_ids))]
