"""The N > 1 path on CPU: two gloo ranks decode disjoint streams with no data-path collective
and agree with a single process running all of them."""

import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from megabake_b200.dp import assign_streams, run_data_parallel
from megabake_b200.synth import new_kv_state, rope_tables, synth_ids, synth_weights, tiny_config

STREAMS, STEPS = 5, 6


def _make_step_factory():
    from oracle import decoder_oracle as oracle  # the checker stands in for the device step on CPU

    config = tiny_config()
    weights = synth_weights(config, seed=0, norm_std=0.1)
    tables = rope_tables(config, 16)

    def make_step(stream):
        keys, values, lengths = new_kv_state(config, 2, 16)
        return lambda ids, positions: oracle.decode_step(config, weights, tables, ids, positions, keys, values, lengths)

    first = [synth_ids(2, config.vocab, seed=stream, name="dp") for stream in range(STREAMS)]
    return make_step, first


def _rank_main(rank, world, port, queue):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        make_step, first = _make_step_factory()
        result = run_data_parallel(make_step, first, 0, STEPS)
        assert (result is None) == (rank != 0)
        if rank == 0:
            queue.put([r.tolist() for r in result])
    finally:
        dist.destroy_process_group()


def test_round_robin_partition():
    assert assign_streams(5, 2) == [[0, 2, 4], [1, 3]]
    assert assign_streams(3, 4) == [[0], [1], [2], []]
    assert sorted(s for part in assign_streams(17, 8) for s in part) == list(range(17))


def test_two_gloo_ranks_match_one_process():
    with socket.socket() as probe:
        probe.bind(("127.0.0.1", 0))
        port = probe.getsockname()[1]
    context = mp.get_context("spawn")
    queue = context.Queue()
    workers = [context.Process(target=_rank_main, args=(rank, 2, port, queue)) for rank in range(2)]
    for worker in workers:
        worker.start()
    parallel = queue.get(timeout=240)
    for worker in workers:
        worker.join(timeout=60)
        assert worker.exitcode == 0
    make_step, first = _make_step_factory()
    single = run_data_parallel(make_step, first, 0, STEPS, rank=0, world=1)
    assert parallel == [r.tolist() for r in single]
