"""Tensor-parallel decode: the partition and the reduce order on CPU (threads and two gloo ranks),
the in-kernel all-reduce on one GPU against a stand-in peer (its flags written by the host), a
peer that never arrives (bounded wait -> TIMEOUT), and two real ranks where two GPUs exist."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import assert_parity
from megabake_b200.synth import new_kv_state, rope_tables, synth_ids, synth_weights, tiny_config
from megabake_b200.tp import shard_config, shard_weights

STEPS = 3


def _model():
    config = tiny_config(hidden=256, q_heads=8, kv_heads=4, intermediate=512, vocab=1024, tied=False, layers=3)
    return config, synth_weights(config, seed=12, norm_std=0.1)


def _rank_state(shard, batch, capacity, device="cpu"):
    return new_kv_state(shard, batch, capacity, device)


def _unsharded_logits(config, weights, ids_per_step, batch, capacity):
    from oracle import decoder_oracle as oracle

    tables = rope_tables(config, capacity)
    state = new_kv_state(config, batch, capacity)
    out = []
    with torch.no_grad():
        for step, ids in enumerate(ids_per_step):
            positions = torch.full((batch, 1), step, dtype=torch.int64)
            out.append(oracle.decode_step(config, weights, tables, ids, positions, *state))
    return out


def _ids(config, batch):
    return [synth_ids(batch, config.vocab, seed=20 + step, name="tp").view(batch, 1) for step in range(STEPS)]


def test_shards_partition_the_model():
    config, weights = _model()
    shard = shard_config(config, 4)
    assert (shard.q_heads, shard.kv_heads, shard.intermediate, shard.vocab) == (2, 1, 128, 256)
    parts = [shard_weights(config, weights, rank, 4) for rank in range(4)]
    name = "model.layers.1.self_attn.o_proj.weight"
    assert torch.equal(torch.cat([p[name] for p in parts], dim=1), weights[name])
    name = "model.layers.2.mlp.gate_proj.weight"
    assert torch.equal(torch.cat([p[name] for p in parts], dim=0), weights[name])
    assert torch.equal(torch.cat([p["lm_head.weight"] for p in parts], dim=0), weights["lm_head.weight"])
    assert parts[3]["model.embed_tokens.weight"] is weights["model.embed_tokens.weight"]
    with pytest.raises(ValueError, match="does not divide"):
        shard_config(config, 3)


@pytest.mark.parametrize("size", [2, 4])
def test_sharded_math_matches_the_unsharded_model(size):
    """Partial sums in fp32, added in rank order, rounded once: within the logit tolerance of the
    single-device reference path, step after step, with every rank's cache holding its own heads."""
    from oracle import tp_oracle

    config, weights = _model()
    shard = shard_config(config, size)
    shards = [shard_weights(config, weights, rank, size) for rank in range(size)]
    batch, capacity = 2, 8
    tables = rope_tables(config, capacity)
    states = [_rank_state(shard, batch, capacity) for _ in range(size)]
    expected = _unsharded_logits(config, weights, _ids(config, batch), batch, capacity)
    for step, ids in enumerate(_ids(config, batch)):
        positions = torch.full((batch, 1), step, dtype=torch.int64)
        logits = tp_oracle.group_decode_step(shard, size, shards, tables, ids, positions, states)
        assert_parity(logits, expected[step], f"tp{size} logits at step {step}")
    assert all(int(length) == STEPS for state in states for length in state[2])


def _gloo_rank(rank, world, port, queue):
    from oracle import tp_oracle

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        config, weights = _model()
        shard = shard_config(config, world)
        mine = shard_weights(config, weights, rank, world)
        batch, capacity = 2, 8
        tables = rope_tables(config, capacity)
        state = _rank_state(shard, batch, capacity)

        def allreduce(partial):
            parts = [torch.empty_like(partial) for _ in range(world)]
            dist.all_gather(parts, partial.contiguous())
            total = parts[0].clone()
            for other in parts[1:]:
                total = total + other  # rank order, as the kernel adds them
            return total

        out = []
        with torch.no_grad():
            for step, ids in enumerate(_ids(config, batch)):
                positions = torch.full((batch, 1), step, dtype=torch.int64)
                piece = tp_oracle.rank_decode_step(shard, mine, tables, ids, positions, *state, allreduce)
                parts = [torch.empty_like(piece) for _ in range(world)]
                dist.all_gather(parts, piece.contiguous())
                out.append(torch.cat(parts, dim=-1))
        if rank == 0:
            queue.put([t.float().tolist() for t in out])
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_reduce_in_rank_order():
    from oracle import tp_oracle

    with socket.socket() as probe:
        probe.bind(("127.0.0.1", 0))
        port = probe.getsockname()[1]
    context = mp.get_context("spawn")
    queue = context.Queue()
    workers = [context.Process(target=_gloo_rank, args=(rank, 2, port, queue)) for rank in range(2)]
    for worker in workers:
        worker.start()
    gathered = [torch.tensor(t) for t in queue.get(timeout=240)]
    for worker in workers:
        worker.join(timeout=60)
        assert worker.exitcode == 0
    config, weights = _model()
    shard = shard_config(config, 2)
    shards = [shard_weights(config, weights, rank, 2) for rank in range(2)]
    torch.set_num_threads(1)
    states = [_rank_state(shard, 2, 8) for _ in range(2)]
    tables = rope_tables(config, 8)
    for step, ids in enumerate(_ids(config, 2)):
        positions = torch.full((2, 1), step, dtype=torch.int64)
        threaded = tp_oracle.group_decode_step(shard, 2, shards, tables, ids, positions, states)
        assert torch.equal(gathered[step], threaded.float()), f"step {step}: two processes and two threads disagree"


# --------------------------------------------------------------------------- one GPU
def _gpu_rank0_with_stand_in_peer(wait_ms=None, post_flags=True):
    """Rank 0 of a group of two on one GPU.  The peer's exchange buffer is a second local buffer
    nobody reads; the peer's partial sums in rank 0's own buffer stay zero and its arrival stamps
    are written by the host (or not at all)."""
    from megabake_b200.tp import ExchangeBuffers, TensorParallelDecoder

    device = torch.device("cuda:0")
    config, weights = _model()
    mine = {name: tensor.to(device) for name, tensor in shard_weights(config, weights, 0, 2).items()}
    exchange = ExchangeBuffers.local(1 << 20, 2, device)
    decoder = TensorParallelDecoder(config, mine, rank=0, size=2, max_tokens=4, max_positions=16, device=device,
                                    exchange=exchange)
    if post_flags:  # the stand-in peer "has arrived" at every all-reduce there will ever be
        flags = torch.tensor([0, 0x7FFFFFFF], dtype=torch.int32, device=device)
        own = exchange._keep[0]
        offset = exchange.pointers[0] - own.data_ptr()
        own[offset:offset + 8].copy_(flags.view(torch.uint8))
        torch.cuda.synchronize(device)
    return config, weights, decoder


@pytest.mark.gpu
def test_in_kernel_allreduce_against_a_stand_in_peer():
    """With the peer contributing zeros, rank 0's result is the model made of rank 0's heads, MLP
    columns and vocabulary rows alone: the oracle runs exactly that."""
    from oracle import tp_oracle

    config, weights, decoder = _gpu_rank0_with_stand_in_peer()
    device = decoder.device
    shard = decoder.config
    mine_cpu = shard_weights(config, weights, 0, 2)
    batch, capacity = 3, 16
    tables = rope_tables(config, capacity)
    state = _rank_state(shard, batch, capacity, device)
    ref_state = _rank_state(shard, batch, capacity)
    for step in range(4):
        ids = synth_ids(batch, config.vocab, seed=30 + step, name="tp").view(batch, 1)
        positions = torch.full((batch, 1), step, dtype=torch.int64)
        logits = decoder.decode(ids.to(device), positions.to(device), *state)
        decoder.check()
        with torch.no_grad():
            expected = tp_oracle.rank_decode_step(shard, mine_cpu, tables, ids, positions, *ref_state, lambda partial: partial)
        assert_parity(logits, expected, f"rank 0 logits at step {step}")
    assert_parity(state[0][-1], ref_state[0][-1], "last layer key cache")
    assert all(int(length) == 4 for length in state[2])


@pytest.mark.gpu
def test_a_peer_that_never_arrives_times_out(monkeypatch):
    """Failure detection without a hang: nothing ever writes the peer's arrival stamp, the bounded
    wait (40 ms) runs out, the status names the wait on the peer flag, nothing was published."""
    monkeypatch.setenv("MEGABAKE_WAIT_LIMIT_MS", "40")
    config, weights, decoder = _gpu_rank0_with_stand_in_peer(post_flags=False)
    device = decoder.device
    state = _rank_state(decoder.config, 1, 16, device)
    ids = torch.tensor([[5]], device=device)
    decoder.decode(ids, torch.zeros((1, 1), dtype=torch.int64, device=device), *state)
    result = decoder.status()
    assert result["status"] == "TIMEOUT" and result["where"] == 11 and result["detail"] == 1, result
    assert int(state[2][1]) == 0  # layer 1 was never reached
    assert decoder.status()["status"] == "OK"


# --------------------------------------------------------------------------- two GPUs
def _nccl_rank(rank, world, port, queue):
    from megabake_b200.tp import TensorParallelDecoder

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    device = torch.device("cuda", rank)
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        config, weights = _model()
        mine = {name: tensor.to(device) for name, tensor in shard_weights(config, weights, rank, world).items()}
        decoder = TensorParallelDecoder(config, mine, rank=rank, size=world, max_tokens=4, max_positions=16, device=device)
        batch, capacity = 2, 8
        state = _rank_state(decoder.config, batch, capacity, device)
        out = []
        for step, ids in enumerate(_ids(config, batch)):
            positions = torch.full((batch, 1), step, dtype=torch.int64, device=device)
            out.append(decoder.gather_logits(decoder.decode(ids.to(device), positions, *state)).cpu())
        decoder.check()
        if rank == 0:
            queue.put([t.float().tolist() for t in out])
        dist.barrier()
        decoder.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.gpu
def test_two_gpu_ranks_match_the_sharded_and_the_unsharded_oracle():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from oracle import tp_oracle

    with socket.socket() as probe:
        probe.bind(("127.0.0.1", 0))
        port = probe.getsockname()[1]
    context = mp.get_context("spawn")
    queue = context.Queue()
    workers = [context.Process(target=_nccl_rank, args=(rank, 2, port, queue)) for rank in range(2)]
    for worker in workers:
        worker.start()
    logits = [torch.tensor(t) for t in queue.get(timeout=300)]
    for worker in workers:
        worker.join(timeout=120)
        assert worker.exitcode == 0
    config, weights = _model()
    shard = shard_config(config, 2)
    shards = [shard_weights(config, weights, rank, 2) for rank in range(2)]
    states = [_rank_state(shard, 2, 8) for _ in range(2)]
    tables = rope_tables(config, 8)
    unsharded = _unsharded_logits(config, weights, _ids(config, 2), 2, 8)
    for step, ids in enumerate(_ids(config, 2)):
        positions = torch.full((2, 1), step, dtype=torch.int64)
        sharded = tp_oracle.group_decode_step(shard, 2, shards, tables, ids, positions, states)
        assert_parity(logits[step], sharded.float(), f"two GPUs vs sharded oracle, step {step}")
        assert_parity(logits[step], unsharded[step].float(), f"two GPUs vs unsharded reference path, step {step}")
