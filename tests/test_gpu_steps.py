"""GPU tests of what sits around a decode launch: the device-side greedy sampler and the
multi-step entry point, errors that surface on the warm path without a per-step
synchronisation, and a bounded device wait that runs out (TIMEOUT) and leaves the handle usable."""

import ctypes
import os

import pytest
import torch

from conftest import assert_parity, load_golden, record_stat
from megabake_b200 import _native
from megabake_b200.diagnostics import CompilerError
from megabake_b200.synth import DecoderConfig, new_kv_state, synth_ids, synth_weights, tiny_config

pytestmark = pytest.mark.gpu
DEVICE = torch.device("cuda:0")


def make_kernel(config, weights, **kwargs):
    from megabake_b200.runtime import DecoderKernel

    return DecoderKernel(config, weights, device=DEVICE, **kwargs)


def greedy_on_host(kernel, config, ids, start, steps, state):
    """The step-by-step path: one launch per token, argmax of the returned logits on the host side."""
    batch = ids.shape[0]
    tokens = []
    ids = ids.clone()
    for step in range(steps):
        positions = torch.full((batch, 1), start + step, dtype=torch.int64, device=DEVICE)
        logits = kernel.decode(ids, positions, *state)
        ids = logits[:, 0].float().argmax(-1).view(batch, 1)
        tokens.append(ids[:, 0].clone())
    return torch.stack(tokens, dim=1)


@pytest.mark.parametrize("batch,engine", [(1, "auto"), (3, "auto"), (6, "auto"), (9, "auto"), (2, "tcgen05")])
def test_decode_steps_equals_the_step_by_step_path(batch, engine):
    """Row table (1 token), split-K table (3) and the tensor engine (6, 9, forced 2)."""
    config = tiny_config(q_heads=4, kv_heads=2, hidden=256)
    weights = synth_weights(config, seed=4, norm_std=0.1, device=DEVICE)
    kernel = make_kernel(config, weights, max_tokens=batch, max_positions=32, engine=engine)
    first = synth_ids(batch, config.vocab, seed=4).view(batch, 1).to(DEVICE)
    steps = 12
    expected = greedy_on_host(kernel, config, first, 0, steps, new_kv_state(config, batch, 32, DEVICE))
    state = new_kv_state(config, batch, 32, DEVICE)
    ids, positions = first.clone(), torch.zeros((batch, 1), dtype=torch.int64, device=DEVICE)
    tokens, logits = kernel.decode_steps(ids, positions, *state, steps=steps, return_logits=True)
    kernel.check()
    assert torch.equal(tokens, expected)
    assert torch.equal(ids[:, 0], expected[:, -1]) and torch.equal(positions, torch.full_like(positions, steps))
    assert all(int(length) == steps for length in state[2])
    assert torch.equal(logits[:, 0].float().argmax(-1), expected[:, -1])


@pytest.mark.parametrize("name", ["c1", "c2"])
def test_free_running_greedy_decode_of_the_golden_models(name):
    """64 advancing steps fed by the kernel's own tokens (device-side sampler) after the golden
    prompt: identical to the step-by-step path bit for bit, and compared with the reference's
    greedy tokens (first diverging step recorded, as tools/dump_megakernels.py:292-316 reports it)."""
    record = load_golden(f"decode_{name}.pt")
    config = DecoderConfig(**record["config"])
    weights = synth_weights(config, seed=record["seed"], norm_std=record["norm_std"], device=DEVICE)
    capacity, prompt = record["capacity"], record["prompt"].to(DEVICE)
    golden = record["tokens"].to(DEVICE)
    kernel = make_kernel(config, weights, max_tokens=1, max_positions=capacity)

    def prefix(state):
        for position in range(prompt.shape[1] - 1):
            kernel.decode(prompt[:, position:position + 1].contiguous(),
                          torch.full((1, 1), position, dtype=torch.int64, device=DEVICE), *state)

    steps = golden.shape[1] - prompt.shape[1]
    last = prompt.shape[1] - 1
    state_a, state_b = new_kv_state(config, 1, capacity, DEVICE), new_kv_state(config, 1, capacity, DEVICE)
    prefix(state_a)
    expected = greedy_on_host(kernel, config, prompt[:, last:last + 1].contiguous(), last, steps, state_a)
    prefix(state_b)
    ids = prompt[:, last:last + 1].contiguous()
    positions = torch.full((1, 1), last, dtype=torch.int64, device=DEVICE)
    tokens = kernel.decode_steps(ids, positions, *state_b, steps=steps)
    kernel.check()
    assert torch.equal(tokens, expected), "device-side sampler and host argmax disagree"
    same = (tokens[0] == golden[0, prompt.shape[1]:]).long()
    first_divergence = int(same.argmin()) if int(same.min()) == 0 else steps
    record_stat(f"free_running_{name}", steps=steps, first_diverging_step=first_divergence,
                equal_tokens=int(same.sum()))
    assert steps == 64
    for cache_a, cache_b in zip(state_a[0] + state_a[1], state_b[0] + state_b[1]):
        assert torch.equal(cache_a, cache_b)


def test_full_cache_raises_on_the_next_call_and_hands_out_nan():
    config = tiny_config()
    kernel = make_kernel(config, synth_weights(config, device=DEVICE), max_tokens=1, max_positions=8)
    keys, values, lengths = new_kv_state(config, 1, 4, DEVICE)
    ids = torch.tensor([[3]], device=DEVICE)
    for position in range(4):
        logits = kernel.decode(ids, torch.full((1, 1), position, dtype=torch.int64, device=DEVICE), keys, values, lengths)
    assert torch.isfinite(logits.float()).all()
    refused = kernel.decode(ids, torch.full((1, 1), 4, dtype=torch.int64, device=DEVICE), keys, values, lengths)
    torch.cuda.synchronize(DEVICE)
    assert torch.isnan(refused.float()).all() and int(lengths[0]) == 4
    with pytest.raises(CompilerError, match="state-capacity"):
        kernel.decode(ids, torch.full((1, 1), 4, dtype=torch.int64, device=DEVICE), keys, values, lengths)
    for length in lengths:
        length.fill_(2)
    again = kernel.decode(ids, torch.full((1, 1), 2, dtype=torch.int64, device=DEVICE), keys, values, lengths)
    kernel.check()
    assert torch.isfinite(again.float()).all() and int(lengths[0]) == 3


def test_cuda_op_reports_a_full_cache_on_its_next_call():
    query = torch.zeros(1, 1, 2, 64, dtype=torch.bfloat16, device=DEVICE)
    key = torch.zeros(1, 1, 2, 64, dtype=torch.bfloat16, device=DEVICE)
    cache_k = torch.zeros(1, 2, 2, 64, dtype=torch.bfloat16, device=DEVICE)
    cache_v = torch.zeros_like(cache_k)
    length = torch.full((1,), 2, dtype=torch.int32, device=DEVICE)  # already full
    refused = torch.ops.megabake.kv_attention(query, key, key, cache_k, cache_v, length)
    torch.cuda.synchronize(DEVICE)
    assert torch.isnan(refused.float()).all() and int(length) == 2
    with pytest.raises(CompilerError, match="state-capacity"):
        torch.ops.megabake.kv_attention(query, key, key, cache_k, cache_v, length)
    length.zero_()
    ok = torch.ops.megabake.kv_attention(query, key, key, cache_k, cache_v, length)
    torch.cuda.synchronize(DEVICE)
    assert torch.isfinite(ok.float()).all() and int(length) == 1


def test_a_bad_id_refuses_the_whole_step():
    """One out-of-range id among six sequences: nothing is appended, no length moves, the logits are NaN."""
    config = tiny_config(q_heads=4, kv_heads=1, hidden=256)
    kernel = make_kernel(config, synth_weights(config, seed=3, norm_std=0.1, device=DEVICE), max_tokens=6, max_positions=16)
    keys, values, lengths = new_kv_state(config, 6, 16, DEVICE)
    ids = synth_ids(6, config.vocab, seed=3).view(6, 1).to(DEVICE)
    ids[1, 0] = config.vocab  # out of range
    logits = kernel.decode(ids, torch.zeros((6, 1), dtype=torch.int64, device=DEVICE), keys, values, lengths)
    assert kernel.status()["status"] == "BAD_INDEX"
    assert torch.isnan(logits.float()).all() and all(int(length) == 0 for length in lengths)
    assert all(not bool(cache.any()) for cache in keys)


@pytest.mark.parametrize("batch", [1, 3, 9])
def test_a_grid_barrier_that_cannot_be_reached_times_out_and_the_handle_recovers(batch, monkeypatch):
    """Failure detection without a hang: the host skews the barrier count it expects, the kernel's
    bounded wait (40 ms here) runs out, the status word says TIMEOUT, the valid lengths have not
    moved, and after the reset the same handle decodes correctly.  One token count per kernel:
    row table, split-K table, tensor engine."""
    monkeypatch.setenv("MEGABAKE_WAIT_LIMIT_MS", "40")
    config = tiny_config(q_heads=4, kv_heads=2, hidden=256)
    weights = synth_weights(config, seed=6, norm_std=0.1, device=DEVICE)
    kernel = make_kernel(config, weights, max_tokens=batch, max_positions=16)
    reference = make_kernel(config, weights, max_tokens=batch, max_positions=16)
    ids = synth_ids(batch, config.vocab, seed=6).view(batch, 1).to(DEVICE)
    positions = torch.zeros((batch, 1), dtype=torch.int64, device=DEVICE)
    expected = reference.decode(ids, positions, *new_kv_state(config, batch, 16, DEVICE))
    state = new_kv_state(config, batch, 16, DEVICE)
    _native.check("mk_debug_skew_barrier", kernel.lib.mk_debug_skew_barrier(kernel._handle, 1 << 20))
    kernel.decode(ids, positions, *state)
    result = kernel.status()
    assert result["status"] == "TIMEOUT", result
    assert all(int(length) == 0 for length in state[2])
    assert kernel.status()["status"] == "OK"
    logits = kernel.decode(ids, positions, *state)
    kernel.check()
    assert torch.equal(logits, expected) and all(int(length) == 1 for length in state[2])


def test_static_scratch_status_recovers_from_a_refused_launch():
    """The allocation-free attention entry point has no handle: its status word lives in the static
    array and is read and cleared through mk_kv_attention_static_status."""
    lib = _native.load()
    torch.cuda.set_device(DEVICE)
    stream = ctypes.c_void_p(torch.cuda.current_stream(DEVICE).cuda_stream)
    query = torch.zeros(1, 1, 2, 64, dtype=torch.bfloat16, device=DEVICE)
    cache = torch.zeros(1, 2, 2, 64, dtype=torch.bfloat16, device=DEVICE)
    cache_v = torch.zeros_like(cache)
    length = torch.full((1,), 2, dtype=torch.int32, device=DEVICE)
    output = torch.zeros(2, 1, 64, dtype=torch.bfloat16, device=DEVICE)

    def call():
        return lib.mk_kv_attention_static(2, 2, 64, query.data_ptr(), query.data_ptr(), query.data_ptr(), cache.data_ptr(),
                                          cache_v.data_ptr(), length.data_ptr(), 1, 2, output.data_ptr(), 0, stream)

    info = _native.MkStatusInfo()
    assert call() == _native.MK_OK  # refused on the device: the cache is full
    assert lib.mk_kv_attention_static_status(0, stream, ctypes.byref(info)) == _native.MK_ERR_DEVICE_STATUS
    assert _native.STATUS_NAMES[info.status] == "KV_OVERFLOW" and torch.isnan(output.float()).all()
    assert lib.mk_kv_attention_static_status(0, stream, ctypes.byref(info)) == _native.MK_OK
    length.zero_()
    assert call() == _native.MK_OK
    assert lib.mk_kv_attention_static_status(0, stream, ctypes.byref(info)) == _native.MK_OK
    assert int(length) == 1 and torch.isfinite(output.float()).all()


@pytest.mark.parametrize("lengths_now", [[5, 0, 9], [700, 3, 350, 64, 699]])
def test_per_sequence_valid_lengths_match_the_oracle_one_sequence_at_a_time(lengths_now):
    """Sequences of different lengths in one batch (beyond the reference's one-length-per-batch contract):
    every sequence must come out as if it had been decoded alone by the reference path."""
    from megabake_b200.synth import rope_tables, synth_normal
    from oracle import decoder_oracle as oracle

    config = tiny_config(q_heads=8, kv_heads=2, hidden=512, intermediate=1024)
    batch, capacity = len(lengths_now), 768
    weights = synth_weights(config, seed=8, norm_std=0.1, device=DEVICE)
    kernel = make_kernel(config, weights, max_tokens=batch, max_positions=capacity)
    tables = rope_tables(config, capacity, device=DEVICE)
    keys, values, _ = new_kv_state(config, batch, capacity, DEVICE)
    for layer in range(config.layers):
        keys[layer].copy_(synth_normal(tuple(keys[layer].shape), seed=8, name=f"k{layer}", std=0.5, device=DEVICE))
        values[layer].copy_(synth_normal(tuple(values[layer].shape), seed=8, name=f"v{layer}", std=0.5, device=DEVICE))
    lengths = [torch.tensor(lengths_now, dtype=torch.int32, device=DEVICE) for _ in range(config.layers)]
    alone = []  # one private batch-1 state per sequence for the oracle
    for row, filled in enumerate(lengths_now):
        alone.append(([k[row:row + 1].clone() for k in keys], [v[row:row + 1].clone() for v in values],
                      [torch.full((1,), filled, dtype=torch.int32, device=DEVICE) for _ in range(config.layers)]))
    ids = synth_ids(batch, config.vocab, seed=8).view(batch, 1).to(DEVICE)
    for step in range(3):
        positions = torch.tensor([[n + step] for n in lengths_now], dtype=torch.int64, device=DEVICE)
        logits = kernel.decode_ragged(ids, positions, keys, values, lengths)
        kernel.check()
        with torch.no_grad():
            expected = torch.cat([oracle.decode_step(config, weights, tables, ids[row:row + 1], positions[row:row + 1], *alone[row])
                                  for row in range(batch)])
        assert_parity(logits, expected, f"ragged logits at step {step}")
        ids = expected[:, 0].float().argmax(-1).view(batch, 1)
    assert all(torch.equal(length.cpu(), torch.tensor([n + 3 for n in lengths_now], dtype=torch.int32)) for length in lengths)
    for row, filled in enumerate(lengths_now):
        assert_parity(keys[-1][row:row + 1, :filled + 3], alone[row][0][-1][:, :filled + 3], f"sequence {row} key cache")


def test_step_from_host_matches_decode_steps():
    """The one-call host-driven step (ids and positions up, sampled token down, synchronised) walks the
    same greedy path as the device-resident loop: same tokens, same caches, same lengths."""
    from megabake_b200.runtime import DecoderKernel
    from megabake_b200.synth import new_kv_state, synth_ids, synth_weights, tiny_config

    device = torch.device("cuda:0")
    config = tiny_config()
    weights = synth_weights(config, seed=0, device=device)
    kernel = DecoderKernel(config, weights, max_tokens=2, max_positions=32, device=device)
    batch, steps = 2, 6
    first = synth_ids(batch, config.vocab, seed=5, name="host-step").view(batch, 1)
    state_a = new_kv_state(config, batch, 32, device)
    state_b = new_kv_state(config, batch, 32, device)
    ids = first.to(device)
    positions = torch.zeros((batch, 1), dtype=torch.int64, device=device)
    expected = kernel.decode_steps(ids, positions, *state_a, steps=steps).cpu()
    host_ids, host_pos, host_tok = (torch.empty((batch, 1), dtype=torch.int64).pin_memory() for _ in range(3))
    host_ids.copy_(first)
    for step in range(steps):
        host_pos.fill_(step)
        kernel.step_from_host(host_ids, host_pos, *state_b, host_tok)
        assert torch.equal(host_tok.view(-1), expected[:, step]), f"step {step}"
        host_ids.copy_(host_tok)
    kernel.check()
    for layer in range(config.layers):
        assert torch.equal(state_a[0][layer], state_b[0][layer]) and torch.equal(state_a[1][layer], state_b[1][layer])
        assert int(state_a[2][layer]) == int(state_b[2][layer]) == steps
