"""The handle-free, allocation-free decode attention entry point against the handle-based
one: same inputs, two calls in a row, bit-identical outputs, caches and lengths.  Collected
last so that it runs after every other GPU test has used the library; it also passes alone."""

import ctypes

import pytest
import torch

from megabake_b200 import _native
from megabake_b200.synth import synth_normal, synth_weights, tiny_config

pytestmark = pytest.mark.gpu


def _static_call(lib, heads, kv_heads, dim, query, key, value, key_cache, value_cache, length, output):
    device = query.device.index
    stream = torch.cuda.current_stream(query.device).cuda_stream
    return lib.mk_kv_attention_static(
        heads, kv_heads, dim, query.data_ptr(), key.data_ptr(), value.data_ptr(), key_cache.data_ptr(),
        value_cache.data_ptr(), length.data_ptr(), query.shape[0], key_cache.shape[1], output.data_ptr(),
        device, ctypes.c_void_p(stream))


@pytest.mark.parametrize("shape", [(2, 4, 2, 64, 48, 5), (3, 8, 1, 64, 700, 650), (1, 4, 4, 128, 40, 0)])
def test_static_scratch_entry_point_matches_the_handle_one(shape):
    from megabake_b200.runtime import DecoderKernel

    batch, heads, kv_heads, dim, capacity, filled = shape
    device = torch.device("cuda:0")
    torch.cuda.set_device(device)
    lib = _native.load()
    config = tiny_config(q_heads=heads, kv_heads=kv_heads, head_dim=dim, hidden=heads * dim)
    kernel = DecoderKernel(config, synth_weights(config, device=device), max_tokens=batch, max_positions=16, device=device)
    caches = [synth_normal((batch, capacity, kv_heads, dim), seed=21, name=f"c{i}", std=1.0, device=device) for i in (0, 1)]
    state_a = [caches[0].clone(), caches[1].clone(), torch.full((1,), filled, dtype=torch.int32, device=device)]
    state_b = [caches[0].clone(), caches[1].clone(), torch.full((1,), filled, dtype=torch.int32, device=device)]
    for call in range(2):
        query = synth_normal((batch, 1, heads, dim), seed=22, name=f"q{call}", std=1.0, device=device)
        key = synth_normal((batch, 1, kv_heads, dim), seed=22, name=f"k{call}", std=1.0, device=device)
        value = synth_normal((batch, 1, kv_heads, dim), seed=22, name=f"v{call}", std=1.0, device=device)
        expected = kernel.kv_attention(query, key, value, *state_a)
        kernel.check()
        output = torch.full((batch * heads, 1, dim), float("nan"), dtype=torch.bfloat16, device=device)
        _native.check("mk_kv_attention_static",
                      _static_call(lib, heads, kv_heads, dim, query, key, value, *state_b, output))
        torch.cuda.synchronize(device)
        assert torch.equal(output, expected), f"call {call}: outputs differ"
        assert torch.equal(state_a[0], state_b[0]) and torch.equal(state_a[1], state_b[1])
        assert int(state_b[2]) == filled + call + 1 == int(state_a[2])


def test_static_scratch_entry_point_matches_the_reference_recording_and_the_oracle():
    """The same calls the reference's own op made when the golden file was recorded (tests/golden/ops.pt),
    then two split-context steps against the oracle: outputs within the tolerance of the op tests
    (2e-2 absolute + 1e-2 relative), caches and lengths exact."""
    from conftest import assert_parity, load_golden
    from oracle import decoder_oracle as oracle

    device = torch.device("cuda:0")
    torch.cuda.set_device(device)
    lib = _native.load()
    record = load_golden("ops.pt")
    first = record["calls"][0]
    key_cache = torch.zeros_like(first["key_cache"], device=device)
    value_cache = torch.zeros_like(first["value_cache"], device=device)
    length = torch.zeros(1, dtype=torch.int32, device=device)
    for index, call in enumerate(record["calls"]):
        source = call["source"].to(device)
        batch, _, heads, dim = source.shape
        kv_heads = call["key"].shape[2]
        output = torch.full((batch * heads, 1, dim), float("nan"), dtype=torch.bfloat16, device=device)
        _native.check("mk_kv_attention_static",
                      _static_call(lib, heads, kv_heads, dim, source, call["key"].to(device), call["value"].to(device),
                                   key_cache, value_cache, length, output))
        torch.cuda.synchronize(device)
        assert_parity(output, call["output"], f"static kv_attention, recorded call {index}")
        assert torch.equal(key_cache.cpu(), call["key_cache"]) and torch.equal(value_cache.cpu(), call["value_cache"])
        assert torch.equal(length.cpu(), call["length"])

    batch, heads, kv_heads, dim, capacity, filled = 2, 8, 2, 64, 600, 597
    key_cache = synth_normal((batch, capacity, kv_heads, dim), seed=31, name="kc", std=1.0, device=device)
    value_cache = synth_normal((batch, capacity, kv_heads, dim), seed=31, name="vc", std=1.0, device=device)
    ref_k, ref_v = key_cache.clone(), value_cache.clone()
    length = torch.full((1,), filled, dtype=torch.int32, device=device)
    ref_length = length.clone()
    for step in range(2):
        query = synth_normal((batch, 1, heads, dim), seed=31, name=f"q{step}", std=1.0, device=device)
        key = synth_normal((batch, 1, kv_heads, dim), seed=31, name=f"k{step}", std=1.0, device=device)
        value = synth_normal((batch, 1, kv_heads, dim), seed=31, name=f"v{step}", std=1.0, device=device)
        output = torch.full((batch * heads, 1, dim), float("nan"), dtype=torch.bfloat16, device=device)
        _native.check("mk_kv_attention_static",
                      _static_call(lib, heads, kv_heads, dim, query, key, value, key_cache, value_cache, length, output))
        torch.cuda.synchronize(device)
        expected = oracle.kv_attention(query, key, value, ref_k, ref_v, ref_length)
        assert_parity(output, expected, f"static kv_attention against the oracle, step {step}")
    assert torch.equal(key_cache, ref_k) and torch.equal(value_cache, ref_v) and int(length) == filled + 2 == int(ref_length)


def test_static_scratch_entry_point_rejects_what_does_not_fit():
    device = torch.device("cuda:0")
    torch.cuda.set_device(device)
    lib = _native.load()
    batch, heads, dim = 64, 32, 128  # 64 * 16 * (192 * 32 + 4 * 128 * 32) bytes = 22 MiB > 4 MiB
    tensor = torch.zeros(batch, 1, heads, dim, dtype=torch.bfloat16, device=device)
    cache = torch.zeros(batch, 2, heads, dim, dtype=torch.bfloat16, device=device)
    length = torch.zeros(1, dtype=torch.int32, device=device)
    output = torch.zeros(batch * heads, 1, dim, dtype=torch.bfloat16, device=device)
    code = _static_call(lib, heads, heads, dim, tensor, tensor, tensor, cache, cache.clone(), length, output)
    assert code == _native.MK_ERR_WORKSPACE
    message = lib.mk_last_error().decode()
    assert "static array holds 4194304" in message and "use mk_kv_attention" in message
    torch.cuda.synchronize(device)
    assert int(length) == 0
