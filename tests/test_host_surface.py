"""CPU tests of the host side: the C-ABI library loads and exports what the header declares,
option validation and error formats match the reference's, the ops keep their schemas, the
backend recognises decoder graphs and keeps the mode contract, ``bucketed`` pads and checks."""

import re
from pathlib import Path

import pytest
import torch

import megabake_b200 as megabake
from megabake_b200 import _native
from megabake_b200.synth import new_kv_state, synth_normal, synth_weights, tiny_config

ROOT = Path(__file__).resolve().parent.parent


def test_library_exports_every_declared_symbol():
    header = (ROOT / "include" / "megabake_b200.h").read_text()
    declared = set(re.findall(r"\b(mk_[a-z_]+)\s*\(", header))
    lib = _native.load()
    assert declared == set(_native.EXPORTS)
    for name in declared:
        assert hasattr(lib, name), name


def test_option_validation_messages():
    with pytest.raises(ValueError, match="Unsupported mode"):
        megabake.make_backend(mode="train")
    with pytest.raises(ValueError, match="Unsupported fallback"):
        megabake.make_backend(fallback="eager")
    with pytest.raises(TypeError, match="cache must be a boolean"):
        megabake.make_backend(cache="yes")
    with pytest.raises(TypeError, match="model_name"):
        megabake.make_backend(model_name="")
    with pytest.raises(TypeError, match="compile_kernel"):
        megabake.make_backend(compile_kernel="maybe")
    with pytest.raises(ValueError, match="scheduler"):
        megabake.make_backend(scheduler="fifo")
    backend = megabake.make_backend(mode="decode")
    assert backend.__name__ == "megabake_backend"
    assert dict(backend.megabake_options)["fallback"] == "error" and backend.megabake_options["mode"] == "decode"
    with pytest.raises(TypeError):
        backend.megabake_options["mode"] = "prefill"


def test_compiler_error_format():
    error = megabake.CompilerError(
        megabake.CompilerDiagnostic("plan-search", "no body", ("op:1", "op:2"), ("region:3",), "a GEMM body"),
        safe_for_fallback=True)
    assert str(error) == "plan-search: no body; source operations: op:1, op:2; regions: region:3; requirement: a GEMM body"
    assert isinstance(error, ValueError) and error.safe_for_fallback


def test_op_schemas_and_fakes():
    kv = torch.ops.megabake.kv_attention.default._schema
    assert [a.name for a in kv.arguments] == ["source", "key", "value", "key_cache", "value_cache", "valid_length"]
    assert [a.name for a in kv.arguments if a.alias_info is not None and a.alias_info.is_write] == [
        "key_cache", "value_cache", "valid_length"]
    att = torch.ops.megabake.attention.default._schema
    assert [a.name for a in att.arguments] == ["query", "key", "value", "mask", "scale"]
    query = torch.empty(2, 5, 4, 64, device="meta", dtype=torch.bfloat16)
    key = torch.empty(2, 5, 2, 64, device="meta", dtype=torch.bfloat16)
    assert torch.ops.megabake.attention(query, key, key, None, 0.125).shape == (8, 5, 64)
    with pytest.raises(RuntimeError, match="one-token decode only"):
        torch.ops.megabake.kv_attention(torch.zeros(1, 2, 1, 64, dtype=torch.bfloat16), *[torch.zeros(1, 2, 1, 64, dtype=torch.bfloat16)] * 4,
                                        torch.zeros(1, dtype=torch.int32))
    with pytest.raises(RuntimeError, match="exceeds capacity"):
        token = torch.zeros(1, 1, 1, 64, dtype=torch.bfloat16)
        torch.ops.megabake.kv_attention(token, token, token, torch.zeros(1, 2, 1, 64, dtype=torch.bfloat16),
                                        torch.zeros(1, 2, 1, 64, dtype=torch.bfloat16), torch.full((1,), 2, dtype=torch.int32))


def _tiny_llama(config, seed=0):
    from transformers import LlamaConfig, LlamaForCausalLM

    hf = LlamaConfig(hidden_size=config.hidden, intermediate_size=config.intermediate,
                     num_attention_heads=config.q_heads, num_key_value_heads=config.kv_heads,
                     num_hidden_layers=config.layers, vocab_size=config.vocab, head_dim=config.head_dim,
                     max_position_embeddings=32, rms_norm_eps=config.rms_eps, tie_word_embeddings=True,
                     rope_parameters={"rope_type": "default", "rope_theta": config.rope_theta})
    model = LlamaForCausalLM(hf).to(torch.bfloat16).eval()
    model.load_state_dict(synth_weights(config, seed=seed, norm_std=0.1), strict=False)
    return model


def test_backend_reference_path_and_recognition_on_cpu():
    from oracle import decoder_oracle as oracle
    from megabake_b200.synth import rope_tables

    config = tiny_config(rope_style="hf", layers=2)
    model = _tiny_llama(config)
    wrapper = megabake.ExplicitStateDecoder(model).eval()
    backend = megabake.make_backend(mode="decode", compile_kernel=False)
    compiled = torch.compile(wrapper, backend=backend, fullgraph=True, dynamic=False)
    keys, values, lengths = new_kv_state(config, 2, 8)
    state = [t for triple in zip(keys, values, lengths) for t in triple]
    ref_keys, ref_values, ref_lengths = new_kv_state(config, 2, 8)
    weights = synth_weights(config, seed=0, norm_std=0.1)
    tables = rope_tables(config, 32)
    ids = torch.tensor([[5], [9]])
    with torch.no_grad():
        for position in range(3):
            positions = torch.full((2, 1), position)
            logits = compiled(ids, positions, *state)
            expected = oracle.decode_step(config, weights, tables, ids, positions, ref_keys, ref_values, ref_lengths)
            assert torch.equal(logits, expected)
            ids = expected[:, 0].float().argmax(-1).view(2, 1)
    assert int(lengths[0]) == 3 and torch.equal(keys[1], ref_keys[1])
    context = backend.megabake_contexts[-1]
    assert context.requirements["execution"] == "reference"
    example = [torch.tensor([[5], [9]]), torch.zeros(2, 1, dtype=torch.int64)]
    binding = None

    def probe(graph_module, example_inputs):
        nonlocal binding
        binding = megabake.recognise_decoder(graph_module, example_inputs, "decode")
        with pytest.raises(ValueError, match="prefill mode cannot compile a stateful KV cache update"):
            megabake.recognise_decoder(graph_module, example_inputs, "prefill")
        return graph_module.forward

    torch._dynamo.reset()
    with torch.no_grad():
        torch.compile(wrapper, backend=probe, fullgraph=True, dynamic=False)(*example, *state)
    assert binding.stateful and binding.config.layers == 2 and binding.config.q_heads == config.q_heads
    assert binding.config.kv_heads == config.kv_heads and binding.config.rope_style == "hf" and binding.config.tied
    assert binding.config.rms_eps == pytest.approx(config.rms_eps) and binding.capacity == 8
    assert len(binding.weight_indices) == 2 * 9 + 3 and len(binding.state_indices) == 2


def test_prefill_mode_rejects_a_stateful_graph_without_the_kernel():
    config = tiny_config(rope_style="hf", layers=1)
    wrapper = megabake.ExplicitStateDecoder(_tiny_llama(config)).eval()
    compiled = torch.compile(wrapper, backend=megabake.make_backend(mode="prefill", compile_kernel=False),
                             fullgraph=True, dynamic=False)
    keys, values, lengths = new_kv_state(config, 1, 4)
    with pytest.raises(Exception, match="prefill mode cannot compile a stateful KV cache update"):
        with torch.no_grad():
            compiled(torch.tensor([[1]]), torch.zeros(1, 1, dtype=torch.int64), keys[0], values[0], lengths[0])


def test_unrecognised_graph_raises_before_any_device_work():
    backend = megabake.make_backend(mode="prefill", compile_kernel=True)
    with pytest.raises(Exception, match="plan-search"):
        torch.compile(lambda x: torch.relu(x) + 1, backend=backend, fullgraph=True)(torch.ones(4))


def test_hf_attention_routes_prefill_through_the_op():
    config = tiny_config(rope_style="hf", layers=2)
    model = _tiny_llama(config)
    ids = torch.tensor([[3, 8, 1, 200, 17]])
    with torch.no_grad():
        model.set_attn_implementation("eager")
        eager = model(input_ids=ids).logits
        assert megabake.register_transformers_attention() == "megabake"
        model.set_attn_implementation("megabake")
        routed = model(input_ids=ids).logits
    assert torch.equal(eager, routed)


def test_decode_step_matches_past_key_values_decode():
    config = tiny_config(rope_style="hf", layers=2)
    model = _tiny_llama(config).float()
    ids = torch.tensor([[3, 8, 1, 200]])
    with torch.no_grad():
        model.set_attn_implementation("eager")
        expected = model(input_ids=ids).logits
        step = megabake.DecodeStep(model, capacity=8)
        state = []
        for shapes in step.state_shapes(batch=1, dtype=torch.float32):
            state += [torch.zeros(shape, dtype=dtype) for shape, dtype in shapes]
        for position in range(ids.shape[1]):
            logits = step(ids[:, position:position + 1], torch.tensor([[position]]), *state)
            torch.testing.assert_close(logits[:, 0], expected[:, position], atol=1e-4, rtol=1e-4)
    assert int(state[2]) == 4


def test_bucketed_pads_cuts_and_checks():
    class Causal(torch.nn.Module):
        def forward(self, values):
            return torch.cumsum(values, dim=1)

    wrapped = megabake.bucketed(Causal(), backend="eager", sequence_args={"values": 1}, buckets=(4, 8))
    values = torch.arange(5.0).view(1, 5)
    assert torch.equal(wrapped(values), torch.cumsum(values, dim=1))
    assert wrapped.verified == {8} and wrapped.bucket_for(3) == 4
    with pytest.raises(ValueError, match="exceeds the largest bucket"):
        wrapped(torch.zeros(1, 9))
    with pytest.raises(ValueError, match="at least one sequence argument"):
        megabake.bucketed(Causal(), backend="eager", sequence_args={})

    class Leaky(torch.nn.Module):
        def forward(self, values):
            return values + values.sum(dim=1, keepdim=True)

    with pytest.raises(megabake.PaddingDependence):
        megabake.bucketed(Leaky(), backend="eager", sequence_args={"values": 1}, buckets=(8,))(torch.ones(1, 3))


def test_synthetic_weights_are_a_pure_function_of_seed_and_name():
    first = synth_normal((64, 33), seed=4, name="w")
    assert torch.equal(first, synth_normal((64, 33), seed=4, name="w"))
    assert not torch.equal(first, synth_normal((64, 33), seed=5, name="w"))
    big = synth_normal((1 << 16,), seed=0, name="stat", dtype=torch.float32)
    assert abs(float(big.mean())) < 1e-3 and abs(float(big.std()) - 0.02) < 5e-4
    config = megabake.CONFIGS["smollm-1.7b"]
    assert config.streamed_parameters() == 1_711_376_384
    assert config.decode_bytes(1, 1024) == 2 * 1_711_376_384 + 2 * 24 * 2048 * 2 * 1025
