"""GPU tests of the reference-facing surface: ``make_backend`` compiles Dynamo-captured Hugging
Face decoders to the megakernel, and the ``megabake::`` ops dispatch to it on CUDA tensors."""

import pytest
import torch

import megabake_b200 as megabake
from megabake_b200.synth import new_kv_state, rope_tables, synth_ids, synth_normal, synth_weights, tiny_config
from tests.conftest import assert_parity, load_golden

pytestmark = pytest.mark.gpu
DEVICE = torch.device("cuda:0")


def _hf_model(config, seed=0, norm_std=0.1, positions=64):
    from transformers import LlamaConfig, LlamaForCausalLM, Qwen2Config, Qwen2ForCausalLM

    common = dict(hidden_size=config.hidden, intermediate_size=config.intermediate,
                  num_attention_heads=config.q_heads, num_key_value_heads=config.kv_heads,
                  num_hidden_layers=config.layers, vocab_size=config.vocab, head_dim=config.head_dim,
                  max_position_embeddings=positions, rms_norm_eps=config.rms_eps, tie_word_embeddings=True,
                  rope_parameters={"rope_type": "default", "rope_theta": config.rope_theta})
    model = Qwen2ForCausalLM(Qwen2Config(**common)) if config.qkv_bias else LlamaForCausalLM(LlamaConfig(**common))
    model = model.to(torch.bfloat16).eval()
    model.load_state_dict(synth_weights(config, seed=seed, norm_std=norm_std), strict=False)
    return model.to(DEVICE)


@pytest.mark.parametrize("bias", [False, True])
def test_backend_compiles_stateful_decoder_and_matches_the_oracle(bias):
    from oracle import decoder_oracle as oracle

    config = tiny_config(rope_style="hf", layers=3, qkv_bias=bias, q_heads=4, kv_heads=2)
    model = _hf_model(config)
    backend = megabake.make_backend(mode="decode", compile_kernel=True)
    step = torch.compile(megabake.ExplicitStateDecoder(model).eval(), backend=backend, fullgraph=True, dynamic=False)
    batch, capacity = 2, 16
    keys, values, lengths = new_kv_state(config, batch, capacity, DEVICE)
    state = [t for triple in zip(keys, values, lengths) for t in triple]
    weights = synth_weights(config, seed=0, norm_std=0.1)
    tables = rope_tables(config, 64)
    ref_keys, ref_values, ref_lengths = new_kv_state(config, batch, capacity)
    ids = synth_ids(batch, config.vocab, seed=5).view(batch, 1)
    with torch.no_grad():
        for position in range(6):
            positions = torch.full((batch, 1), position, dtype=torch.int64)
            logits = step(ids.to(DEVICE), positions.to(DEVICE), *state)
            expected = oracle.decode_step(config, weights, tables, ids, positions, ref_keys, ref_values, ref_lengths)
            assert_parity(logits.cpu(), expected, f"logits at step {position}")
            ids = expected[:, 0].float().argmax(-1).view(batch, 1)
    assert [int(n) for n in lengths] == [6] * config.layers
    assert_parity(keys[-1].cpu(), ref_keys[-1], "last layer key cache")
    context = backend.megabake_contexts[-1]
    assert context.requirements["execution"] == "megakernel" and context.requirements["gate_relative_l2"] < 0.02
    forward = backend.megabake_last_callable
    assert forward.megabake_compiled.launch_info()["launches"] >= 7  # the gate's call and six steps
    assert forward.megabake_compiled.status()["status"] == "OK"


def test_backend_sees_replaced_weights():
    config = tiny_config(rope_style="hf", layers=2)
    model = _hf_model(config)
    step = torch.compile(megabake.ExplicitStateDecoder(model).eval(),
                         backend=megabake.make_backend(mode="decode", compile_kernel=True), fullgraph=True, dynamic=False)
    keys, values, lengths = new_kv_state(config, 1, 8, DEVICE)
    state = [t for triple in zip(keys, values, lengths) for t in triple]
    ids, positions = torch.tensor([[7]], device=DEVICE), torch.zeros(1, 1, dtype=torch.int64, device=DEVICE)
    with torch.no_grad():
        before = step(ids, positions, *state).clone()
        model.model.layers[1].mlp.down_proj.weight.mul_(-1.0)  # in place: visible without rebinding
        for length in lengths:
            length.zero_()
        after = step(ids, positions, *state)
    assert not torch.equal(before, after)


def test_backend_compiles_hf_prefill_through_the_attention_interface():
    config = tiny_config(rope_style="hf", layers=2)
    model = _hf_model(config)
    megabake.register_transformers_attention()
    ids = synth_ids(6, config.vocab, seed=2).view(1, 6).to(DEVICE)
    with torch.no_grad():
        model.set_attn_implementation("eager")
        expected = model(input_ids=ids).logits
        model.set_attn_implementation("megabake")
        backend = megabake.make_backend(mode="prefill", compile_kernel=True)
        compiled = torch.compile(model, backend=backend, fullgraph=True, dynamic=False)
        logits = compiled(input_ids=ids, use_cache=False).logits
    assert backend.megabake_contexts[-1].requirements["execution"] == "megakernel"
    assert_parity(logits.cpu(), expected.cpu(), "prefill logits")


def test_prefill_mode_rejects_stateful_graph_before_device_work():
    config = tiny_config(rope_style="hf", layers=1)
    model = _hf_model(config)
    step = torch.compile(megabake.ExplicitStateDecoder(model).eval(),
                         backend=megabake.make_backend(mode="prefill", compile_kernel=True), fullgraph=True, dynamic=False)
    keys, values, lengths = new_kv_state(config, 1, 8, DEVICE)
    with pytest.raises(Exception, match="prefill mode cannot compile a stateful KV cache update"):
        with torch.no_grad():
            step(torch.tensor([[1]], device=DEVICE), torch.zeros(1, 1, dtype=torch.int64, device=DEVICE),
                 keys[0], values[0], lengths[0])
    assert int(lengths[0]) == 0


def test_ops_dispatch_to_the_kernel_on_cuda():
    record = load_golden("ops.pt")
    first = record["calls"][0]
    key_cache = torch.zeros_like(first["key_cache"], device=DEVICE)
    value_cache = torch.zeros_like(first["value_cache"], device=DEVICE)
    length = torch.zeros(1, dtype=torch.int32, device=DEVICE)
    for index, call in enumerate(record["calls"]):
        output = torch.ops.megabake.kv_attention(call["source"].to(DEVICE), call["key"].to(DEVICE),
                                                 call["value"].to(DEVICE), key_cache, value_cache, length)
        assert_parity(output.cpu(), call["output"], f"kv_attention call {index}")
        assert torch.equal(key_cache.cpu(), call["key_cache"]) and torch.equal(length.cpu(), call["length"])
    attention = record["attention"]
    query, key, value = (attention[name].to(DEVICE) for name in ("query", "key", "value"))
    masked = torch.ops.megabake.attention(query, key, value, attention["mask"].to(DEVICE), attention["scale"])
    plain = torch.ops.megabake.attention(query, key, value, None, attention["scale"])
    assert_parity(masked.cpu(), attention["output"], "attention with mask")
    assert_parity(plain.cpu(), attention["output_nomask"], "attention without mask")


def test_decode_step_module_on_cuda_runs_the_kv_attention_op():
    config = tiny_config(rope_style="hf", layers=2)
    model = _hf_model(config)
    ids = synth_ids(4, config.vocab, seed=9).view(1, 4).to(DEVICE)
    with torch.no_grad():
        model.set_attn_implementation("eager")
        expected = model(input_ids=ids).logits
        step = megabake.DecodeStep(model, capacity=8)
        state = []
        for shapes in step.state_shapes(batch=1, dtype=torch.bfloat16):
            state += [torch.zeros(shape, dtype=dtype, device=DEVICE) for shape, dtype in shapes]
        for position in range(4):
            logits = step(ids[:, position:position + 1], torch.tensor([[position]], device=DEVICE), *state)
            assert_parity(logits[:, 0].cpu(), expected[:, position].cpu(), f"position {position}")
