"""Pin the CPU oracle to the golden vectors the reference's own code produced
(tests/golden/make_golden.py).  On the kind of host that wrote the files the
match must be bit for bit; elsewhere token ids and lengths must still be equal
and floating-point values within the parity tolerance."""

import pytest
import torch

from conftest import assert_deep_parity, assert_parity, load_golden
from megabake_b200.synth import DecoderConfig, rope_tables, synth_weights
from oracle import decoder_oracle as oracle


def test_kv_attention_matches_reference_op(exact_cpu):
    record = load_golden("ops.pt")
    first = record["calls"][0]
    key_cache = torch.zeros_like(first["key_cache"])
    value_cache = torch.zeros_like(first["value_cache"])
    length = torch.zeros(1, dtype=torch.int32)
    for index, call in enumerate(record["calls"]):
        output = oracle.kv_attention(call["source"], call["key"], call["value"], key_cache, value_cache, length)
        assert_parity(output, call["output"], f"kv_attention call {index}", exact=exact_cpu)
        assert torch.equal(key_cache, call["key_cache"]) and torch.equal(value_cache, call["value_cache"])
        assert torch.equal(length, call["length"])


def test_kv_attention_rejects_overflow_and_long_queries():
    cache = torch.zeros(1, 2, 1, 64, dtype=torch.bfloat16)
    token = torch.zeros(1, 1, 1, 64, dtype=torch.bfloat16)
    length = torch.full((1,), 2, dtype=torch.int32)
    with pytest.raises(RuntimeError, match="exceeds capacity"):
        oracle.kv_attention(token, token, token, cache, cache.clone(), length)
    with pytest.raises(RuntimeError, match="one-token decode only"):
        oracle.kv_attention(token.expand(1, 2, 1, 64), token, token, cache, cache.clone(), length)


def test_attention_matches_reference_op(exact_cpu):
    record = load_golden("ops.pt")["attention"]
    masked = oracle.attention(record["query"], record["key"], record["value"], record["mask"], record["scale"])
    assert_parity(masked, record["output"], "attention with causal mask", exact=exact_cpu)
    plain = oracle.attention(record["query"], record["key"], record["value"], None, record["scale"])
    assert_parity(plain, record["output_nomask"], "attention without mask", exact=exact_cpu)


def _decode_against(name, exact, steps=None, deep=False):
    """``deep``: on a host other than the one that wrote the file, a 24-layer x 2048-channel model's
    bf16 logits are compared by relative L2 (two CPU generations already differ by a few percent
    there) and near-tied greedy tokens may differ; on the writing host everything is bit for bit."""
    record = load_golden(f"decode_{name}.pt")
    config = DecoderConfig(**record["config"])
    weights = synth_weights(config, seed=record["seed"], norm_std=record["norm_std"])
    tables = rope_tables(config, record["capacity"])
    prompt = record["prompt"]
    total = prompt.shape[1] + record["steps"]
    run = total - 1 if steps is None else min(steps, total - 1)
    keys, values, lengths = oracle.new_state(config, prompt.shape[0], record["capacity"])
    tokens = record["tokens"]
    offset = total - 1 - record["topk_values"].shape[0]
    with torch.no_grad():
        for position in range(run):
            ids = tokens[:, position].reshape(-1, 1)
            positions = torch.full_like(ids, position)
            logits = oracle.decode_step(config, weights, tables, ids, positions, keys, values, lengths)
            loose = deep and not exact
            if position + 1 >= prompt.shape[1] and not loose:
                assert torch.equal(logits[:, 0].float().argmax(-1), tokens[:, position + 1]), f"{name}: token {position + 1}"
            if position in record["full_logits"]:
                if loose:
                    assert_deep_parity(logits, record["full_logits"][position], f"{name} logits at {position}")
                else:
                    assert_parity(logits, record["full_logits"][position], f"{name} logits at {position}", exact=exact)
            if position >= offset and not loose:
                top = torch.gather(logits[:, 0].float(), 1, record["topk_indices"][position - offset].long())
                assert_parity(top.to(torch.bfloat16), record["topk_values"][position - offset], f"{name} top-k at {position}", exact=exact)
    if run == total - 1:
        assert torch.equal(torch.stack(lengths), record["lengths"])
        close = assert_deep_parity if (deep and not exact) else (lambda a, b, what: assert_parity(a, b, what, exact=exact))
        for layer, (key_cache, value_cache) in record["caches"].items():
            close(keys[layer], key_cache, f"{name} key cache {layer}")
            close(values[layer], value_cache, f"{name} value cache {layer}")


def test_decode_tiny_llama_form(exact_cpu):
    _decode_against("tiny", exact_cpu)


def test_decode_tiny_qwen_form(exact_cpu):
    _decode_against("tiny_hf", exact_cpu)


def test_decode_smollm_135m_shape(exact_cpu):
    _decode_against("c1", exact_cpu)


def test_decode_qwen2_half_b_shape_first_steps(exact_cpu):
    _decode_against("c2", exact_cpu, steps=10)


def test_decode_smollm_1_7b_shape_short_run(exact_cpu):
    """The headline shape (24 layers x 2048 channels): the reference's 4-token prompt and 28 greedy tokens."""
    _decode_against("c3_short", exact_cpu, deep=True)


@pytest.mark.parametrize("name", ["tiny", "c1", "c2"])
def test_prefill_matches_reference_model(name, exact_cpu):
    record = load_golden(f"prefill_{name}.pt")
    config = DecoderConfig(**record["config"])
    weights = synth_weights(config, seed=record["seed"], norm_std=record["norm_std"])
    ids = record["ids"]
    batch, length = ids.shape
    tables = rope_tables(config, max(length, 16))
    positions = torch.arange(length).expand(batch, length)
    with torch.no_grad():
        logits = oracle.prefill(config, weights, tables, ids, positions, oracle.causal_mask(batch, length))
    assert_parity(logits[:, -1], record["last_logits"], f"prefill {name} last logits", exact=exact_cpu)
    top = torch.gather(logits.float(), 2, record["topk_indices"].long()).to(torch.bfloat16)
    assert_parity(top, record["topk_values"], f"prefill {name} top-k", exact=exact_cpu)
    if "logits" in record:
        assert_parity(logits, record["logits"], f"prefill {name} logits", exact=exact_cpu)
