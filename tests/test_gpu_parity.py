"""GPU parity tests: the CUDA path, called through the C ABI, against the golden vectors
the reference's own code produced and against the CPU/GPU oracle on the same seeded inputs.

Tolerance for floating point is the north star's: 2e-2 absolute + 1e-2 relative on bf16
values computed with fp32 accumulation.  Integer state (valid lengths, appended cache rows
copied from inputs) must match exactly.
"""

import pytest
import torch

from conftest import (ATOL, RTOL, assert_deep_parity, assert_no_worse_than, assert_parity, load_golden, record_stat,
                      relative_l2, token_agrees, token_defensible)
from megabake_b200.synth import (CONFIGS, DecoderConfig, new_kv_state, rope_tables, synth_ids, synth_normal,
                                 synth_weights, tiny_config)

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def device():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    return torch.device("cuda:0")


def make_kernel(config, weights, device, **kwargs):
    from megabake_b200.runtime import DecoderKernel

    return DecoderKernel(config, weights, device=device, **kwargs)


# --------------------------------------------------------------------------- projections
@pytest.mark.parametrize("engine", ["tcgen05", "fma"])
@pytest.mark.parametrize("shape", [(1, 128, 64), (1, 256, 2048), (4, 576, 576), (3, 192, 576), (1, 2048, 8192),
                                   (16, 2048, 2048), (20, 1024, 1024), (2, 896, 4864), (5, 100, 128)])
def test_linear_matches_fp32_reference(device, engine, shape):
    rows, n, k = shape
    config = tiny_config()
    kernel = make_kernel(config, synth_weights(config, device=device), device, max_tokens=32, max_positions=16,
                         engine=engine)
    source = synth_normal((rows, k), seed=1, name=f"x{shape}", std=1.0, device=device)
    weight = synth_normal((n, k), seed=2, name=f"w{shape}", std=0.05, device=device)
    bias = synth_normal((n,), seed=3, name=f"b{shape}", std=0.5, device=device)
    expected = (source.float() @ weight.float().T + bias.float()).to(torch.bfloat16)
    result = kernel.linear(source, weight, bias)
    kernel.check()
    assert_parity(result, expected, f"linear {shape} on {engine}")
    assert (result == expected).float().mean().item() > 0.98
    no_bias = kernel.linear(source, weight)
    assert_parity(no_bias, (source.float() @ weight.float().T).to(torch.bfloat16), f"linear without bias {shape}")


# --------------------------------------------------------------------------- decode vs golden
def run_golden_decode(name, device, engine, steps=None, deep=False):
    close = assert_deep_parity if deep else assert_parity
    record = load_golden(f"decode_{name}.pt")
    config = DecoderConfig(**record["config"])
    weights = synth_weights(config, seed=record["seed"], norm_std=record["norm_std"], device=device)
    capacity = record["capacity"]
    prompt = record["prompt"]
    batch = prompt.shape[0]
    kernel = make_kernel(config, weights, device, max_tokens=batch, max_positions=capacity, engine=engine)
    keys, values, lengths = new_kv_state(config, batch, capacity, device)
    tokens = record["tokens"].to(device)
    total = tokens.shape[1]
    run = total - 1 if steps is None else min(total - 1, steps)
    offset = total - 1 - record["topk_values"].shape[0]
    ties = 0
    worst_l2 = 0.0
    for position in range(run):
        ids = tokens[:, position].reshape(batch, 1).contiguous()
        positions = torch.full((batch, 1), position, dtype=torch.int64, device=device)
        logits = kernel.decode(ids, positions, keys, values, lengths)
        if position in record["full_logits"]:
            close(logits, record["full_logits"][position], f"{name} logits at {position}")
            worst_l2 = max(worst_l2, relative_l2(logits, record["full_logits"][position]))
        if position >= offset:
            golden_indices = record["topk_indices"][position - offset]
            golden_values = record["topk_values"][position - offset]
            mine = torch.gather(logits[:, 0].float().cpu(), 1, golden_indices.long()).to(torch.bfloat16)
            close(mine, golden_values, f"{name} top-k logits at {position}")
            if position + 1 >= prompt.shape[1]:
                for row in range(batch):
                    assert token_agrees(logits[row, 0].cpu(), golden_indices[row], golden_values[row]), (
                        f"{name}: greedy token at position {position + 1} differs beyond a bf16 tie")
                    ties += int(int(logits[row, 0].float().argmax()) != int(golden_indices[row, 0]))
    kernel.check()
    record_stat(f"teacher_forced_{name}_{engine}", calls=run, argmax_differs_from_golden=ties,
                worst_rel_l2_to_golden_logits=worst_l2)
    if run == total - 1:
        assert torch.equal(torch.stack(lengths).cpu(), record["lengths"])
        rows = record.get("cache_rows")
        for layer, (key_cache, value_cache) in record["caches"].items():
            mine_k = keys[layer] if rows is None else keys[layer][:, rows.to(device)]
            mine_v = values[layer] if rows is None else values[layer][:, rows.to(device)]
            close(mine_k, key_cache, f"{name} key cache {layer}")
            close(mine_v, value_cache, f"{name} value cache {layer}")
    return ties, run


@pytest.mark.parametrize("engine", ["tcgen05", "fma"])
@pytest.mark.parametrize("name", ["tiny", "tiny_hf"])
def test_decode_tiny_matches_reference(device, name, engine):
    ties, _ = run_golden_decode(name, device, engine)
    assert ties == 0


@pytest.mark.parametrize("engine", ["tcgen05", "fma"])
def test_decode_smollm_135m_64_steps(device, engine):
    ties, run = run_golden_decode("c1", device, engine, deep=True)
    # measured on a B200: 5 (tensor engine) and 4 (small-launch kernel) of 64 greedy tokens differ from the
    # CPU-made golden ones, each at a position where the reference's own top two logits tie in bf16
    # (token_agrees checks that)
    assert run == 67 and ties <= 5


@pytest.mark.parametrize("engine", ["auto", "tcgen05"])
def test_decode_qwen2_half_b_64_steps(device, engine):
    ties, run = run_golden_decode("c2", device, engine, deep=True)
    # measured on a B200: 1 of 64 (tensor engine) and 2 of 64 (small-launch kernel, whose attention sums in
    # tensor-core order for grouped heads), each a bf16 tie of the reference's own top two logits
    assert run == 67 and ties <= 2


def run_yardstick_decode(name, device):
    """Golden decode for the 24-layer, 2048-channel shape.  Teacher-forced on the reference's
    tokens, three evaluations run side by side on this device: the kernel, the oracle in bf16
    (eager PyTorch) and the oracle in fp32.  Logits and cache rows must be no further from fp32
    than the reference path's own bf16 evaluations (eager here, the CPU golden); every greedy
    token must be the golden one or one that bf16 noise can defend."""
    from oracle import decoder_oracle as oracle

    record = load_golden(f"decode_{name}.pt")
    config = DecoderConfig(**record["config"])
    weights = synth_weights(config, seed=record["seed"], norm_std=record["norm_std"], device=device)
    weights32 = {key: tensor.float() for key, tensor in weights.items()}
    capacity, tokens = record["capacity"], record["tokens"].to(device)
    batch, total = tokens.shape
    kernel = make_kernel(config, weights, device, max_tokens=batch, max_positions=capacity)
    tables = rope_tables(config, capacity, device=device)
    tables32 = rope_tables(config, capacity, device=device, dtype=torch.float32)
    mine_state = new_kv_state(config, batch, capacity, device)
    eager_state = new_kv_state(config, batch, capacity, device)
    truth_state = new_kv_state(config, batch, capacity, device)
    truth_state = ([k.float() for k in truth_state[0]], [v.float() for v in truth_state[1]], truth_state[2])
    offset = total - 1 - record["topk_values"].shape[0]
    same_as_golden = generated = 0
    for position in range(total - 1):
        ids = tokens[:, position].reshape(batch, 1).contiguous()
        positions = torch.full((batch, 1), position, dtype=torch.int64, device=device)
        mine = kernel.decode(ids, positions, *mine_state)
        with torch.no_grad():
            eager = oracle.decode_step(config, weights, tables, ids, positions, *eager_state)
            truth = oracle.decode_step(config, weights32, tables32, ids, positions, *truth_state)
        if position < offset:
            continue
        rivals = [eager]
        if position in record["full_logits"]:
            rivals.append(record["full_logits"][position])
        assert_no_worse_than(mine, rivals, truth, f"{name} logits at {position}")
        if position + 1 >= record["prompt"].shape[1]:
            golden_token = record["topk_indices"][position - offset][:, 0]
            for row in range(batch):
                generated += 1
                same_as_golden += int(int(mine[row, 0].float().argmax()) == int(golden_token[row]))
                assert token_defensible(mine[row, 0], eager[row, 0], truth[row, 0]), (
                    f"{name}: greedy token at position {position + 1} is not one bf16 noise can defend")
    kernel.check()
    record_stat(f"teacher_forced_{name}", generated=generated, same_as_golden=same_as_golden)
    # measured on a B200: 26 of 28 (short run) and 14 of 16 (context 1024) equal the CPU-made golden tokens; the
    # others are defensible (above) and eager PyTorch on the same GPU differs from the golden run as often
    assert generated > 0 and generated - same_as_golden <= 2, f"{same_as_golden} of {generated} tokens equal the golden ones"
    assert torch.equal(torch.stack(mine_state[2]).cpu(), record["lengths"])
    rows = record.get("cache_rows")
    for layer, (key_cache, value_cache) in record["caches"].items():
        for mine_cache, eager_cache, truth_cache, golden in (
                (mine_state[0][layer], eager_state[0][layer], truth_state[0][layer], key_cache),
                (mine_state[1][layer], eager_state[1][layer], truth_state[1][layer], value_cache)):
            pick = (lambda t: t) if rows is None else (lambda t: t[:, rows.to(t.device)])
            assert_no_worse_than(pick(mine_cache), [pick(eager_cache), golden], pick(truth_cache), f"{name} cache {layer}")


def test_decode_smollm_1_7b_short(device):
    run_yardstick_decode("c3_short", device)


def test_decode_smollm_1_7b_context_1024(device):
    """Headline shape at its benchmark context: 1024 teacher-forced positions, then the
    reference's 16 greedy tokens; logits of the last 20 calls, sampled cache rows, lengths."""
    run_yardstick_decode("c3", device)


# --------------------------------------------------------------------------- decode vs oracle on the same device
def oracle_decode_compare(config, device, batch, capacity, prefill, steps, engine="auto", seed=5):
    from oracle import decoder_oracle as oracle

    weights = synth_weights(config, seed=seed, norm_std=0.1, device=device)
    kernel = make_kernel(config, weights, device, max_tokens=batch, max_positions=capacity, engine=engine)
    tables = rope_tables(config, capacity, device=device)
    keys, values, lengths = new_kv_state(config, batch, capacity, device)
    ref_keys, ref_values, ref_lengths = new_kv_state(config, batch, capacity, device)
    if prefill:
        for layer in range(config.layers):
            shape = (batch, prefill, config.kv_heads, config.head_dim)
            for mine, theirs, tag in ((keys, ref_keys, "k"), (values, ref_values, "v")):
                filled = synth_normal(shape, seed=seed, name=f"{tag}{layer}", std=0.5, device=device)
                mine[layer][:, :prefill] = filled
                theirs[layer][:, :prefill] = filled
            lengths[layer].fill_(prefill)
            ref_lengths[layer].fill_(prefill)
    ids = synth_ids(batch, config.vocab, seed=seed).view(batch, 1).to(device)
    for step in range(steps):
        positions = torch.full((batch, 1), prefill + step, dtype=torch.int64, device=device)
        logits = kernel.decode(ids, positions, keys, values, lengths)
        with torch.no_grad():
            expected = oracle.decode_step(config, weights, tables, ids, positions, ref_keys, ref_values, ref_lengths)
        kernel.check()
        assert_parity(logits, expected, f"logits at step {step}")
        ids = expected[:, 0].float().argmax(-1).view(batch, 1)
    assert torch.equal(torch.stack(lengths), torch.stack(ref_lengths))
    for layer in (0, config.layers - 1):
        assert_parity(keys[layer], ref_keys[layer], f"key cache {layer}")
        assert_parity(values[layer], ref_values[layer], f"value cache {layer}")


def test_decode_error_no_worse_than_eager_bf16(device):
    """The reference's own yardstick (tests/gpu/test_task31_full_model.py:205-211): measured
    against the same model evaluated in fp32, the kernel may be no further off than eager
    bf16 on the same device times 1.25 plus 1e-3 in relative L2 (1.5 in the largest element
    error, see assert_no_worse_than) -- logits and cache contents, 30 layers."""
    from oracle import decoder_oracle as oracle

    config = CONFIGS["smollm-135m"]
    capacity, batch, steps = 32, 1, 6
    weights = synth_weights(config, seed=0, device=device)
    weights32 = {name: tensor.float() for name, tensor in weights.items()}
    kernel = make_kernel(config, weights, device, max_tokens=batch, max_positions=capacity)
    tables = rope_tables(config, capacity, device=device)
    tables32 = rope_tables(config, capacity, device=device, dtype=torch.float32)
    mine_state = new_kv_state(config, batch, capacity, device)
    eager_state = new_kv_state(config, batch, capacity, device)
    truth_state = new_kv_state(config, batch, capacity, device)
    truth_state = ([k.float() for k in truth_state[0]], [v.float() for v in truth_state[1]], truth_state[2])
    ids = synth_ids(batch, config.vocab, seed=3).view(batch, 1).to(device)
    for step in range(steps):
        positions = torch.full((batch, 1), step, dtype=torch.int64, device=device)
        mine = kernel.decode(ids, positions, *mine_state)
        with torch.no_grad():
            eager = oracle.decode_step(config, weights, tables, ids, positions, *eager_state)
            truth = oracle.decode_step(config, weights32, tables32, ids, positions, *truth_state)
        kernel.check()
        assert_no_worse_than(mine, [eager], truth, f"step {step}: logits")
        ids = truth[:, 0].argmax(-1).view(batch, 1)
    for layer in (0, 15, 29):
        for what, mine_cache, eager_cache, truth_cache in zip(("key", "value"), mine_state[:2], eager_state[:2], truth_state[:2]):
            assert_no_worse_than(mine_cache[layer][:, :steps], [eager_cache[layer][:, :steps]], truth_cache[layer][:, :steps],
                                 f"{what} cache {layer}")


@pytest.mark.parametrize("engine", ["auto", "tcgen05"])
@pytest.mark.parametrize("batch", [1, 2, 3, 4, 5, 8, 16, 21])
def test_decode_batches_match_oracle(device, batch, engine):
    """Batches 1-4 run the small-launch kernel under "auto" (one instantiation per token count),
    larger ones the tensor engine (token tiles of 16 and 32)."""
    oracle_decode_compare(tiny_config(q_heads=4, kv_heads=1, hidden=256), device, batch, capacity=24, prefill=0, steps=4,
                          engine=engine)


@pytest.mark.parametrize("engine", ["tcgen05", "fma"])
def test_decode_split_context_matches_oracle(device, engine):
    """A long filled prefix makes the attention phase cut the context across CTAs."""
    config = tiny_config(q_heads=8, kv_heads=2, hidden=512, intermediate=1024)
    oracle_decode_compare(config, device, batch=2, capacity=1024, prefill=700, steps=3, engine=engine)


@pytest.mark.parametrize("batch", [4, 5, 8, 9, 33])
def test_decode_is_one_launch_per_step(device, batch):
    """Every decode step is exactly one cooperative launch, whatever the batch."""
    config = tiny_config(q_heads=4, kv_heads=1, hidden=256)
    weights = synth_weights(config, seed=3, norm_std=0.1, device=device)
    kernel = make_kernel(config, weights, device, max_tokens=batch, max_positions=16, engine="auto")
    keys, values, lengths = new_kv_state(config, batch, 16, device)
    ids = synth_ids(batch, config.vocab, seed=3).view(batch, 1).to(device)
    before = kernel.launch_info()["launches"]
    kernel.decode(ids, torch.zeros((batch, 1), dtype=torch.int64, device=device), keys, values, lengths)
    kernel.check()
    assert kernel.launch_info()["launches"] - before == 1
    assert all(int(length.item()) == 1 for length in lengths)


def test_decode_to_the_last_cache_row(device):
    oracle_decode_compare(tiny_config(), device, batch=2, capacity=8, prefill=5, steps=3)


@pytest.mark.parametrize("engine", ["auto", "tcgen05"])
def test_decode_qwen_form_gqa7_bias(device, engine):
    config = tiny_config(hidden=448, q_heads=7, kv_heads=1, intermediate=960, qkv_bias=True, rope_style="hf",
                         rms_eps=1e-6, rope_theta=1e6)
    oracle_decode_compare(config, device, batch=2, capacity=96, prefill=70, steps=3, engine=engine)


@pytest.mark.parametrize("engine", ["auto", "tcgen05"])
def test_decode_head_dim_128(device, engine):
    config = tiny_config(hidden=512, q_heads=4, kv_heads=2, head_dim=128, intermediate=768)
    oracle_decode_compare(config, device, batch=1, capacity=160, prefill=130, steps=3, engine=engine)


@pytest.mark.parametrize("head_dim", [64, 128])
def test_small_launch_attention_walks_several_tiles(device, head_dim):
    """32 (sequence, head) row groups leave four context chunks of ~350 keys: more than one
    shared-memory tile per chunk (304 keys of 64, 152 of 128), the new key in the last tile."""
    config = tiny_config(hidden=512, q_heads=8, kv_heads=8, head_dim=head_dim, intermediate=768)
    oracle_decode_compare(config, device, batch=4, capacity=1500, prefill=1400, steps=2)


def test_small_launch_kernel_falls_back_beyond_its_score_buffer(device):
    """Capacities past 16 chunks x 4096 / group keys go to the tensor engine, same results."""
    config = tiny_config(q_heads=8, kv_heads=1, hidden=512, intermediate=1024)
    oracle_decode_compare(config, device, batch=1, capacity=8200, prefill=600, steps=2)


def test_decode_is_deterministic_at_full_size(device):
    """Size-independent property at the headline shape: two runs from the same state are bit-identical."""
    config = CONFIGS["smollm-1.7b"]
    weights = synth_weights(config, seed=0, device=device)
    kernel = make_kernel(config, weights, device, max_tokens=1, max_positions=2048)
    outputs = []
    for _ in range(2):
        keys, values, lengths = new_kv_state(config, 1, 2048, device)
        for layer in range(config.layers):
            keys[layer][:, :1024] = synth_normal((1, 1024, 32, 64), seed=0, name=f"k{layer}", std=1.0, device=device)
            values[layer][:, :1024] = synth_normal((1, 1024, 32, 64), seed=0, name=f"v{layer}", std=1.0, device=device)
            lengths[layer].fill_(1024)
        ids = torch.tensor([[1234]], device=device)
        run = []
        for step in range(3):
            positions = torch.full((1, 1), 1024 + step, dtype=torch.int64, device=device)
            logits = kernel.decode(ids, positions, keys, values, lengths)
            run.append(logits.clone())
            ids = logits[:, 0].float().argmax(-1).view(1, 1)
        kernel.check()
        outputs.append((run, keys[5][:, 1024:1027].clone(), int(lengths[0].item())))
    for first, second in zip(outputs[0][0], outputs[1][0]):
        assert torch.equal(first, second)
    assert torch.equal(outputs[0][1], outputs[1][1]) and outputs[0][2] == outputs[1][2] == 1027
    assert torch.isfinite(outputs[0][0][-1].float()).all()


# --------------------------------------------------------------------------- the two ops
def test_kv_attention_op_matches_reference(device):
    record = load_golden("ops.pt")
    config = tiny_config(q_heads=4, kv_heads=2)
    kernel = make_kernel(config, synth_weights(config, device=device), device, max_tokens=4, max_positions=16)
    first = record["calls"][0]
    key_cache = torch.zeros_like(first["key_cache"], device=device)
    value_cache = torch.zeros_like(first["value_cache"], device=device)
    length = torch.zeros(1, dtype=torch.int32, device=device)
    for index, call in enumerate(record["calls"]):
        output = kernel.kv_attention(call["source"].to(device), call["key"].to(device), call["value"].to(device),
                                     key_cache, value_cache, length)
        kernel.check()
        assert_parity(output, call["output"], f"kv_attention call {index}")
        assert torch.equal(key_cache.cpu(), call["key_cache"]) and torch.equal(value_cache.cpu(), call["value_cache"])
        assert torch.equal(length.cpu(), call["length"])


def test_kv_attention_op_long_context_and_overflow(device):
    from oracle import decoder_oracle as oracle

    config = tiny_config(q_heads=8, kv_heads=2, hidden=512)
    kernel = make_kernel(config, synth_weights(config, device=device), device, max_tokens=2, max_positions=16)
    batch, capacity, filled = 2, 600, 598
    key_cache = synth_normal((batch, capacity, 2, 64), seed=9, name="kc", std=1.0, device=device)
    value_cache = synth_normal((batch, capacity, 2, 64), seed=9, name="vc", std=1.0, device=device)
    ref_k, ref_v = key_cache.clone(), value_cache.clone()
    length = torch.full((1,), filled, dtype=torch.int32, device=device)
    ref_length = length.clone()
    for step in range(2):
        query = synth_normal((batch, 1, 8, 64), seed=9, name=f"q{step}", std=1.0, device=device)
        key = synth_normal((batch, 1, 2, 64), seed=9, name=f"k{step}", std=1.0, device=device)
        value = synth_normal((batch, 1, 2, 64), seed=9, name=f"v{step}", std=1.0, device=device)
        output = kernel.kv_attention(query, key, value, key_cache, value_cache, length)
        expected = oracle.kv_attention(query, key, value, ref_k, ref_v, ref_length)
        kernel.check()
        assert_parity(output, expected, f"split-context kv_attention step {step}")
    assert torch.equal(key_cache, ref_k) and torch.equal(value_cache, ref_v) and int(length.item()) == capacity
    # The cache is full now: the reference raises, the kernel reports through its status word and changes nothing.
    kernel.kv_attention(query, key, value, key_cache, value_cache, length)
    assert kernel.status()["status"] == "KV_OVERFLOW"
    assert int(length.item()) == capacity and torch.equal(key_cache, ref_k)
    assert kernel.status()["status"] == "OK"


def test_attention_op_matches_reference(device):
    record = load_golden("ops.pt")["attention"]
    config = tiny_config(q_heads=4, kv_heads=2)
    kernel = make_kernel(config, synth_weights(config, device=device), device, max_tokens=32, max_positions=16)
    query, key, value = (record[name].to(device) for name in ("query", "key", "value"))
    masked = kernel.attention(query, key, value, record["mask"].to(device), record["scale"])
    plain = kernel.attention(query, key, value, None, record["scale"])
    kernel.check()
    assert_parity(masked, record["output"], "attention with causal mask")
    assert_parity(plain, record["output_nomask"], "attention without mask")


# --------------------------------------------------------------------------- prefill
@pytest.mark.parametrize("name", ["tiny", "c1", "c2"])
def test_prefill_matches_reference_model(device, name):
    record = load_golden(f"prefill_{name}.pt")
    config = DecoderConfig(**record["config"])
    weights = synth_weights(config, seed=record["seed"], norm_std=record["norm_std"], device=device)
    ids = record["ids"].to(device)
    batch, length = ids.shape
    kernel = make_kernel(config, weights, device, max_tokens=batch * length, max_positions=max(length, 16))
    logits = kernel.prefill(ids)
    kernel.check()
    if name == "tiny":
        assert_parity(logits[:, -1], record["last_logits"], f"prefill {name} last logits")
        top = torch.gather(logits.float().cpu(), 2, record["topk_indices"].long()).to(torch.bfloat16)
        assert_parity(top, record["topk_values"], f"prefill {name} top-k")
        if "logits" in record:
            assert_parity(logits, record["logits"], f"prefill {name} logits")
        return
    # 24-30 layers: the reference path's own bf16 evaluations are the yardstick
    from oracle import decoder_oracle as oracle

    positions = torch.arange(length, device=device).expand(batch, length).contiguous()
    mask = oracle.causal_mask(batch, length).to(device)
    weights32 = {key: tensor.float() for key, tensor in weights.items()}
    with torch.no_grad():
        eager = oracle.prefill(config, weights, rope_tables(config, max(length, 16), device=device), ids, positions, mask)
        truth = oracle.prefill(config, weights32, rope_tables(config, max(length, 16), device=device, dtype=torch.float32),
                               ids, positions, mask.float())
    assert_no_worse_than(logits[:, -1], [eager[:, -1], record["last_logits"]], truth[:, -1], f"prefill {name} last logits")
    assert_no_worse_than(logits, [eager], truth, f"prefill {name} logits")
    assert token_defensible(logits[0, -1], eager[0, -1], truth[0, -1])


def test_prefill_with_mask_and_ragged_length_matches_oracle(device):
    from oracle import decoder_oracle as oracle

    config = tiny_config(rope_style="hf")
    weights = synth_weights(config, seed=11, norm_std=0.1, device=device)
    batch, length = 2, 37
    kernel = make_kernel(config, weights, device, max_tokens=batch * length, max_positions=64)
    tables = rope_tables(config, 64, device=device)
    ids = synth_ids(batch * length, config.vocab, seed=11).view(batch, length).to(device)
    positions = torch.arange(length, device=device).expand(batch, length).contiguous()
    mask = oracle.causal_mask(batch, length).to(device).contiguous()
    with torch.no_grad():
        expected = oracle.prefill(config, weights, tables, ids, positions, mask)
    assert_parity(kernel.prefill(ids, positions, mask), expected, "prefill with an explicit causal mask")
    assert_parity(kernel.prefill(ids), expected, "prefill with the implied causal mask")
    kernel.check()


# --------------------------------------------------------------------------- status, rebinding, trace
def test_device_status_instead_of_trap(device):
    config = tiny_config()
    weights = synth_weights(config, device=device)
    kernel = make_kernel(config, weights, device, max_tokens=2, max_positions=8)
    keys, values, lengths = new_kv_state(config, 1, 8, device)
    good = torch.tensor([[3]], device=device)
    position = torch.zeros((1, 1), dtype=torch.int64, device=device)
    kernel.decode(torch.tensor([[config.vocab]], device=device), position, keys, values, lengths)
    assert kernel.status()["status"] == "BAD_INDEX" and int(lengths[0].item()) == 0
    kernel.decode(good, torch.full((1, 1), 8, dtype=torch.int64, device=device), keys, values, lengths)
    assert kernel.status()["status"] == "BAD_INDEX"
    for length in lengths:
        length.fill_(8)
    kernel.decode(good, position, keys, values, lengths)
    assert kernel.status()["status"] == "KV_OVERFLOW" and int(lengths[0].item()) == 8
    for length in lengths:
        length.fill_(0)
    logits = kernel.decode(good, position, keys, values, lengths)
    kernel.check()
    assert torch.isfinite(logits.float()).all() and int(lengths[0].item()) == 1


def test_rebinding_a_replaced_weight_is_visible(device):
    config = tiny_config()
    weights = synth_weights(config, seed=1, device=device)
    kernel = make_kernel(config, weights, device, max_tokens=1, max_positions=8)

    def one_step():
        keys, values, lengths = new_kv_state(config, 1, 8, device)
        return kernel.decode(torch.tensor([[7]], device=device), torch.zeros((1, 1), dtype=torch.int64, device=device),
                             keys, values, lengths)

    before = one_step()
    assert not kernel.rebind_if_changed(weights)
    weights = dict(weights)
    weights["model.layers.1.mlp.down_proj.weight"] = torch.zeros_like(weights["model.layers.1.mlp.down_proj.weight"])
    assert kernel.rebind_if_changed(weights)
    after = one_step()
    kernel.check()
    assert not torch.equal(before, after)


@pytest.mark.parametrize("engine", ["tcgen05", "auto"])
def test_event_trace_reports_every_phase(device, engine):
    from megabake_b200.runtime import decode_trace

    config = tiny_config()
    kernel = make_kernel(config, synth_weights(config, device=device), device, max_tokens=1, max_positions=8, engine=engine)
    keys, values, lengths = new_kv_state(config, 1, 8, device)
    buffer = kernel.set_trace(256)
    kernel.decode(torch.tensor([[7]], device=device), torch.zeros((1, 1), dtype=torch.int64, device=device), keys,
                  values, lengths)
    kernel.check()
    codes, times = decode_trace(buffer)
    barriers = int((codes[0] == 5).sum())
    # seven grid barriers per layer on the tensor engine (five between phases, two behind the norm phases) and one
    # behind the final norm; the small-launch kernel at one token hands every phase's outputs to the next as
    # stamped words and keeps a single barrier at the end of the launch
    assert barriers == (7 * config.layers + 1 if engine == "tcgen05" else 1)
    stamps = times[0][codes[0] > 0][:barriers]
    assert bool((stamps[1:] >= stamps[:-1]).all())
    kernel.set_trace(0)
