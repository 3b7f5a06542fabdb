"""Generate the golden vectors under tests/golden/ by running the REFERENCE's own code.

Run once, in a container that has the reference checkout (read-only):

    python tests/golden/make_golden.py --reference <checkout of the reference> [--cases a,b,...]

The reference package cannot be imported whole here (its ``__init__`` pulls in a
CuTe-DSL release this image does not have), so a stub ``megabake`` package is
put in ``sys.modules`` whose ``__path__`` is the reference's ``src/megabake``;
``megabake.lowering`` (which registers ``megabake::kv_attention`` and
``megabake::attention`` with their eager bodies), ``tests/fixtures.py``
(``StatefulSmolLM``), ``benchmarks/stateful_models.py`` (``StatefulCausalLM``)
and ``megabake.fx_handler.hf_attention`` then import unchanged.  Weights come
from ``megabake_b200.synth`` (a pure integer function of seed/name/index) and
are loaded into the transformers model classes the reference wraps.

Nothing in the test suite or the benchmark reads the reference at run time;
they read the ``.pt`` files this script writes.
"""

from __future__ import annotations

import argparse
import importlib.util
import json
import sys
import time
import types
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))

from megabake_b200.synth import CONFIGS, DecoderConfig, synth_ids, synth_normal, synth_weights, tiny_config  # noqa: E402

TOPK = 16


def load_reference(root: Path):
    stub = types.ModuleType("megabake")
    stub.__path__ = [str(root / "src" / "megabake")]
    sys.modules["megabake"] = stub
    import megabake.lowering as lowering  # noqa: F401  (registers the ops)

    def by_path(name, path):
        spec = importlib.util.spec_from_file_location(name, path)
        module = importlib.util.module_from_spec(spec)
        sys.modules[name] = module
        spec.loader.exec_module(module)
        return module

    fixtures = by_path("reference_fixtures", root / "tests" / "fixtures.py")
    stateful = by_path("reference_stateful_models", root / "benchmarks" / "stateful_models.py")
    import megabake.fx_handler.hf_attention as hf_attention

    return lowering, fixtures, stateful, hf_attention


def build_hf_model(config: DecoderConfig, weights, positions: int):
    """The transformers model class the reference wraps, holding ``weights``."""
    common = dict(
        hidden_size=config.hidden, intermediate_size=config.intermediate,
        num_attention_heads=config.q_heads, num_key_value_heads=config.kv_heads,
        num_hidden_layers=config.layers, vocab_size=config.vocab,
        max_position_embeddings=positions, rms_norm_eps=config.rms_eps,
        tie_word_embeddings=config.tied, head_dim=config.head_dim,
        rope_parameters={"rope_type": "default", "rope_theta": config.rope_theta},
    )
    if config.qkv_bias:
        from transformers import Qwen2Config, Qwen2ForCausalLM

        model = Qwen2ForCausalLM(Qwen2Config(**common))
    else:
        from transformers import LlamaConfig, LlamaForCausalLM

        model = LlamaForCausalLM(LlamaConfig(**common))
    model.set_attn_implementation("eager")
    model.config.use_cache = False
    # Same order as the reference's SmolLMArchitecture (tests/fixtures.py:336):
    # the cast also rounds the rotary inv_freq buffer to bf16.
    model = model.to(dtype=torch.bfloat16).eval()
    missing, unexpected = model.load_state_dict(weights, strict=False)
    assert not unexpected, unexpected
    assert all("rotary" in name or "inv_freq" in name for name in missing), missing
    return model


def topk_of(logits: torch.Tensor):
    values, indices = logits.float().topk(TOPK, dim=-1)
    return values.to(torch.bfloat16), indices.to(torch.int32)


def run_decode_case(config, model_wrapper, prompt, steps, capacity, *, keep_full, keep_cache_layers, cache_rows=None):
    batch = prompt.shape[0]
    shape = (batch, capacity, config.kv_heads, config.head_dim)
    keys = [torch.zeros(shape, dtype=torch.bfloat16) for _ in range(config.layers)]
    values = [torch.zeros(shape, dtype=torch.bfloat16) for _ in range(config.layers)]
    lengths = [torch.zeros(1, dtype=torch.int32) for _ in range(config.layers)]
    interleaved = getattr(model_wrapper, "interleaved_state", False)
    if interleaved:
        state = [t for triple in zip(keys, values, lengths) for t in triple]
    else:
        state = keys + values + lengths
    tokens = [prompt[:, index] for index in range(prompt.shape[1])]
    total = prompt.shape[1] + steps
    record = {"topk_values": [], "topk_indices": [], "full_logits": {}, "logit_sum": []}
    started = time.time()
    with torch.no_grad():
        for position in range(total - 1):
            ids = tokens[position].view(batch, 1)
            positions = torch.full((batch, 1), position, dtype=torch.int64)
            logits = model_wrapper(ids, positions, *state)
            if position + 1 >= prompt.shape[1]:
                tokens.append(logits[:, 0].float().argmax(dim=-1))
            if position >= total - 1 - record_window(prompt.shape[1], steps):
                top_values, top_indices = topk_of(logits[:, 0])
                record["topk_values"].append(top_values)
                record["topk_indices"].append(top_indices)
                record["logit_sum"].append(logits.double().sum())
            if position in keep_full:
                record["full_logits"][position] = logits.clone()
            if position % 64 == 0:
                print(f"  position {position}/{total - 1}  {time.time() - started:.1f}s", flush=True)
    record["tokens"] = torch.stack(tokens, dim=1)
    record["lengths"] = torch.stack(lengths)
    caches = {}
    for layer in keep_cache_layers:
        rows = slice(None) if cache_rows is None else cache_rows
        caches[layer] = (keys[layer][:, rows].clone(), values[layer][:, rows].clone())
    record["caches"] = caches
    record["cache_rows"] = cache_rows
    record["topk_values"] = torch.stack(record["topk_values"])
    record["topk_indices"] = torch.stack(record["topk_indices"])
    record["logit_sum"] = torch.stack(record["logit_sum"])
    return record


_WINDOW = {"value": None}


def record_window(prompt_length, steps):
    return _WINDOW["value"] if _WINDOW["value"] is not None else prompt_length + steps


def decode_wrapper(config, fixtures, stateful, model):
    if config.qkv_bias:
        wrapper = stateful.StatefulCausalLM(model).eval()
        wrapper.interleaved_state = True  # benchmarks/stateful_models.py:149-152
        return wrapper
    return fixtures.StatefulSmolLM(model).eval()  # all keys, all values, all lengths


def case_ops(lowering, out: Path):
    """Known answers for the two custom ops' eager bodies."""
    batch, q_heads, kv_heads, dim, capacity = 2, 4, 2, 64, 16
    record = {"calls": []}
    key_cache = torch.zeros(batch, capacity, kv_heads, dim, dtype=torch.bfloat16)
    value_cache = torch.zeros_like(key_cache)
    length = torch.zeros(1, dtype=torch.int32)
    for call in range(5):
        source = synth_normal((batch, 1, q_heads, dim), seed=28, name=f"q{call}", std=1.0)
        key = synth_normal((batch, 1, kv_heads, dim), seed=28, name=f"k{call}", std=1.0)
        value = synth_normal((batch, 1, kv_heads, dim), seed=28, name=f"v{call}", std=1.0)
        output = lowering.kv_attention(source, key, value, key_cache, value_cache, length)
        record["calls"].append(
            dict(source=source, key=key, value=value, output=output.clone(),
                 key_cache=key_cache.clone(), value_cache=value_cache.clone(), length=length.clone())
        )
    seq = 8
    query = synth_normal((batch, seq, q_heads, dim), seed=27, name="pq", std=1.0)
    key = synth_normal((batch, seq, kv_heads, dim), seed=27, name="pk", std=1.0)
    value = synth_normal((batch, seq, kv_heads, dim), seed=27, name="pv", std=1.0)
    allowed = torch.tril(torch.ones(seq, seq, dtype=torch.bool))
    mask = torch.zeros(seq, seq, dtype=torch.bfloat16).masked_fill(~allowed, torch.finfo(torch.bfloat16).min)
    mask = mask[None, None].expand(batch, 1, seq, seq).contiguous()
    record["attention"] = dict(
        query=query, key=key, value=value, mask=mask, scale=dim ** -0.5,
        output=lowering.attention(query, key, value, mask, dim ** -0.5),
        output_nomask=lowering.attention(query, key, value, None, dim ** -0.5),
    )
    torch.save(record, out / "ops.pt")


def case_decode(name, config, fixtures, stateful, out, *, prompt_length, steps, capacity, batch=1,
                seed=0, norm_std=None, window=None, keep_full=(), cache_layers=(), cache_rows=None):
    print(f"[{name}] building", flush=True)
    weights = synth_weights(config, seed=seed, norm_std=norm_std)
    model = build_hf_model(config, weights, positions=capacity)
    wrapper = decode_wrapper(config, fixtures, stateful, model)
    prompt = synth_ids(batch * prompt_length, config.vocab, seed=seed, name="prompt").view(batch, prompt_length)
    _WINDOW["value"] = window
    record = run_decode_case(
        config, wrapper, prompt, steps, capacity,
        keep_full=set(keep_full), keep_cache_layers=cache_layers, cache_rows=cache_rows,
    )
    record.update(
        config=config.to_dict(), seed=seed, norm_std=norm_std, prompt=prompt, steps=steps,
        capacity=capacity, window=window,
    )
    torch.save(record, out / f"decode_{name}.pt")
    print(f"[{name}] tokens tail {record['tokens'][0, -8:].tolist()}", flush=True)


def case_prefill(name, config, hf_attention, out, *, length, batch=1, seed=0, norm_std=None, full=False):
    print(f"[prefill {name}] building", flush=True)
    weights = synth_weights(config, seed=seed, norm_std=norm_std)
    model = build_hf_model(config, weights, positions=max(length, 16))
    hf_attention.register_transformers_attention()
    model.set_attn_implementation("megabake")
    ids = synth_ids(batch * length, config.vocab, seed=seed, name="prompt").view(batch, length)
    with torch.no_grad():
        logits = model(input_ids=ids).logits
    values, indices = topk_of(logits)
    record = dict(config=config.to_dict(), seed=seed, norm_std=norm_std, ids=ids,
                  topk_values=values, topk_indices=indices, last_logits=logits[:, -1].clone())
    if full:
        record["logits"] = logits.clone()
    torch.save(record, out / f"prefill_{name}.pt")


def host_fingerprint() -> dict:
    """CPU model and SIMD flags: bf16 matmul rounding on the CPU depends on them, so
    the tests demand bit-equality with these files only on a matching host."""
    model, flags = "", ""
    for line in open("/proc/cpuinfo"):
        if line.startswith("model name") and not model:
            model = line.split(":", 1)[1].strip()
        if line.startswith("flags") and not flags:
            names = line.split(":", 1)[1].split()
            flags = " ".join(sorted(n for n in names if n.startswith(("avx", "amx"))))
    return {"cpu_model": model, "simd_flags": flags, "torch": torch.__version__}


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", required=True, help="path of a checkout of the reference project")
    parser.add_argument("--cases", default="ops,tiny,tiny_hf,prefill_tiny,c1,c2,prefill_c1,prefill_c2")
    parser.add_argument("--out", default=str(HERE))
    args = parser.parse_args()
    torch.manual_seed(0)
    lowering, fixtures, stateful, hf_attention = load_reference(Path(args.reference))
    out = Path(args.out)
    cases = set(args.cases.split(","))
    (out / "HOST.json").write_text(json.dumps(host_fingerprint(), indent=1))
    if "ops" in cases:
        case_ops(lowering, out)
    if "tiny" in cases:
        case_decode("tiny", tiny_config(), fixtures, stateful, out, prompt_length=3, steps=12,
                    capacity=16, batch=2, norm_std=0.1, keep_full=range(14), cache_layers=(0, 1))
    if "tiny_hf" in cases:
        config = tiny_config(qkv_bias=True, rope_style="hf", rms_eps=1e-6, rope_theta=1e6,
                             q_heads=6, kv_heads=2, hidden=384, name="tiny_hf")
        case_decode("tiny_hf", config, fixtures, stateful, out, prompt_length=3, steps=12,
                    capacity=16, batch=1, norm_std=0.1, keep_full=range(14), cache_layers=(0, 1))
    if "prefill_tiny" in cases:
        case_prefill("tiny", tiny_config(rope_style="hf", name="tiny_prefill"), hf_attention, out,
                     length=7, batch=2, norm_std=0.1, full=True)
    if "c1" in cases:
        case_decode("c1", CONFIGS["smollm-135m"], fixtures, stateful, out, prompt_length=4, steps=64,
                    capacity=128, keep_full=(3, 66), cache_layers=(0, 29))
    if "c2" in cases:
        case_decode("c2", CONFIGS["qwen2-0.5b"], fixtures, stateful, out, prompt_length=4, steps=64,
                    capacity=128, keep_full=(66,), cache_layers=(0, 23))
    if "prefill_c1" in cases:
        case_prefill("c1", CONFIGS["smollm-135m"], hf_attention, out, length=4)
    if "prefill_c2" in cases:
        case_prefill("c2", CONFIGS["qwen2-0.5b"], hf_attention, out, length=4)
    if "c3" in cases:
        # Headline shape at a long context: 1024 teacher-forced positions, then 16 greedy tokens.
        rows = torch.tensor([0, 1, 511, 1022, 1023, 1024, 1030, 1039])
        case_decode("c3", CONFIGS["smollm-1.7b"], fixtures, stateful, out, prompt_length=1024, steps=16,
                    capacity=2048, window=20, keep_full=(), cache_layers=(0, 23), cache_rows=rows)
    if "c3_short" in cases:
        case_decode("c3_short", CONFIGS["smollm-1.7b"], fixtures, stateful, out, prompt_length=4, steps=28,
                    capacity=128, keep_full=(30,), cache_layers=(23,))


if __name__ == "__main__":
    main()
