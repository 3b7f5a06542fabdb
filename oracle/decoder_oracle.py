"""CPU oracle for the decoder hot path.  TEST INFRASTRUCTURE ONLY.

This file restates, in plain eager PyTorch on plain tensors, what the reference
computes on the path the CUDA megakernel replaces.  Only tests, the smoke check
and the benchmark's CPU-baseline leg may import it; the product package never
does.  Every function names the reference lines it follows.

Parity is pinned: ``tests/golden/make_golden.py`` runs the reference's own code
(its ``megabake::kv_attention`` / ``megabake::attention`` op bodies and its
``StatefulSmolLM`` / ``StatefulCausalLM`` decode wrappers around the
transformers model classes) on the same seeded weights and stores the results
under ``tests/golden/``; ``tests/test_oracle_golden.py`` requires this file to
reproduce them bit for bit.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F


def rms_norm(hidden: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """transformers ``LlamaRMSNorm.forward`` / ``Qwen2RMSNorm.forward`` as called at
    reference tests/fixtures.py:267,302,311: fp32 statistics, one cast to the
    input dtype, then the weight multiply in that dtype."""
    dtype = hidden.dtype
    widened = hidden.to(torch.float32)
    variance = widened.pow(2).mean(-1, keepdim=True)
    widened = widened * torch.rsqrt(variance + eps)
    return weight * widened.to(dtype)


def rotate(source: torch.Tensor, cosine: torch.Tensor, sine: torch.Tensor, style: str) -> torch.Tensor:
    """Rotary embedding on ``[batch, seq, heads, dim]`` with ``cosine``/``sine``
    broadcastable ``[batch, seq, 1, dim]``; every product and sum rounds to bf16.

    ``half_swap`` follows reference tests/fixtures.py:44-54 (the form its decode
    wrapper ``StatefulSmolLM`` uses, tests/fixtures.py:292-293); ``hf`` follows
    transformers ``apply_rotary_pos_emb`` as called at reference
    benchmarks/stateful_models.py:90-91."""
    half = source.shape[-1] // 2
    if style == "half_swap":
        first = source[..., :half] * cosine[..., :half] - source[..., half:] * sine[..., :half]
        second = source[..., half:] * sine[..., :half] + source[..., :half] * cosine[..., :half]
        return torch.cat((first, second), dim=-1)
    if style == "hf":
        rotated = torch.cat((-source[..., half:], source[..., :half]), dim=-1)
        return (source * cosine) + (rotated * sine)
    raise ValueError(f"unknown rope style {style!r}")


def kv_attention(source, key, value, key_cache, value_cache, valid_length) -> torch.Tensor:
    """Reference src/megabake/lowering.py:215-247: append the token's key/value at
    ``valid_length``, advance it, attend over the filled prefix.  Scores are a
    bf16 matmul widened to fp32 and scaled by head_dim**-0.5, softmax in fp32,
    probabilities rounded to bf16, bf16 value matmul."""
    if source.shape[1] != 1:
        raise RuntimeError("megabake kv_attention supports one-token decode only")
    start = int(valid_length.item())
    end = start + source.shape[1]
    if start < 0 or end > key_cache.shape[1]:
        raise RuntimeError(
            f"KV cache length {start} plus {source.shape[1]} exceeds capacity {key_cache.shape[1]}"
        )
    key_cache[:, start:end].copy_(key)
    value_cache[:, start:end].copy_(value)
    valid_length.fill_(end)
    query = source.permute(0, 2, 1, 3)
    keys = key_cache[:, :end].permute(0, 2, 1, 3)
    values = value_cache[:, :end].permute(0, 2, 1, 3)
    if query.shape[1] != keys.shape[1]:
        group = query.shape[1] // keys.shape[1]
        keys = keys.repeat_interleave(group, dim=1)
        values = values.repeat_interleave(group, dim=1)
    scores = (query @ keys.transpose(-2, -1)).float() * source.shape[-1] ** -0.5
    probabilities = torch.softmax(scores, dim=-1).to(source.dtype)
    output = probabilities @ values
    return output.permute(0, 2, 1, 3).reshape(
        source.shape[0] * source.shape[2], source.shape[1], source.shape[3]
    )


def attention(query, key, value, mask, scale: float) -> torch.Tensor:
    """Reference src/megabake/lowering.py:274-300 (Hugging Face eager numerics):
    bf16 score matmul, bf16 scale, bf16 additive mask, fp32 softmax rounded to
    bf16, bf16 value matmul.  ``query`` is [batch, q, heads, dim]."""
    query = query.transpose(1, 2)
    key = key.transpose(1, 2)
    value = value.transpose(1, 2)
    if query.shape[1] != key.shape[1]:
        group = query.shape[1] // key.shape[1]
        key = key.repeat_interleave(group, dim=1)
        value = value.repeat_interleave(group, dim=1)
    scores = torch.matmul(query, key.transpose(2, 3)) * scale
    if mask is not None:
        scores = scores + mask
    probabilities = torch.softmax(scores, dim=-1, dtype=torch.float32).to(query.dtype)
    output = torch.matmul(probabilities, value)
    return output.reshape(-1, output.shape[2], output.shape[3])


def _linear(source, weights, name):
    return F.linear(source, weights[name + ".weight"], weights.get(name + ".bias"))


def _gather_rope(tables, position_ids):
    cosine, sine = tables
    return cosine[position_ids][:, :, None, :], sine[position_ids][:, :, None, :]


def decode_step(config, weights, tables, input_ids, position_ids, key_caches, value_caches, valid_lengths):
    """One-token decode over explicit state.  Llama form: reference
    tests/fixtures.py:247-312 (``StatefulSmolLM.forward``); with q/k/v biases and
    the ``hf`` rotation it is reference benchmarks/stateful_models.py:73-100,134-166
    (``StatefulCausalLM`` on a Qwen2 model).  ``tables`` are the bf16 cos/sin
    tables transformers' rotary embedding yields for each position.  Mutates the
    caches and lengths; returns logits [batch, 1, vocab]."""
    batch = input_ids.shape[0]
    hidden = F.embedding(input_ids, weights["model.embed_tokens.weight"])
    cosine, sine = _gather_rope(tables, position_ids.to(torch.int64))
    for layer in range(config.layers):
        prefix = f"model.layers.{layer}."
        residual = hidden
        normalized = rms_norm(hidden, weights[prefix + "input_layernorm.weight"], config.rms_eps)
        query = _linear(normalized, weights, prefix + "self_attn.q_proj").view(batch, 1, config.q_heads, config.head_dim)
        key = _linear(normalized, weights, prefix + "self_attn.k_proj").view(batch, 1, config.kv_heads, config.head_dim)
        value = _linear(normalized, weights, prefix + "self_attn.v_proj").view(batch, 1, config.kv_heads, config.head_dim)
        query = rotate(query, cosine, sine, config.rope_style)
        key = rotate(key, cosine, sine, config.rope_style)
        attended = kv_attention(query, key, value, key_caches[layer], value_caches[layer], valid_lengths[layer])
        projected = F.linear(attended.reshape(batch, 1, -1), weights[prefix + "self_attn.o_proj.weight"])
        hidden = residual + projected
        residual = hidden
        normalized = rms_norm(hidden, weights[prefix + "post_attention_layernorm.weight"], config.rms_eps)
        gate = F.linear(normalized, weights[prefix + "mlp.gate_proj.weight"])
        up = F.linear(normalized, weights[prefix + "mlp.up_proj.weight"])
        fused = F.silu(gate) * up
        hidden = residual + F.linear(fused, weights[prefix + "mlp.down_proj.weight"])
    final = rms_norm(hidden, weights["model.norm.weight"], config.rms_eps)
    return F.linear(final, weights["lm_head.weight"])


def causal_mask(batch: int, length: int, dtype=torch.bfloat16) -> torch.Tensor:
    """The additive causal mask transformers' ``eager_mask`` builds for a full
    prompt: 0 where key <= query, dtype-min elsewhere; [batch, 1, q, k]."""
    allowed = torch.tril(torch.ones(length, length, dtype=torch.bool))
    mask = torch.zeros(length, length, dtype=dtype).masked_fill(~allowed, torch.finfo(dtype).min)
    return mask[None, None].expand(batch, 1, length, length)


def prefill(config, weights, tables, input_ids, position_ids, mask):
    """Stateless prompt pass: the transformers decoder forward with attention
    routed to ``megabake::attention`` (reference
    src/megabake/fx_handler/hf_attention.py:28-61).  Rotation is transformers'
    own (``hf``) on this path regardless of the decode wrapper's form.
    Returns logits [batch, seq, vocab]."""
    batch, length = input_ids.shape
    hidden = F.embedding(input_ids, weights["model.embed_tokens.weight"])
    cosine, sine = _gather_rope(tables, position_ids.to(torch.int64))
    scale = config.head_dim ** -0.5
    for layer in range(config.layers):
        prefix = f"model.layers.{layer}."
        residual = hidden
        normalized = rms_norm(hidden, weights[prefix + "input_layernorm.weight"], config.rms_eps)
        query = _linear(normalized, weights, prefix + "self_attn.q_proj").view(batch, length, config.q_heads, config.head_dim)
        key = _linear(normalized, weights, prefix + "self_attn.k_proj").view(batch, length, config.kv_heads, config.head_dim)
        value = _linear(normalized, weights, prefix + "self_attn.v_proj").view(batch, length, config.kv_heads, config.head_dim)
        query = rotate(query, cosine, sine, "hf")
        key = rotate(key, cosine, sine, "hf")
        attended = attention(query, key, value, mask, scale)
        attended = attended.view(batch, config.q_heads, length, config.head_dim).transpose(1, 2)
        projected = F.linear(attended.reshape(batch, length, -1), weights[prefix + "self_attn.o_proj.weight"])
        hidden = residual + projected
        residual = hidden
        normalized = rms_norm(hidden, weights[prefix + "post_attention_layernorm.weight"], config.rms_eps)
        gate = F.linear(normalized, weights[prefix + "mlp.gate_proj.weight"])
        up = F.linear(normalized, weights[prefix + "mlp.up_proj.weight"])
        hidden = residual + F.linear(F.silu(gate) * up, weights[prefix + "mlp.down_proj.weight"])
    final = rms_norm(hidden, weights["model.norm.weight"], config.rms_eps)
    return F.linear(final, weights["lm_head.weight"])


def new_state(config, batch: int, capacity: int, device="cpu"):
    """Zero caches [batch, capacity, kv_heads, head_dim] and int32 [1] lengths per layer."""
    shape = (batch, capacity, config.kv_heads, config.head_dim)
    keys = [torch.zeros(shape, dtype=torch.bfloat16, device=device) for _ in range(config.layers)]
    values = [torch.zeros(shape, dtype=torch.bfloat16, device=device) for _ in range(config.layers)]
    lengths = [torch.zeros(1, dtype=torch.int32, device=device) for _ in range(config.layers)]
    return keys, values, lengths


def greedy_decode(config, weights, tables, prompt: torch.Tensor, steps: int, capacity: int, step=None):
    """The harness both sides run: feed the prompt one token at a time through
    the decode step (teacher-forced, filling the cache), then ``steps`` greedy
    tokens.  ``step`` defaults to :func:`decode_step`; the GPU tests pass the
    CUDA path's step with the same signature.  Returns (token ids including the
    prompt, list of logits per call, state)."""
    step = step or (lambda *args: decode_step(config, weights, tables, *args))
    batch = prompt.shape[0]
    device = prompt.device
    keys, values, lengths = new_state(config, batch, capacity, device)
    tokens = [prompt[:, index] for index in range(prompt.shape[1])]
    logits_per_call = []
    total = prompt.shape[1] + steps
    for position in range(total - 1):
        ids = tokens[position].view(batch, 1)
        positions = torch.full((batch, 1), position, dtype=torch.int64, device=device)
        logits = step(ids, positions, keys, values, lengths)
        logits_per_call.append(logits)
        if position + 1 >= prompt.shape[1]:
            tokens.append(logits[:, 0].float().argmax(dim=-1))
    return torch.stack(tokens, dim=1), logits_per_call, (keys, values, lengths)
