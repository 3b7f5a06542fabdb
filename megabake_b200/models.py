"""Decode wrapper for Hugging Face Llama/Qwen2-style causal LMs with explicit KV state.

``ExplicitStateDecoder(model)(input_ids, position_ids, *state)`` runs one token per
sequence; ``state`` holds, per layer, a key cache, a value cache (both
``[batch, capacity, kv_heads, head_dim]``) and an int32 ``[1]`` valid length, either
interleaved per layer (the order ``DecodeStep`` uses) or grouped as all key caches, all
value caches, all lengths (the order of the reference's ``StatefulSmolLM`` fixture,
tests/fixtures.py:254-263).  Attention goes through ``torch.ops.megabake.kv_attention``,
so ``torch.compile(..., backend=make_backend(mode="decode"))`` sees a stateful decode graph.
"""

from __future__ import annotations

import sys

import torch

from . import ops  # noqa: F401


class ExplicitStateDecoder(torch.nn.Module):
    def __init__(self, model: torch.nn.Module, *, grouped_state: bool = False):
        super().__init__()
        self.model = model.model
        self.lm_head = model.lm_head
        self.config = model.config
        self.grouped_state = grouped_state

    def forward(self, input_ids: torch.Tensor, position_ids: torch.Tensor, *state: torch.Tensor):
        layers = self.model.layers
        count = len(layers)
        if len(state) != 3 * count:
            raise ValueError(f"expected {3 * count} state tensors, got {len(state)}")
        if self.grouped_state:
            triples = list(zip(state[:count], state[count:2 * count], state[2 * count:]))
        else:
            triples = [state[3 * i: 3 * i + 3] for i in range(count)]
        hidden = self.model.embed_tokens(input_ids)
        cosine, sine = self.model.rotary_emb(hidden, position_ids.to(torch.int64))
        for layer, (key_cache, value_cache, valid_length) in zip(layers, triples):
            attention = layer.self_attn
            rotate = sys.modules[type(attention).__module__].apply_rotary_pos_emb
            batch, length, _ = hidden.shape
            normalized = layer.input_layernorm(hidden)
            dim = attention.head_dim
            query = attention.q_proj(normalized).view(batch, length, -1, dim)
            key = attention.k_proj(normalized).view(batch, length, -1, dim)
            value = attention.v_proj(normalized).view(batch, length, -1, dim)
            query, key = rotate(query, key, cosine, sine, unsqueeze_dim=2)
            attended = torch.ops.megabake.kv_attention(query, key, value, key_cache, value_cache, valid_length)
            hidden = hidden + attention.o_proj(attended.reshape(batch, length, -1))
            hidden = hidden + layer.mlp(layer.post_attention_layernorm(hidden))
        return self.lm_head(self.model.norm(hidden))
