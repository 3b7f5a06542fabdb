"""Hugging Face ``AttentionInterface`` hook-up: every transformers attention module
dispatches by ``config._attn_implementation``, so registering ``"megabake"`` routes prompt
passes to ``megabake::attention`` and, when per-layer KV state is passed along, one-token
decode to ``megabake::kv_attention``.

Same surface as the reference (src/megabake/fx_handler/hf_attention.py:28-187):
``megabake_attention_forward``, ``megabake_decode_attention``,
``register_transformers_attention`` and ``DecodeStep``.
"""

from __future__ import annotations

import sys
from typing import Any

import torch

from . import ops  # noqa: F401  (registers the ops)

ATTENTION_IMPLEMENTATION = "megabake"


def _needs_model_eager_path(module, dropout, softcap, kwargs) -> bool:
    return bool((dropout and module.training) or softcap is not None or kwargs.get("s_aux") is not None
                or kwargs.get("output_attentions"))


def megabake_attention_forward(module, query, key, value, attention_mask, dropout: float = 0.0,
                               scaling: float | None = None, softcap: float | None = None, **kwargs: Any):
    """transformers' attention-callback signature: ``query`` [batch, heads, q, dim],
    ``key``/``value`` [batch, kv_heads, k, dim]; returns ([batch, q, heads, dim], None)."""
    if _needs_model_eager_path(module, dropout, softcap, kwargs):
        eager = sys.modules[type(module).__module__].eager_attention_forward
        return eager(module, query, key, value, attention_mask, dropout=dropout, scaling=scaling, softcap=softcap, **kwargs)
    batch, heads, length, dim = query.shape
    scale = float(dim ** -0.5 if scaling is None else scaling)
    mask = attention_mask
    if mask is not None:
        mask = mask[:, :, :, : key.shape[-2]]
    out = torch.ops.megabake.attention(query.transpose(1, 2), key.transpose(1, 2), value.transpose(1, 2), mask, scale)
    return out.view(batch, heads, length, dim).transpose(1, 2).contiguous(), None


def megabake_decode_attention(module, query, key, value, attention_mask, dropout: float = 0.0,
                              scaling: float | None = None, softcap: float | None = None,
                              megabake_state=None, **kwargs: Any):
    """One-token decode on the layer's own cache through ``megabake::kv_attention``; without
    ``megabake_state`` this is the prompt path above."""
    if megabake_state is None:
        return megabake_attention_forward(module, query, key, value, attention_mask, dropout=dropout,
                                          scaling=scaling, softcap=softcap, **kwargs)
    if softcap is not None or kwargs.get("s_aux") is not None:
        raise NotImplementedError("decode attention with soft cap or sinks is not declared yet")
    key_cache, value_cache, valid_length = megabake_state[module.layer_idx]
    window = getattr(module, "sliding_window", None)
    if window is not None and key_cache.shape[1] > window:
        raise NotImplementedError(f"cache capacity {key_cache.shape[1]} exceeds the {window}-token sliding window")
    batch, heads, length, dim = query.shape
    if scaling is not None:
        factor = scaling * dim ** 0.5  # the op scales by dim**-0.5: fold any other scale into q
        if abs(factor - 1.0) > 1e-6:
            query = query * factor
    out = torch.ops.megabake.kv_attention(query.transpose(1, 2), key.transpose(1, 2), value.transpose(1, 2),
                                          key_cache, value_cache, valid_length)
    return out.view(batch, heads, length, dim).transpose(1, 2).contiguous(), None


def register_transformers_attention() -> str:
    """Register the ``megabake`` attention and mask implementations; returns the name."""
    from transformers import AttentionInterface
    from transformers.masking_utils import AttentionMaskInterface, eager_mask

    AttentionInterface.register(ATTENTION_IMPLEMENTATION, megabake_decode_attention)
    AttentionMaskInterface.register(ATTENTION_IMPLEMENTATION, eager_mask)  # the op takes the additive eager mask
    return ATTENTION_IMPLEMENTATION


def _pass_through_cache(layer_count: int, capacity: int):
    """A transformers ``Cache`` whose layers store nothing: the new token's key/value go
    straight to the attention call, which owns the storage."""
    from transformers.cache_utils import Cache, CacheLayerMixin

    class PassThroughLayer(CacheLayerMixin):
        is_compileable = True
        is_sliding = False

        def __init__(self):
            super().__init__()
            self.is_initialized = True

        def lazy_initialization(self, *args, **kwargs):
            return None

        def update(self, key_states, value_states, *args, **kwargs):
            return key_states, value_states

        def get_mask_sizes(self, *args, **kwargs):
            return capacity, 0

        def get_seq_length(self, *args, **kwargs):
            return 0

        def get_max_cache_shape(self, *args, **kwargs):
            return capacity

        def get_max_length(self):
            return capacity

    return Cache(layers=[PassThroughLayer() for _ in range(layer_count)])


class DecodeStep(torch.nn.Module):
    """One-token decode for a Hugging Face attention model with explicit state:
    ``forward(input_ids, position_ids, *state)`` where state holds, per layer, a key cache
    and a value cache [batch, capacity, kv_heads, head_dim] and an int32 [1] valid length
    (``state_shapes`` lists them).  Switches ``model`` to the ``megabake`` attention."""

    def __init__(self, model: torch.nn.Module, capacity: int):
        super().__init__()
        register_transformers_attention()
        model.set_attn_implementation(ATTENTION_IMPLEMENTATION)
        self.model = model
        self.capacity = capacity
        config = model.config.get_text_config(decoder=True)
        other = set(getattr(config, "layer_types", None) or ()) - {"full_attention", "sliding_attention"}
        if other:
            raise NotImplementedError(f"decode of {sorted(other)} layers is not declared yet")
        self.layer_count = config.num_hidden_layers
        self.kv_heads = config.num_key_value_heads
        self.head_dim = getattr(config, "head_dim", None) or config.hidden_size // config.num_attention_heads

    def state_shapes(self, batch: int = 1, dtype: torch.dtype = torch.bfloat16):
        cache = ((batch, self.capacity, self.kv_heads, self.head_dim), dtype)
        return [[cache, cache, ((1,), torch.int32)] for _ in range(self.layer_count)]

    def forward(self, input_ids: torch.Tensor, position_ids: torch.Tensor, *state: torch.Tensor):
        if len(state) != 3 * self.layer_count:
            raise ValueError(f"expected {3 * self.layer_count} state tensors, got {len(state)}")
        layers = tuple(tuple(state[3 * i: 3 * i + 3]) for i in range(self.layer_count))
        return self.model(
            input_ids=input_ids, position_ids=position_ids, cache_position=position_ids[0],
            past_key_values=_pass_through_cache(self.layer_count, self.capacity), use_cache=True,
            megabake_state=layers,
        ).logits
