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
    """Explicit-state single-token decode around a Hugging Face causal LM.

    Call it as ``step(input_ids[B, 1], position_ids[B, 1], *state)``.  ``state`` is flat and
    interleaved per layer: key cache, value cache (both ``[B, capacity, kv_heads, head_dim]``),
    valid length (int32 ``[1]``); ``state_shapes`` describes it.  The wrapped model is switched to
    the ``megabake`` attention, whose decode branch hands each layer's triple to
    ``megabake::kv_attention``.  Same calling convention as the reference's ``DecodeStep``
    (src/megabake/fx_handler/hf_attention.py:150-187); unlike it, the stand-in cache object also
    answers the queries transformers 5.5 makes (``get_max_cache_shape``)."""

    _SUPPORTED_LAYER_KINDS = frozenset({"full_attention", "sliding_attention"})

    def __init__(self, model: torch.nn.Module, capacity: int):
        super().__init__()
        text = model.config.get_text_config(decoder=True)
        kinds = set(getattr(text, "layer_types", None) or ())
        if not kinds <= self._SUPPORTED_LAYER_KINDS:
            raise NotImplementedError(
                f"decode of {sorted(kinds - self._SUPPORTED_LAYER_KINDS)} layers is not declared yet")
        self.capacity = int(capacity)
        self.layer_count = int(text.num_hidden_layers)
        self.kv_heads = int(text.num_key_value_heads)
        self.head_dim = int(getattr(text, "head_dim", None) or text.hidden_size // text.num_attention_heads)
        register_transformers_attention()
        model.set_attn_implementation(ATTENTION_IMPLEMENTATION)
        self.model = model

    def state_shapes(self, batch: int = 1, dtype: torch.dtype = torch.bfloat16):
        """Per layer: [(key cache shape, dtype), (value cache shape, dtype), ((1,), int32)]."""
        cache_shape = (batch, self.capacity, self.kv_heads, self.head_dim)
        return [[(cache_shape, dtype), (cache_shape, dtype), ((1,), torch.int32)] for _ in range(self.layer_count)]

    def _per_layer(self, state: tuple[torch.Tensor, ...]):
        wanted = 3 * self.layer_count
        if len(state) != wanted:
            raise ValueError(f"expected {wanted} state tensors, got {len(state)}")
        return tuple(zip(state[0::3], state[1::3], state[2::3]))

    def forward(self, input_ids: torch.Tensor, position_ids: torch.Tensor, *state: torch.Tensor):
        triples = self._per_layer(state)
        stand_in = _pass_through_cache(self.layer_count, self.capacity)
        result = self.model(input_ids=input_ids, position_ids=position_ids, cache_position=position_ids[0],
                            past_key_values=stand_in, use_cache=True, megabake_state=triples)
        return result.logits
