"""Oracle of the tensor-parallel decode step.  TEST INFRASTRUCTURE ONLY.

The reference has no multi-GPU path (src/megabake/compiler.py:1518-1528), so there is nothing of
its own to restate for the exchange; what is restated is its decode step
(tests/fixtures.py:247-312, benchmarks/stateful_models.py:73-166 of the reference, as in
``decoder_oracle.decode_step``) with the two row-sharded projections of a layer computed per
rank and combined the way the CUDA path defines it: each rank's partial sum stays in fp32, the
partial sums are added in rank order, the total is rounded to bf16 once and added to the
residual stream.  Parity of the sharded model against the unsharded reference model is a
tolerance statement (the sum order differs); parity of the CUDA path against this file is the
usual logit tolerance.
"""

from __future__ import annotations

import threading

import torch
import torch.nn.functional as F

from .decoder_oracle import _gather_rope, _linear, kv_attention, rms_norm, rotate


def rank_decode_step(config, weights, tables, input_ids, position_ids, key_caches, value_caches, valid_lengths, allreduce):
    """One rank's decode step.  ``config`` and ``weights`` are the rank's shard
    (megabake_b200.tp.shard_config / shard_weights); ``allreduce(partial_fp32)`` returns the sum
    of every rank's partial in rank order, in fp32.  Returns this rank's logits slice."""
    batch = input_ids.shape[0]
    hidden = F.embedding(input_ids, weights["model.embed_tokens.weight"])
    cosine, sine = _gather_rope(tables, position_ids.to(torch.int64))
    for layer in range(config.layers):
        prefix = f"model.layers.{layer}."
        normalized = rms_norm(hidden, weights[prefix + "input_layernorm.weight"], config.rms_eps)
        query = _linear(normalized, weights, prefix + "self_attn.q_proj").view(batch, 1, config.q_heads, config.head_dim)
        key = _linear(normalized, weights, prefix + "self_attn.k_proj").view(batch, 1, config.kv_heads, config.head_dim)
        value = _linear(normalized, weights, prefix + "self_attn.v_proj").view(batch, 1, config.kv_heads, config.head_dim)
        query = rotate(query, cosine, sine, config.rope_style)
        key = rotate(key, cosine, sine, config.rope_style)
        attended = kv_attention(query, key, value, key_caches[layer], value_caches[layer], valid_lengths[layer])
        partial = F.linear(attended.reshape(batch, 1, -1).float(), weights[prefix + "self_attn.o_proj.weight"].float())
        hidden = hidden + allreduce(partial).to(hidden.dtype)
        normalized = rms_norm(hidden, weights[prefix + "post_attention_layernorm.weight"], config.rms_eps)
        gate = F.linear(normalized, weights[prefix + "mlp.gate_proj.weight"])
        up = F.linear(normalized, weights[prefix + "mlp.up_proj.weight"])
        partial = F.linear((F.silu(gate) * up).float(), weights[prefix + "mlp.down_proj.weight"].float())
        hidden = hidden + allreduce(partial).to(hidden.dtype)
    final = rms_norm(hidden, weights["model.norm.weight"], config.rms_eps)
    return F.linear(final, weights["lm_head.weight"])


class ThreadedGroup:
    """All ranks of a group in one process, one thread each: ``allreduce`` meets at a barrier and
    adds the partial sums in rank order."""

    def __init__(self, size: int):
        self.size = size
        self.barrier = threading.Barrier(size)
        self.slots: list = [None] * size

    def allreduce_for(self, rank: int):
        def allreduce(partial: torch.Tensor) -> torch.Tensor:
            self.slots[rank] = partial
            self.barrier.wait()
            total = self.slots[0].clone()
            for other in range(1, self.size):
                total = total + self.slots[other]
            self.barrier.wait()  # nobody overwrites a slot before everyone has read it
            return total
        return allreduce

    def run(self, function):
        """``function(rank, allreduce)`` on every rank; returns the results in rank order."""
        results: list = [None] * self.size
        errors: list = []

        def work(rank):
            try:
                results[rank] = function(rank, self.allreduce_for(rank))
            except BaseException as error:  # noqa: BLE001 - re-raised below
                errors.append(error)
                self.barrier.abort()

        threads = [threading.Thread(target=work, args=(rank,)) for rank in range(self.size)]
        for thread in threads:
            thread.start()
        for thread in threads:
            thread.join()
        if errors:
            raise errors[0]
        return results


def group_decode_step(config, size, shards, tables, input_ids, position_ids, states):
    """The whole group in this process.  ``config`` is the rank shape, ``shards[r]`` rank r's
    weights, ``states[r]`` its (key caches, value caches, lengths).  Returns logits [batch, 1, vocab]."""
    group = ThreadedGroup(size)
    with torch.no_grad():
        slices = group.run(lambda rank, allreduce: rank_decode_step(
            config, shards[rank], tables, input_ids, position_ids, *states[rank], allreduce))
    return torch.cat(slices, dim=-1)
