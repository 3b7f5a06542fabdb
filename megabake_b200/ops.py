"""The two custom ops of the backend surface, with the reference's names, schemas and
mutation annotations (reference src/megabake/lowering.py:211-309):

    torch.ops.megabake.kv_attention(source, key, value, key_cache, value_cache, valid_length)
    torch.ops.megabake.attention(query, key, value, mask, scale)

For CUDA tensors they launch the sm_100a attention phase of the megakernel through the
C ABI (and raise if the library is missing).  For CPU tensors they run the eager
definition of the op, which is what ``compile_kernel=False`` graphs execute.
"""

from __future__ import annotations

import torch

_NAMESPACE = "megabake"


def _expand_groups(tensor: torch.Tensor, heads: int) -> torch.Tensor:
    if tensor.shape[1] == heads:
        return tensor
    return tensor.repeat_interleave(heads // tensor.shape[1], dim=1)


def _kv_attention_eager(source, key, value, key_cache, value_cache, valid_length):
    filled = int(valid_length.item())
    after = filled + 1
    if filled < 0 or after > key_cache.shape[1]:
        raise RuntimeError(f"KV cache length {filled} plus 1 exceeds capacity {key_cache.shape[1]}")
    key_cache[:, filled:after].copy_(key)
    value_cache[:, filled:after].copy_(value)
    valid_length.fill_(after)
    heads = source.shape[2]
    q = source.permute(0, 2, 1, 3)
    k = _expand_groups(key_cache[:, :after].permute(0, 2, 1, 3), heads)
    v = _expand_groups(value_cache[:, :after].permute(0, 2, 1, 3), heads)
    weights = torch.softmax((q @ k.transpose(-2, -1)).float() * source.shape[-1] ** -0.5, dim=-1).to(source.dtype)
    return (weights @ v).permute(0, 2, 1, 3).reshape(source.shape[0] * heads, 1, source.shape[3])


def _attention_eager(query, key, value, mask, scale):
    heads = query.shape[2]
    q = query.transpose(1, 2)
    k = _expand_groups(key.transpose(1, 2), heads)
    v = _expand_groups(value.transpose(1, 2), heads)
    scores = torch.matmul(q, k.transpose(2, 3)) * scale
    if mask is not None:
        scores = scores + mask
    weights = torch.softmax(scores, dim=-1, dtype=torch.float32).to(q.dtype)
    out = torch.matmul(weights, v)
    return out.reshape(-1, out.shape[2], out.shape[3])


def _gpu_kernels(heads: int, kv_heads: int, dim: int, tokens: int, device):
    from .runtime import AttentionKernels

    return AttentionKernels.for_shape(heads, kv_heads, dim, tokens, device)


def _check_layout(source, key, key_cache=None):
    if source.dtype != torch.bfloat16 and source.is_cuda:
        raise RuntimeError("megabake attention ops run in bfloat16 on CUDA")
    if source.shape[2] % key.shape[2]:
        raise RuntimeError("query heads must be a multiple of key/value heads")


@torch.library.custom_op(f"{_NAMESPACE}::kv_attention", mutates_args=("key_cache", "value_cache", "valid_length"))
def kv_attention(
    source: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
    key_cache: torch.Tensor, value_cache: torch.Tensor, valid_length: torch.Tensor,
) -> torch.Tensor:
    if source.shape[1] != 1:
        raise RuntimeError("megabake kv_attention supports one-token decode only")
    _check_layout(source, key)
    if not source.is_cuda:
        return _kv_attention_eager(source, key, value, key_cache, value_cache, valid_length)
    kernels = _gpu_kernels(source.shape[2], key.shape[2], source.shape[3], source.shape[0], source.device)
    return kernels.kv_attention(source.contiguous(), key.contiguous(), value.contiguous(), key_cache, value_cache,
                                valid_length)


@kv_attention.register_fake
def _(source, key, value, key_cache, value_cache, valid_length):
    return source.new_empty((source.shape[0] * source.shape[2], source.shape[1], source.shape[3]))


@torch.library.custom_op(f"{_NAMESPACE}::attention", mutates_args=())
def attention(
    query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, mask: torch.Tensor | None, scale: float,
) -> torch.Tensor:
    """Softmax attention with Hugging Face eager numerics: ``query`` [batch, q, heads, dim],
    ``key``/``value`` [batch, k, kv_heads, dim], additive ``mask`` broadcastable to
    [batch, heads, q, k]; returns [batch * heads, q, dim]."""
    _check_layout(query, key)
    if not query.is_cuda:
        return _attention_eager(query, key, value, mask, scale)
    batch, q_len, heads, dim = query.shape
    kernels = _gpu_kernels(heads, key.shape[2], dim, batch * q_len, query.device)
    if mask is not None:
        if mask.dim() != 4 or mask.shape[1] != 1:
            mask = mask.expand(batch, heads, q_len, key.shape[1])
            if not all(torch.equal(mask[:, :1], mask[:, h:h + 1]) for h in range(1, heads)):
                raise RuntimeError("megabake attention takes one mask per sequence, shared by its heads")
            mask = mask[:, :1]
        mask = mask.to(torch.bfloat16)
    return kernels.attention(query.contiguous(), key.contiguous(), value.contiguous(), mask, float(scale))


@attention.register_fake
def _(query, key, value, mask, scale):
    return query.new_empty((query.shape[0] * query.shape[2], query.shape[1], query.shape[3]))


KV_ATTENTION_OP = torch.ops.megabake.kv_attention.default
ATTENTION_OP = torch.ops.megabake.attention.default
