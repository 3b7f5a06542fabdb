"""Tensor-parallel decode over the GPUs of one node, one process per GPU.

The reference is single-device (src/megabake/compiler.py:1518-1528 rejects inputs on more than
one device); the benchmark's tensor-parallel configuration (Llama-3-8B shape at 2, 4 and 8 GPUs)
is new work.  Megatron-style sharding of one decoder layer:

* q/k/v are sharded by heads (output rows), gate/up by output rows: each rank computes its heads
  and its slice of the MLP from the whole, replicated residual stream; each rank owns the cache
  of its KV heads only;
* o_proj and down_proj are sharded by input columns: each rank holds a partial sum of the whole
  hidden vector, and the ranks all-reduce it.  The all-reduce runs inside the persistent kernel
  (``tp_allreduce`` in csrc/decoder_kernel.cuh): fp32 partial sums are stored into every rank's
  exchange buffer over NVLink, stamped flags say they are there, and every rank adds them in
  rank order, so the residual stream stays bit-identical on all ranks;
* the lm_head is sharded by vocabulary rows: a rank returns the logits of its slice, and
  ``gather_logits`` assembles them with one NCCL all-gather (the only library collective on the
  path; the embedding table is replicated, it is a row gather).

``torch.distributed`` is plumbing here: it carries the CUDA IPC handles of the exchange buffers
at start-up, the barrier after binding, and the final all-gather of logits.
"""

from __future__ import annotations

import ctypes
from dataclasses import replace
from typing import Mapping, Sequence

import torch

from . import _native
from .runtime import DecoderKernel
from .synth import DecoderConfig


def shard_config(config: DecoderConfig, size: int) -> DecoderConfig:
    """The shape one rank of ``size`` runs: its heads, its MLP columns, its vocabulary rows."""
    for what, value in (("q_heads", config.q_heads), ("kv_heads", config.kv_heads),
                        ("intermediate", config.intermediate), ("vocab", config.vocab)):
        if value % size:
            raise ValueError(f"{what} = {value} does not divide over {size} ranks")
    if (config.intermediate // size) % 64 or (config.vocab // size) % 8:
        raise ValueError("a rank's MLP slice must be a multiple of 64 columns and its vocabulary slice of 8 rows")
    return replace(config, q_heads=config.q_heads // size, kv_heads=config.kv_heads // size,
                   intermediate=config.intermediate // size, vocab=config.vocab // size, tied=False,
                   name=f"{config.name}-tp{size}")


def shard_weights(config: DecoderConfig, weights: Mapping[str, torch.Tensor], rank: int, size: int) -> dict[str, torch.Tensor]:
    """Rank ``rank``'s slice of a full state dict (contiguous copies; norms and the embedding whole)."""
    def rows(tensor, count):
        part = count // size
        return tensor[rank * part:(rank + 1) * part].contiguous()

    def columns(tensor, count):
        part = count // size
        return tensor[:, rank * part:(rank + 1) * part].contiguous()

    out: dict[str, torch.Tensor] = {
        "model.embed_tokens.weight": weights["model.embed_tokens.weight"],
        "model.norm.weight": weights["model.norm.weight"],
        "lm_head.weight": rows(weights["lm_head.weight"], config.vocab),
    }
    for layer in range(config.layers):
        prefix = f"model.layers.{layer}."
        out[prefix + "input_layernorm.weight"] = weights[prefix + "input_layernorm.weight"]
        out[prefix + "post_attention_layernorm.weight"] = weights[prefix + "post_attention_layernorm.weight"]
        for proj, count in (("q", config.q_size), ("k", config.kv_size), ("v", config.kv_size)):
            out[prefix + f"self_attn.{proj}_proj.weight"] = rows(weights[prefix + f"self_attn.{proj}_proj.weight"], count)
            bias = weights.get(prefix + f"self_attn.{proj}_proj.bias")
            if bias is not None:
                out[prefix + f"self_attn.{proj}_proj.bias"] = rows(bias, count)
        out[prefix + "self_attn.o_proj.weight"] = columns(weights[prefix + "self_attn.o_proj.weight"], config.q_size)
        out[prefix + "mlp.gate_proj.weight"] = rows(weights[prefix + "mlp.gate_proj.weight"], config.intermediate)
        out[prefix + "mlp.up_proj.weight"] = rows(weights[prefix + "mlp.up_proj.weight"], config.intermediate)
        out[prefix + "mlp.down_proj.weight"] = columns(weights[prefix + "mlp.down_proj.weight"], config.intermediate)
    return out


class ExchangeBuffers:
    """This rank's exchange buffer and its peers', addressed from this process.

    ``ExchangeBuffers.local(...)`` serves a single process that addresses every rank's buffer
    itself (tests with a stand-in peer); ``ExchangeBuffers.over_ipc(...)`` exchanges CUDA IPC
    handles through ``torch.distributed`` and opens the peers' buffers."""

    def __init__(self, pointers: Sequence[int], nbytes: int, keep: list, opened: list):
        self.pointers = list(pointers)
        self.nbytes = nbytes
        self._keep = keep        # tensors that own memory
        self._opened = opened    # IPC base pointers to close

    @staticmethod
    def allocate(nbytes: int, device: torch.device) -> torch.Tensor:
        # IPC shares whole allocations; ask for at least 2 MiB so the caching allocator gives this
        # buffer a block of its own rather than a slice of its small-block pool.
        tensor = torch.zeros(max(nbytes + 256, 2 << 20), dtype=torch.uint8, device=device)
        return tensor

    @classmethod
    def local(cls, nbytes: int, size: int, device: torch.device) -> "ExchangeBuffers":
        tensors = [cls.allocate(nbytes, device) for _ in range(size)]
        pointers = [(t.data_ptr() + 255) // 256 * 256 for t in tensors]
        return cls(pointers, nbytes, tensors, [])

    @classmethod
    def over_ipc(cls, nbytes: int, rank: int, size: int, device: torch.device, group=None) -> "ExchangeBuffers":
        import torch.distributed as dist

        lib = _native.load()
        mine = cls.allocate(nbytes, device)
        base = (mine.data_ptr() + 255) // 256 * 256
        torch.cuda.synchronize(device)
        handle = _native.MkIpcHandle()
        _native.check("mk_ipc_export", lib.mk_ipc_export(ctypes.c_void_p(base), ctypes.byref(handle)))
        gathered: list = [None] * size
        dist.all_gather_object(gathered, bytes(handle), group=group)
        pointers, opened = [], []
        for peer, blob in enumerate(gathered):
            if peer == rank:
                pointers.append(base)
                continue
            theirs = _native.MkIpcHandle.from_buffer_copy(blob)
            pointer, ipc_base = ctypes.c_void_p(), ctypes.c_void_p()
            _native.check("mk_ipc_open", lib.mk_ipc_open(ctypes.byref(theirs), ctypes.byref(pointer), ctypes.byref(ipc_base)))
            pointers.append(pointer.value)
            opened.append(ipc_base.value)
        return cls(pointers, nbytes, [mine], opened)

    def close(self) -> None:
        lib = _native.load()
        for base in self._opened:
            lib.mk_ipc_close(ctypes.c_void_p(base))
        self._opened = []


class TensorParallelDecoder:
    """One rank of a tensor-parallel decoder: a ``DecoderKernel`` on this rank's shard whose
    o_proj/down_proj all-reduce runs inside the kernel over the peers' exchange buffers.

    ``weights`` is this rank's shard (``shard_weights``); ``config`` the full model's shape.
    Every rank calls ``decode`` with the same ids and positions; the caches hold this rank's KV
    heads: ``[batch, capacity, kv_heads / size, head_dim]``."""

    def __init__(self, config: DecoderConfig, weights: Mapping[str, torch.Tensor], *, rank: int, size: int,
                 max_tokens: int, max_positions: int, device, exchange: ExchangeBuffers | None = None, group=None,
                 tables=None) -> None:
        self.full_config = config
        self.rank, self.size = rank, size
        self.group = group
        self.config = shard_config(config, size)
        self.device = torch.device(device)
        self.kernel = DecoderKernel(self.config, weights, max_tokens=max_tokens, max_positions=max_positions,
                                    device=self.device, engine="tcgen05", tables=tables,
                                    tensor_parallel=(rank, size, config.vocab))
        lib = self.kernel.lib
        nbytes = lib.mk_tp_exchange_bytes(ctypes.byref(self.kernel._cfg))
        if exchange is None:
            exchange = ExchangeBuffers.over_ipc(nbytes, rank, size, self.device, group)
        self.exchange = exchange
        pointers = (ctypes.c_void_p * size)(*exchange.pointers)
        with torch.cuda.device(self.device):
            self.kernel._call("mk_tp_bind", lib.mk_tp_bind(self.kernel._handle, pointers, exchange.nbytes, self.kernel._stream()))
            torch.cuda.synchronize(self.device)
        if group is not None or (exchange._opened and size > 1):
            import torch.distributed as dist

            dist.barrier(group=group)  # every rank has cleared its flags before anyone launches

    def decode(self, input_ids, position_ids, key_caches, value_caches, valid_lengths) -> torch.Tensor:
        """One token per sequence on every rank; returns this rank's logits slice [batch, 1, vocab / size]."""
        return self.kernel.decode(input_ids, position_ids, key_caches, value_caches, valid_lengths)

    def gather_logits(self, shard: torch.Tensor) -> torch.Tensor:
        """All ranks' vocabulary slices, in rank order: [batch, 1, vocab]."""
        import torch.distributed as dist

        parts = [torch.empty_like(shard) for _ in range(self.size)]
        dist.all_gather(parts, shard.contiguous(), group=self.group)
        return torch.cat(parts, dim=-1)

    def check(self) -> None:
        self.kernel.check()

    def status(self) -> dict:
        return self.kernel.status()

    def close(self) -> None:
        self.kernel.close()
        self.exchange.close()
