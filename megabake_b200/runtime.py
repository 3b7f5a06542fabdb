"""Launch state for one decoder on one GPU: the Python face of the C ABI.

Mirrors what the reference's ``bind_callable`` / ``_RuntimeState`` do around its
kernel (src/megabake/compiler.py:922-1103, 1877-2668): the caller owns weights,
KV caches, valid lengths and token ids; the runtime owns the workspace; outputs
are freshly allocated on every call; one lock serialises bind + launch; launches
go to the current CUDA stream and return without synchronising.
"""

from __future__ import annotations

import ctypes
import threading
from typing import Mapping, Sequence

import torch

from . import _native
from ._native import MkConfig, MkLayerWeights, MkStatusInfo, MkWeights, NativeError
from .diagnostics import CompilerDiagnostic, CompilerError
from .synth import DecoderConfig, rope_tables


def _ptr(tensor: torch.Tensor | None) -> int | None:
    return None if tensor is None else tensor.data_ptr()


def _require(tensor: torch.Tensor, name: str, *, dtype, device, shape=None) -> None:
    if not isinstance(tensor, torch.Tensor):
        raise CompilerError(CompilerDiagnostic("input-binding", f"{name} is not a tensor"))
    if tensor.dtype != dtype or tensor.device != device or not tensor.is_contiguous():
        raise CompilerError(CompilerDiagnostic(
            "input-binding",
            f"{name} must be a contiguous {dtype} tensor on {device}; got {tensor.dtype} on {tensor.device} "
            f"with strides {tuple(tensor.stride())}",
        ))
    if shape is not None and tuple(tensor.shape) != tuple(shape):
        raise CompilerError(CompilerDiagnostic(
            "input-binding", f"{name} has shape {tuple(tensor.shape)}, expected {tuple(shape)}"))


EVENT_NAMES = {1: "phase_enter", 2: "operand_staged", 3: "first_accumulator", 4: "phase_done",
               5: "barrier_done", 6: "attention_done", 7: "attention_inputs", 8: "attention_scores",
               9: "attention_statistics", 10: "attention_values", 11: "attention_partial", 12: "first_copy"}


def decode_trace(buffer: torch.Tensor):
    """Split a trace buffer into (codes, nanoseconds) int64 arrays [ctas, events]; code 0 = unused slot."""
    raw = buffer.cpu()
    codes = (raw >> 56) & 0xFF
    times = raw & ((1 << 56) - 1)
    return codes, times


class DecoderKernel:
    """One persistent-kernel decoder bound to a set of weights.

    ``weights`` uses Hugging Face parameter names (``model.layers.N.self_attn.q_proj.weight`` ...).
    ``max_tokens`` bounds batch (decode) or batch x sequence (prefill) per launch.
    """

    def __init__(
        self,
        config: DecoderConfig,
        weights: Mapping[str, torch.Tensor],
        *,
        max_tokens: int = 16,
        max_positions: int = 2048,
        device: str | torch.device = "cuda:0",
        engine: str = "auto",
        sm_limit: int = 0,
        tables: tuple[torch.Tensor, torch.Tensor] | None = None,
        tensor_parallel: tuple[int, int, int] | None = None,
    ) -> None:
        """``tensor_parallel`` = (rank, size, rows of the replicated embedding table) makes this
        kernel one rank of a group: ``config`` is then the rank's shard (see megabake_b200/tp.py)."""
        self.config = config
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise CompilerError(CompilerDiagnostic("runtime-binding", "the megakernel runs on CUDA devices only"))
        if self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())
        self.lib = _native.load()
        self.max_tokens = int(max_tokens)
        self.max_positions = int(max_positions)
        self._lock = threading.Lock()
        self._cfg = MkConfig(
            hidden=config.hidden, layers=config.layers, q_heads=config.q_heads, kv_heads=config.kv_heads,
            head_dim=config.head_dim, intermediate=config.intermediate, vocab=config.vocab,
            rms_eps=config.rms_eps, qkv_bias=int(config.qkv_bias),
            rope_style=_native.ROPE_STYLES[config.rope_style], max_tokens=self.max_tokens,
            max_positions=self.max_positions, engine=_native.ENGINES[engine], sm_limit=int(sm_limit),
            tp_size=0, tp_rank=0, embed_rows=0,
        )
        if tensor_parallel is not None:
            self._cfg.tp_rank, self._cfg.tp_size, self._cfg.embed_rows = (int(v) for v in tensor_parallel)
        with torch.cuda.device(self.device):
            size = self.lib.mk_workspace_bytes(ctypes.byref(self._cfg), self.device.index)
            if size == 0:
                raise self._compiler_error("plan-search", NativeError(
                    "mk_workspace_bytes", _native.MK_ERR_UNSUPPORTED, self.lib.mk_last_error().decode()))
            self.workspace = torch.empty(size + 256, dtype=torch.uint8, device=self.device)
            base = (self.workspace.data_ptr() + 255) // 256 * 256
            handle = ctypes.c_void_p()
            self._call("mk_create", self.lib.mk_create(
                ctypes.byref(self._cfg), base, size, self.device.index, self._stream(), ctypes.byref(handle)))
        self._handle = handle
        self._bound_ptrs: tuple[int, ...] | None = None
        self._state_key = None
        self._state_arrays = None
        self._install_status_mirror()
        if tables is None:
            tables = rope_tables(config, self.max_positions, device=self.device)
        self.tables = tables
        self.bind(weights)

    # ------------------------------------------------------------------ helpers
    def _stream(self) -> int:
        return torch.cuda.current_stream(self.device).cuda_stream

    def _compiler_error(self, stage: str, error: NativeError) -> CompilerError:
        return CompilerError(CompilerDiagnostic(stage, str(error)), safe_for_fallback=False)

    def _call(self, function: str, code: int, stage: str = "runtime-binding") -> None:
        if code == _native.MK_OK:
            return
        error = NativeError(function, code, self.lib.mk_last_error().decode(errors="replace"))
        if code == _native.MK_ERR_UNSUPPORTED:
            raise self._compiler_error("plan-search", error)
        if code in (_native.MK_ERR_ALIGNMENT, _native.MK_ERR_INVALID, _native.MK_ERR_UNBOUND):
            raise self._compiler_error(stage, error)
        raise error

    def _install_status_mirror(self) -> None:
        """One pinned int32 the kernel also writes its status to: `raise_if_failed` reads it
        without synchronising, so a launch that was refused (full cache, bad id) or gave up a
        wait is reported at the caller's next call instead of handing out NaN silently
        (the reference raises: src/megabake/lowering.py:229, src/megabake/compiler.py:2690)."""
        self._host_step_logits = None
        self._mirror = torch.zeros(1, dtype=torch.int32).pin_memory()
        with torch.cuda.device(self.device):
            self._call("mk_set_status_mirror", self.lib.mk_set_status_mirror(self._handle, self._mirror.data_ptr()))

    def raise_if_failed(self) -> None:
        """Non-blocking: raise what an earlier launch reported, if anything."""
        if int(self._mirror[0]) != 0:
            self.check()

    def close(self) -> None:
        handle, self._handle = getattr(self, "_handle", None), None
        if handle:
            self.lib.mk_destroy(handle)

    def __del__(self):  # pragma: no cover - interpreter shutdown order
        try:
            self.close()
        except Exception:
            pass

    # ------------------------------------------------------------------ weights
    def bind(self, weights: Mapping[str, torch.Tensor]) -> None:
        """Bind every parameter by pointer (again after the caller replaces a tensor)."""
        config = self.config
        names = ["model.embed_tokens.weight", "model.norm.weight", "lm_head.weight"]
        per_layer = [
            "input_layernorm.weight", "self_attn.q_proj.weight", "self_attn.k_proj.weight",
            "self_attn.v_proj.weight", "self_attn.o_proj.weight", "post_attention_layernorm.weight",
            "mlp.gate_proj.weight", "mlp.up_proj.weight", "mlp.down_proj.weight",
        ]
        if config.qkv_bias:
            per_layer += ["self_attn.q_proj.bias", "self_attn.k_proj.bias", "self_attn.v_proj.bias"]
        for layer in range(config.layers):
            names += [f"model.layers.{layer}.{name}" for name in per_layer]
        kept = {}
        for name in names:
            tensor = weights.get(name)
            if tensor is None and name == "lm_head.weight" and config.tied:
                tensor = weights["model.embed_tokens.weight"]
            if tensor is None:
                raise CompilerError(CompilerDiagnostic("runtime-binding", f"missing parameter {name}"))
            _require(tensor, name, dtype=torch.bfloat16, device=self.device)
            kept[name] = tensor
        cosine, sine = self.tables
        _require(cosine, "rope cos table", dtype=torch.bfloat16, device=self.device,
                 shape=(self.max_positions, config.head_dim))
        _require(sine, "rope sin table", dtype=torch.bfloat16, device=self.device,
                 shape=(self.max_positions, config.head_dim))
        layers = (MkLayerWeights * config.layers)()
        for index in range(config.layers):
            prefix = f"model.layers.{index}."
            entry = layers[index]
            entry.input_norm = _ptr(kept[prefix + "input_layernorm.weight"])
            entry.q = _ptr(kept[prefix + "self_attn.q_proj.weight"])
            entry.k = _ptr(kept[prefix + "self_attn.k_proj.weight"])
            entry.v = _ptr(kept[prefix + "self_attn.v_proj.weight"])
            entry.q_bias = _ptr(kept.get(prefix + "self_attn.q_proj.bias"))
            entry.k_bias = _ptr(kept.get(prefix + "self_attn.k_proj.bias"))
            entry.v_bias = _ptr(kept.get(prefix + "self_attn.v_proj.bias"))
            entry.o = _ptr(kept[prefix + "self_attn.o_proj.weight"])
            entry.post_norm = _ptr(kept[prefix + "post_attention_layernorm.weight"])
            entry.gate = _ptr(kept[prefix + "mlp.gate_proj.weight"])
            entry.up = _ptr(kept[prefix + "mlp.up_proj.weight"])
            entry.down = _ptr(kept[prefix + "mlp.down_proj.weight"])
        packed = MkWeights(
            embed=_ptr(kept["model.embed_tokens.weight"]), final_norm=_ptr(kept["model.norm.weight"]),
            lm_head=_ptr(kept["lm_head.weight"]), rope_cos=_ptr(cosine), rope_sin=_ptr(sine), layers=layers,
        )
        with self._lock, torch.cuda.device(self.device):
            self._call("mk_bind_weights", self.lib.mk_bind_weights(self._handle, ctypes.byref(packed), self._stream()))
        self._weights = kept  # keep the tensors alive while their pointers are bound
        self._bound_ptrs = tuple(t.data_ptr() for t in kept.values())

    def rebind_if_changed(self, weights: Mapping[str, torch.Tensor]) -> bool:
        """Re-bind when any parameter tensor was replaced; returns whether it did."""
        pointers = tuple(weights[name].data_ptr() if name in weights else self._weights[name].data_ptr()
                         for name in self._weights)
        if pointers == self._bound_ptrs:
            return False
        self.bind(weights)
        return True

    # ------------------------------------------------------------------ launches
    def decode(
        self,
        input_ids: torch.Tensor,
        position_ids: torch.Tensor,
        key_caches: Sequence[torch.Tensor],
        value_caches: Sequence[torch.Tensor],
        valid_lengths: Sequence[torch.Tensor],
    ) -> torch.Tensor:
        """One token per sequence: appends to the caches, advances the lengths,
        returns logits [batch, 1, vocab].  Same contract as the reference's decode
        wrappers (tests/fixtures.py:247-312)."""
        config = self.config
        batch = input_ids.shape[0]
        if input_ids.dim() != 2 or input_ids.shape[1] != 1:
            raise RuntimeError("megabake kv_attention supports one-token decode only")
        _require(input_ids, "input_ids", dtype=torch.int64, device=self.device, shape=(batch, 1))
        _require(position_ids, "position_ids", dtype=torch.int64, device=self.device, shape=(batch, 1))
        keys, values, lengths, capacity = self._checked_state(batch, key_caches, value_caches, valid_lengths)
        self.raise_if_failed()
        logits = torch.empty((batch, 1, config.vocab), dtype=torch.bfloat16, device=self.device)
        with self._lock, torch.cuda.device(self.device):
            self._call("mk_decode", self.lib.mk_decode(
                self._handle, input_ids.data_ptr(), position_ids.data_ptr(), batch, keys, values, lengths,
                capacity, logits.data_ptr(), self._stream()), stage="input-binding")
        return logits

    def decode_ragged(self, input_ids, position_ids, key_caches, value_caches, valid_lengths) -> torch.Tensor:
        """``decode`` for sequences of different lengths: every ``valid_lengths[layer]`` is int32
        ``[batch]`` (one filled-position count per sequence), ``position_ids[b]`` that sequence's
        position.  Beyond the reference's contract of one length per batch
        (src/megabake/lowering.py:160-190)."""
        config = self.config
        batch = input_ids.shape[0]
        _require(input_ids, "input_ids", dtype=torch.int64, device=self.device, shape=(batch, 1))
        _require(position_ids, "position_ids", dtype=torch.int64, device=self.device, shape=(batch, 1))
        keys, values, lengths, capacity = self._checked_state(batch, key_caches, value_caches, valid_lengths, per_sequence=True)
        self.raise_if_failed()
        logits = torch.empty((batch, 1, config.vocab), dtype=torch.bfloat16, device=self.device)
        with self._lock, torch.cuda.device(self.device):
            self._call("mk_decode_ragged", self.lib.mk_decode_ragged(
                self._handle, input_ids.data_ptr(), position_ids.data_ptr(), batch, keys, values, lengths,
                capacity, logits.data_ptr(), self._stream()), stage="input-binding")
        return logits

    def _checked_state(self, batch, key_caches, value_caches, valid_lengths, per_sequence: bool = False):
        """Pointer arrays of the caller's state; shapes and dtypes are validated whenever any
        state tensor or the batch differs from the last call's."""
        config = self.config
        if not (len(key_caches) == len(value_caches) == len(valid_lengths) == config.layers):
            raise ValueError(f"expected {3 * config.layers} state tensors, got "
                             f"{len(key_caches) + len(value_caches) + len(valid_lengths)}")
        capacity = key_caches[0].shape[1]
        key = (batch, per_sequence) + tuple(t.data_ptr() for group in (key_caches, value_caches, valid_lengths) for t in group)
        if key != self._state_key:
            cache_shape = (batch, capacity, config.kv_heads, config.head_dim)
            for layer in range(config.layers):
                _require(key_caches[layer], f"key cache {layer}", dtype=torch.bfloat16, device=self.device, shape=cache_shape)
                _require(value_caches[layer], f"value cache {layer}", dtype=torch.bfloat16, device=self.device, shape=cache_shape)
                _require(valid_lengths[layer], f"valid length {layer}", dtype=torch.int32, device=self.device,
                         shape=(batch,) if per_sequence else (1,))
            count = config.layers
            self._state_arrays = tuple((ctypes.c_void_p * count)(*[t.data_ptr() for t in group])
                                       for group in (key_caches, value_caches, valid_lengths))
            self._state_key = key
        return (*self._state_arrays, capacity)

    def decode_steps(
        self,
        input_ids: torch.Tensor,
        position_ids: torch.Tensor,
        key_caches: Sequence[torch.Tensor],
        value_caches: Sequence[torch.Tensor],
        valid_lengths: Sequence[torch.Tensor],
        steps: int,
        return_logits: bool = False,
    ):
        """``steps`` greedy decode steps with no host round trip in between: the kernel picks each
        token (``torch.argmax`` semantics on the bf16 logits), feeds it back as the next id and
        advances the position.  ``input_ids`` and ``position_ids`` ([batch, 1] int64) are updated in
        place and hold the next step's inputs afterwards.  Returns the tokens [batch, steps]
        (and the last step's logits [batch, 1, vocab] if asked).  No synchronisation."""
        config = self.config
        batch = input_ids.shape[0]
        _require(input_ids, "input_ids", dtype=torch.int64, device=self.device, shape=(batch, 1))
        _require(position_ids, "position_ids", dtype=torch.int64, device=self.device, shape=(batch, 1))
        keys, values, lengths, capacity = self._checked_state(batch, key_caches, value_caches, valid_lengths)
        self.raise_if_failed()
        tokens = torch.empty((steps, batch), dtype=torch.int64, device=self.device)
        logits = torch.empty((batch, 1, config.vocab), dtype=torch.bfloat16, device=self.device)
        with self._lock, torch.cuda.device(self.device):
            self._call("mk_decode_steps", self.lib.mk_decode_steps(
                self._handle, input_ids.data_ptr(), position_ids.data_ptr(), batch, keys, values, lengths,
                capacity, int(steps), tokens.data_ptr(), logits.data_ptr(), self._stream()), stage="input-binding")
        tokens = tokens.transpose(0, 1)
        return (tokens, logits) if return_logits else tokens

    def step_from_host(
        self,
        host_ids: torch.Tensor,
        host_positions: torch.Tensor,
        key_caches: Sequence[torch.Tensor],
        value_caches: Sequence[torch.Tensor],
        valid_lengths: Sequence[torch.Tensor],
        host_tokens: torch.Tensor,
    ) -> torch.Tensor:
        """One greedy step whose inputs and result live in host memory: ``host_ids`` and
        ``host_positions`` ([batch, 1] int64, pinned) go up, the kernel samples on the device, the
        chosen tokens land in ``host_tokens`` ([batch, 1] int64, pinned), and the stream is
        synchronised: one native call.  Returns ``host_tokens``."""
        batch = host_ids.shape[0]
        for name, tensor in (("host_ids", host_ids), ("host_positions", host_positions), ("host_tokens", host_tokens)):
            if tensor.device.type != "cpu" or tensor.dtype != torch.int64 or tuple(tensor.shape) != (batch, 1) \
                    or not tensor.is_contiguous():
                raise CompilerError(CompilerDiagnostic(
                    "input-binding", f"{name} must be a contiguous CPU int64 tensor of shape ({batch}, 1)"))
        keys, values, lengths, capacity = self._checked_state(batch, key_caches, value_caches, valid_lengths)
        self.raise_if_failed()
        if self._host_step_logits is None or self._host_step_logits.shape[0] != batch:
            self._host_step_logits = torch.empty((batch, 1, self.config.vocab), dtype=torch.bfloat16, device=self.device)
        with self._lock, torch.cuda.device(self.device):
            self._call("mk_decode_step_host", self.lib.mk_decode_step_host(
                self._handle, host_ids.data_ptr(), host_positions.data_ptr(), batch, keys, values, lengths, capacity,
                self._host_step_logits.data_ptr(), host_tokens.data_ptr(), self._stream()), stage="input-binding")
        self.raise_if_failed()
        return host_tokens

    def prefill(self, input_ids: torch.Tensor, position_ids: torch.Tensor | None = None,
                mask: torch.Tensor | None = None) -> torch.Tensor:
        """Stateless prompt pass: logits [batch, sequence, vocab]; ``mask`` is the
        additive bf16 [batch, 1, sequence, sequence] mask, None means causal."""
        batch, sequence = input_ids.shape
        _require(input_ids, "input_ids", dtype=torch.int64, device=self.device)
        if position_ids is None:
            position_ids = torch.arange(sequence, device=self.device).expand(batch, sequence).contiguous()
        _require(position_ids, "position_ids", dtype=torch.int64, device=self.device, shape=(batch, sequence))
        if mask is not None:
            _require(mask, "attention mask", dtype=torch.bfloat16, device=self.device, shape=(batch, 1, sequence, sequence))
        self.raise_if_failed()
        logits = torch.empty((batch, sequence, self.config.vocab), dtype=torch.bfloat16, device=self.device)
        with self._lock, torch.cuda.device(self.device):
            self._call("mk_prefill", self.lib.mk_prefill(
                self._handle, input_ids.data_ptr(), position_ids.data_ptr(), _ptr(mask), batch, sequence,
                logits.data_ptr(), self._stream()), stage="input-binding")
        return logits

    def linear(self, source: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
        """``source @ weight.T (+ bias)`` through the projection engine (bf16, fp32 accumulate)."""
        rows, k = source.shape
        n = weight.shape[0]
        _require(source, "source", dtype=torch.bfloat16, device=self.device)
        _require(weight, "weight", dtype=torch.bfloat16, device=self.device, shape=(n, k))
        if bias is not None:
            _require(bias, "bias", dtype=torch.bfloat16, device=self.device, shape=(n,))
        out = torch.empty((rows, n), dtype=torch.bfloat16, device=self.device)
        with self._lock, torch.cuda.device(self.device):
            self._call("mk_linear", self.lib.mk_linear(
                self._handle, source.data_ptr(), weight.data_ptr(), _ptr(bias), out.data_ptr(), rows, n, k,
                self._stream()))
        return out

    def kv_attention(self, source, key, value, key_cache, value_cache, valid_length) -> torch.Tensor:
        """``megabake::kv_attention`` (reference src/megabake/lowering.py:211-247) on the GPU."""
        batch, length, heads, dim = source.shape
        if length != 1:
            raise RuntimeError("megabake kv_attention supports one-token decode only")
        for name, tensor in (("source", source), ("key", key), ("value", value), ("key_cache", key_cache), ("value_cache", value_cache)):
            _require(tensor, name, dtype=torch.bfloat16, device=self.device)
        _require(valid_length, "valid_length", dtype=torch.int32, device=self.device, shape=(1,))
        self.raise_if_failed()
        out = torch.empty((batch * heads, 1, dim), dtype=torch.bfloat16, device=self.device)
        with self._lock, torch.cuda.device(self.device):
            self._call("mk_kv_attention", self.lib.mk_kv_attention(
                self._handle, source.data_ptr(), key.data_ptr(), value.data_ptr(), key_cache.data_ptr(),
                value_cache.data_ptr(), valid_length.data_ptr(), batch, key_cache.shape[1], out.data_ptr(),
                self._stream()))
        return out

    def attention(self, query, key, value, mask, scale: float) -> torch.Tensor:
        """``megabake::attention`` (reference src/megabake/lowering.py:273-300) on the GPU."""
        batch, q_len, heads, dim = query.shape
        k_len = key.shape[1]
        for name, tensor in (("query", query), ("key", key), ("value", value)):
            _require(tensor, name, dtype=torch.bfloat16, device=self.device)
        if mask is not None:
            mask = mask.expand(batch, 1, q_len, k_len).contiguous()
            _require(mask, "mask", dtype=torch.bfloat16, device=self.device)
        out = torch.empty((batch * heads, q_len, dim), dtype=torch.bfloat16, device=self.device)
        with self._lock, torch.cuda.device(self.device):
            self._call("mk_attention", self.lib.mk_attention(
                self._handle, query.data_ptr(), key.data_ptr(), value.data_ptr(), _ptr(mask), float(scale),
                batch, q_len, k_len, out.data_ptr(), self._stream()))
        return out

    # ------------------------------------------------------------------ status
    def status(self) -> dict:
        """Synchronise and read the device status word (resets the handle's counters if it is not OK)."""
        info = MkStatusInfo()
        with self._lock, torch.cuda.device(self.device):
            code = self.lib.mk_status(self._handle, self._stream(), ctypes.byref(info))
        result = dict(status=_native.STATUS_NAMES.get(info.status, str(info.status)), where=info.where,
                      cta=info.cta, detail=info.detail, code=code)
        if code not in (_native.MK_OK, _native.MK_ERR_DEVICE_STATUS):
            self._call("mk_status", code)
        return result

    def check(self) -> None:
        """Raise if the device reported a KV overflow, a bad index or a timed-out wait."""
        result = self.status()
        if result["status"] == "KV_OVERFLOW":
            raise CompilerError(CompilerDiagnostic(
                "state-capacity", "KV cache valid length plus one token exceeds capacity"))
        if result["status"] != "OK":
            raise RuntimeError(f"megakernel device status {result}")

    def set_trace(self, events_per_cta: int = 0) -> torch.Tensor | None:
        """Turn the per-CTA event trace on (returns the int64 [ctas, events] buffer the
        next launches fill; decode with :func:`decode_trace`) or off (0)."""
        if events_per_cta <= 0:
            self._trace = None
            self._call("mk_set_trace", self.lib.mk_set_trace(self._handle, None, 0))
            return None
        ctas = self.launch_info()["ctas"]
        self._trace = torch.zeros((ctas, events_per_cta), dtype=torch.int64, device=self.device)
        self._call("mk_set_trace", self.lib.mk_set_trace(self._handle, self._trace.data_ptr(), events_per_cta))
        return self._trace

    def describe(self) -> str:
        """What this kernel will launch: CTAs, copy form, tile plan per phase table."""
        buffer = ctypes.create_string_buffer(4096)
        self._call("mk_describe", self.lib.mk_describe(self._handle, buffer, len(buffer)))
        return buffer.value.decode()

    def launch_info(self) -> dict:
        ctas, smem, launches = ctypes.c_int32(), ctypes.c_int32(), ctypes.c_int64()
        self._call("mk_launch_info", self.lib.mk_launch_info(
            self._handle, ctypes.byref(ctas), ctypes.byref(smem), ctypes.byref(launches)))
        return dict(ctas=ctas.value, smem_bytes=smem.value, launches=launches.value)


class AttentionKernels:
    """Launch state for the two attention ops alone (no decoder weights): what
    ``torch.ops.megabake.kv_attention`` / ``attention`` dispatch to for CUDA tensors."""

    _cache: dict = {}
    _cache_lock = threading.Lock()

    def __init__(self, q_heads: int, kv_heads: int, head_dim: int, max_tokens: int, device: torch.device):
        self.device = torch.device(device)
        self.lib = _native.load()
        self.max_tokens = max_tokens
        self._lock = threading.Lock()
        self._cfg = MkConfig(
            hidden=q_heads * head_dim, layers=1, q_heads=q_heads, kv_heads=kv_heads, head_dim=head_dim,
            intermediate=64, vocab=64, rms_eps=1e-5, qkv_bias=0, rope_style=0, max_tokens=max_tokens,
            max_positions=1, engine=0, sm_limit=0,
        )
        with torch.cuda.device(self.device):
            size = self.lib.mk_workspace_bytes(ctypes.byref(self._cfg), self.device.index)
            if size == 0:
                raise CompilerError(CompilerDiagnostic("plan-search", self.lib.mk_last_error().decode(errors="replace")))
            self.workspace = torch.empty(size + 256, dtype=torch.uint8, device=self.device)
            base = (self.workspace.data_ptr() + 255) // 256 * 256
            handle = ctypes.c_void_p()
            code = self.lib.mk_create(ctypes.byref(self._cfg), base, size, self.device.index,
                                      torch.cuda.current_stream(self.device).cuda_stream, ctypes.byref(handle))
            if code != _native.MK_OK:
                raise CompilerError(CompilerDiagnostic("plan-search", self.lib.mk_last_error().decode(errors="replace")))
        self._handle = handle
        self._install_status_mirror()

    @classmethod
    def for_shape(cls, q_heads: int, kv_heads: int, head_dim: int, tokens: int, device: torch.device) -> "AttentionKernels":
        device = torch.device(device)
        if device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())
        key = (q_heads, kv_heads, head_dim, device.index)
        with cls._cache_lock:
            found = cls._cache.get(key)
            if found is None or found.max_tokens < tokens:
                capacity = max(16, 1 << (max(tokens, 1) - 1).bit_length())
                found = cls(q_heads, kv_heads, head_dim, capacity, device)
                cls._cache[key] = found
        return found

    # The launches reuse DecoderKernel's methods: same handle layout, same checks.
    _stream = DecoderKernel._stream
    _call = DecoderKernel._call
    _compiler_error = DecoderKernel._compiler_error
    kv_attention = DecoderKernel.kv_attention
    attention = DecoderKernel.attention
    status = DecoderKernel.status
    check = DecoderKernel.check
    raise_if_failed = DecoderKernel.raise_if_failed
    _install_status_mirror = DecoderKernel._install_status_mirror
