"""Seeded synthetic decoder weights and inputs that are bit-identical on every machine.

The reference draws random-init weights with ``torch.manual_seed`` and Hugging
Face's initialisers (``tests/fixtures.py:315-336`` of the reference).  Those go
through ``normal_``, whose vectorised CPU code path differs between CPU
generations and from the CUDA generator, so a golden file made on one host
would not match weights drawn on another.  Here every element is a pure
integer function of ``(seed, tensor name, flat index)``: two rounds of a 32-bit
mixing hash give eight bytes, their sum (Irwin-Hall, n=8) is centred and scaled
to the requested standard deviation with one fp32 multiply and rounded to
bf16.  Integer tensor ops behave identically on CPU and CUDA, so the same
function fills weights in place on the GPU for full-size benchmarks.
"""

from __future__ import annotations

import zlib
from dataclasses import dataclass, asdict

import torch

_MASK32 = 0xFFFFFFFF
_MIX = 0x45D9F3B  # < 2**27, so products of a 32-bit value stay below 2**63
_BYTES_STD = 209.02232416658274  # sqrt(8 * (256**2 - 1) / 12)


@dataclass(frozen=True)
class DecoderConfig:
    """Shape of a Llama/Qwen2-style decoder (the only family the kernel runs)."""

    hidden: int
    layers: int
    q_heads: int
    kv_heads: int
    head_dim: int
    intermediate: int
    vocab: int
    rms_eps: float = 1e-5
    rope_theta: float = 1e4
    qkv_bias: bool = False
    tied: bool = True
    # "half_swap": rotation written in the reference's decode fixture
    # (tests/fixtures.py:44-54: second half = x2*sin + x1*cos);
    # "hf": transformers' apply_rotary_pos_emb (second half = x2*cos + x1*sin).
    rope_style: str = "half_swap"
    # transformers keeps inv_freq as a buffer, so ``model.to(bfloat16)`` rounds it.
    inv_freq_bf16: bool = True
    name: str = "decoder"

    def to_dict(self) -> dict:
        return asdict(self)

    @property
    def q_size(self) -> int:
        return self.q_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.kv_heads * self.head_dim

    def streamed_parameters(self) -> int:
        """Parameters read once per decode step (linears, norms, biases, lm_head)."""
        per_layer = (
            self.hidden * self.q_size
            + 2 * self.hidden * self.kv_size
            + self.q_size * self.hidden
            + 3 * self.hidden * self.intermediate
            + 2 * self.hidden
        )
        if self.qkv_bias:
            per_layer += self.q_size + 2 * self.kv_size
        return self.layers * per_layer + self.hidden + self.vocab * self.hidden

    def decode_bytes(self, batch: int, context: int) -> int:
        """Algorithmic HBM bytes of one decode step: every streamed parameter once,
        the cached keys/values of ``context`` positions, and the appended row."""
        kv_row = 2 * self.layers * batch * self.kv_size * 2
        return 2 * self.streamed_parameters() + kv_row * context + kv_row


CONFIGS: dict[str, DecoderConfig] = {
    "smollm-135m": DecoderConfig(
        hidden=576, layers=30, q_heads=9, kv_heads=3, head_dim=64, intermediate=1536,
        vocab=49152, rms_eps=1e-5, rope_theta=1e4, name="smollm-135m",
    ),
    "qwen2-0.5b": DecoderConfig(
        hidden=896, layers=24, q_heads=14, kv_heads=2, head_dim=64, intermediate=4864,
        vocab=151936, rms_eps=1e-6, rope_theta=1e6, qkv_bias=True, rope_style="hf",
        name="qwen2-0.5b",
    ),
    "smollm-1.7b": DecoderConfig(
        hidden=2048, layers=24, q_heads=32, kv_heads=32, head_dim=64, intermediate=8192,
        vocab=49152, rms_eps=1e-5, rope_theta=1e4, name="smollm-1.7b",
    ),
    "llama3-8b": DecoderConfig(
        hidden=4096, layers=32, q_heads=32, kv_heads=8, head_dim=128, intermediate=14336,
        vocab=128256, rms_eps=1e-5, rope_theta=5e5, tied=False, name="llama3-8b",
    ),
}


def tiny_config(**overrides) -> DecoderConfig:
    """A few-layer shape for fast tests; every dimension still a multiple of 64."""
    base = dict(
        hidden=256, layers=2, q_heads=4, kv_heads=2, head_dim=64, intermediate=512,
        vocab=1024, rms_eps=1e-5, rope_theta=1e4, name="tiny",
    )
    base.update(overrides)
    return DecoderConfig(**base)


def _mix32(x: torch.Tensor) -> torch.Tensor:
    x = ((x ^ (x >> 16)) * _MIX) & _MASK32
    x = ((x ^ (x >> 16)) * _MIX) & _MASK32
    return x ^ (x >> 16)


def _byte_sum(x: torch.Tensor) -> torch.Tensor:
    pairs = (x & 0x00FF00FF) + ((x >> 8) & 0x00FF00FF)
    return (pairs & 0xFFFF) + (pairs >> 16)


def _salt(seed: int, name: str) -> int:
    return (zlib.crc32(name.encode()) * 2654435761 + seed * 40503 + 12345) & _MASK32


def synth_normal(
    shape, *, seed: int, name: str, std: float = 0.02,
    device="cpu", dtype=torch.bfloat16, chunk: int = 1 << 24,
) -> torch.Tensor:
    """Approximately N(0, std) values that depend only on (seed, name, index)."""
    count = 1
    for extent in shape:
        count *= int(extent)
    out = torch.empty(count, dtype=dtype, device=device)
    salt = _salt(seed, name)
    scale = torch.tensor(std / _BYTES_STD, dtype=torch.float32, device=device)

    def fill(start: int, stop: int) -> None:
        index = torch.arange(start, stop, dtype=torch.int64, device=device)
        first = _mix32((index + salt) & _MASK32)
        second = _mix32((first + 0x9E3779B9 + (index >> 32)) & _MASK32)
        total = _byte_sum(first) + _byte_sum(second) - 1020
        out[start:stop] = (total.to(torch.float32) * scale).to(dtype)

    if torch.device(device).type == "cpu" and count > (1 << 22):
        # On the host the two dozen element-wise passes are memory-bound: pieces that stay in cache,
        # spread over the cores, fill a 1.7 G-parameter model in a minute instead of four.
        from concurrent.futures import ThreadPoolExecutor
        import os

        piece = 1 << 20
        with ThreadPoolExecutor(max(1, min(32, os.cpu_count() or 1))) as pool:
            list(pool.map(lambda start: fill(start, min(count, start + piece)), range(0, count, piece)))
    else:
        for start in range(0, count, chunk):
            fill(start, min(count, start + chunk))
    return out.view(*shape)


def synth_ids(count: int, vocab: int, *, seed: int, name: str = "ids") -> torch.Tensor:
    """``count`` token ids uniform in [0, vocab) (int64, CPU)."""
    index = torch.arange(count, dtype=torch.int64)
    return _mix32((index + _salt(seed, name)) & _MASK32) % vocab


def weight_names(config: DecoderConfig) -> list[tuple[str, tuple[int, ...], str]]:
    """(Hugging Face parameter name, shape, kind) in model order; kind is
    ``normal`` (N(0, 0.02)) or ``ones`` (norm weights keep their default)."""
    names: list[tuple[str, tuple[int, ...], str]] = [
        ("model.embed_tokens.weight", (config.vocab, config.hidden), "normal")
    ]
    for layer in range(config.layers):
        prefix = f"model.layers.{layer}."
        names.append((prefix + "input_layernorm.weight", (config.hidden,), "ones"))
        for proj, rows in (("q", config.q_size), ("k", config.kv_size), ("v", config.kv_size)):
            names.append((prefix + f"self_attn.{proj}_proj.weight", (rows, config.hidden), "normal"))
            if config.qkv_bias:
                names.append((prefix + f"self_attn.{proj}_proj.bias", (rows,), "normal"))
        names.append((prefix + "self_attn.o_proj.weight", (config.hidden, config.q_size), "normal"))
        names.append((prefix + "post_attention_layernorm.weight", (config.hidden,), "ones"))
        names.append((prefix + "mlp.gate_proj.weight", (config.intermediate, config.hidden), "normal"))
        names.append((prefix + "mlp.up_proj.weight", (config.intermediate, config.hidden), "normal"))
        names.append((prefix + "mlp.down_proj.weight", (config.hidden, config.intermediate), "normal"))
    names.append(("model.norm.weight", (config.hidden,), "ones"))
    if not config.tied:
        names.append(("lm_head.weight", (config.vocab, config.hidden), "normal"))
    return names


def synth_weights(
    config: DecoderConfig, *, seed: int = 0, device="cpu", norm_std: float | None = None
) -> dict[str, torch.Tensor]:
    """State dict (Hugging Face names, bf16) for ``config``.

    ``norm_std`` set to a float draws the norm weights as 1 + N(0, norm_std)
    instead of ones, so tests exercise the weight multiply of RMSNorm.
    """
    weights: dict[str, torch.Tensor] = {}
    for name, shape, kind in weight_names(config):
        if kind == "normal":
            weights[name] = synth_normal(shape, seed=seed, name=name, device=device)
        elif norm_std is None:
            weights[name] = torch.ones(shape, dtype=torch.bfloat16, device=device)
        else:
            noise = synth_normal(shape, seed=seed, name=name, std=norm_std, device=device, dtype=torch.float32)
            weights[name] = (1.0 + noise).to(torch.bfloat16)
    if config.tied:
        weights["lm_head.weight"] = weights["model.embed_tokens.weight"]
    return weights


def rope_tables(config: DecoderConfig, positions: int, device="cpu", dtype=torch.bfloat16) -> tuple[torch.Tensor, torch.Tensor]:
    """bf16 cos/sin tables ``[positions, head_dim]`` computed the way
    transformers' rotary embedding does (modeling_llama.py: fp32 outer product
    of inv_freq and position, cos/sin in fp32, one cast to bf16).  Computed on
    the CPU so the table does not depend on the device's cos/sin routines."""
    dim = config.head_dim
    inv_freq = 1.0 / (
        config.rope_theta ** (torch.arange(0, dim, 2, dtype=torch.int64).to(torch.float32) / dim)
    )
    if config.inv_freq_bf16:
        inv_freq = inv_freq.to(torch.bfloat16).to(torch.float32)
    position = torch.arange(positions, dtype=torch.int64).to(torch.float32)
    freqs = position[:, None] * inv_freq[None, :]
    emb = torch.cat((freqs, freqs), dim=-1)
    cos = emb.cos().to(dtype)
    sin = emb.sin().to(dtype)
    return cos.to(device).contiguous(), sin.to(device).contiguous()


def new_kv_state(config: DecoderConfig, batch: int, capacity: int, device="cpu"):
    """Zeroed decode state: per layer a key cache and a value cache
    ``[batch, capacity, kv_heads, head_dim]`` (bf16) and an int32 ``[1]`` valid length."""
    shape = (batch, capacity, config.kv_heads, config.head_dim)
    keys = [torch.zeros(shape, dtype=torch.bfloat16, device=device) for _ in range(config.layers)]
    values = [torch.zeros(shape, dtype=torch.bfloat16, device=device) for _ in range(config.layers)]
    lengths = [torch.zeros(1, dtype=torch.int32, device=device) for _ in range(config.layers)]
    return keys, values, lengths
