"""``bucketed``: prompts of any length through a handful of fixed-shape compiled kernels.

Written from the contract of the reference's ``megabake.bucketed`` (src/megabake/buckets.py:49-184:
constructor arguments, the two error types, first-call verification), not from its text.  The
megakernel is compiled for static shapes; a caller's sequence arguments are extended at their end
to the smallest bucket that holds them, the bucket's kernel runs, and outputs are narrowed back.
That is only exact when real positions never look at the filler (a causal decoder with the filler
behind the prompt), so each bucket proves it once, in eager mode, before its results are trusted:
two different fillers must give identical outputs at the real positions, and those outputs must
agree with the unpadded call.
"""

from __future__ import annotations

import inspect
from collections.abc import Callable, Mapping, Sequence
from typing import Any

import torch
from torch.utils import _pytree as pytree

DEFAULT_BUCKETS = (16, 32, 64, 128, 256, 512)
_RELATIVE_L2_LIMIT = 0.05  # eager on a longer shape may pick other kernels; reading the filler is off by far more


class PaddingDependence(ValueError):
    """Outputs at real positions change with the padding, so buckets are inexact."""


def _extend(tensor: torch.Tensor, dim: int, extra: int, filler) -> torch.Tensor:
    """``tensor`` with ``extra`` more entries along ``dim``: a constant, or (filler is None) junk
    that differs from any constant, used only to prove that nobody reads it."""
    shape = list(tensor.shape)
    shape[dim] = extra
    if filler is not None:
        tail = tensor.new_full(shape, filler)
    else:
        ramp = torch.arange(extra, device=tensor.device).view([-1 if axis == dim else 1 for axis in range(tensor.dim())])
        junk = (ramp % 2) if not tensor.dtype.is_floating_point else (ramp % 3).to(torch.float32) * 1.5 - 1.0
        tail = junk.to(tensor.dtype).expand(shape)
    return torch.cat((tensor, tail), dim=dim)


def _narrow_outputs(tree: Any, dim: int, bucket: int, length: int) -> Any:
    if bucket == length:
        return tree

    def narrow(leaf: Any) -> Any:
        if isinstance(leaf, torch.Tensor) and leaf.dim() > dim and leaf.shape[dim] == bucket:
            return leaf.narrow(dim, 0, length)
        return leaf

    return pytree.tree_map(narrow, tree)


def _tensors(tree: Any) -> list[torch.Tensor]:
    return [leaf for leaf in pytree.tree_leaves(tree) if isinstance(leaf, torch.Tensor)]


class bucketed:
    """Call ``module`` at any sequence length up to ``max(buckets)``.

    ``sequence_args`` maps argument names to their sequence dimension, ``pad_values`` names the
    filler per argument (default 0), and tensor outputs whose extent along ``output_dim`` equals
    the bucket are narrowed to the caller's length."""

    def __init__(self, module: torch.nn.Module | Callable[..., Any], *, backend: Any,
                 sequence_args: Mapping[str, int], pad_values: Mapping[str, int | float] | None = None,
                 buckets: Sequence[int] = DEFAULT_BUCKETS, output_dim: int = 1, verify: bool = True) -> None:
        if not sequence_args:
            raise ValueError("bucketed needs at least one sequence argument")
        sizes = sorted(set(int(size) for size in buckets))
        if not sizes or sizes[0] < 1:
            raise ValueError("buckets must be positive lengths")
        self.module = module
        self.buckets = tuple(sizes)
        self.sequence_args = dict(sequence_args)
        self.pad_values = {name: (pad_values or {}).get(name, 0) for name in self.sequence_args}
        self.output_dim = output_dim
        self.verify = verify
        self.verified: set[int] = set()
        callee = module.forward if isinstance(module, torch.nn.Module) else module
        self._bind = inspect.signature(callee).bind
        # one Dynamo compile per bucket shape, on top of whatever the caller compiled before
        limit = torch._dynamo.config.recompile_limit
        torch._dynamo.config.recompile_limit = max(limit, len(self.buckets) + 1)
        self.compiled = torch.compile(module, backend=backend, fullgraph=True, dynamic=False)

    def bucket_for(self, length: int) -> int:
        fitting = [size for size in self.buckets if size >= length]
        if not fitting:
            raise ValueError(f"length {length} exceeds the largest bucket {self.buckets[-1]}")
        return fitting[0]

    def _sequence_length(self, arguments: Mapping[str, Any]) -> int:
        found = {name: arguments[name].shape[dim] for name, dim in self.sequence_args.items()
                 if isinstance(arguments.get(name), torch.Tensor)}
        if not found:
            raise ValueError("no sequence argument was passed")
        if len(set(found.values())) > 1:
            raise ValueError(f"sequence arguments disagree on the length: {found}")
        return next(iter(found.values()))

    def _at_bucket(self, arguments: Mapping[str, Any], length: int, bucket: int, junk: bool) -> dict[str, Any]:
        padded = dict(arguments)
        for name, dim in self.sequence_args.items():
            value = arguments.get(name)
            if bucket > length and isinstance(value, torch.Tensor):
                padded[name] = _extend(value, dim, bucket - length, None if junk else self.pad_values[name])
        return padded

    def __call__(self, *args: Any, **kwargs: Any) -> Any:
        arguments = dict(self._bind(*args, **kwargs).arguments)
        length = self._sequence_length(arguments)
        bucket = self.bucket_for(length)
        with torch.no_grad():
            raw = self.compiled(**self._at_bucket(arguments, length, bucket, junk=False))
        result = _narrow_outputs(raw, self.output_dim, bucket, length)
        if self.verify and bucket not in self.verified:
            self._prove_padding_is_ignored(arguments, length, bucket)
            self.verified.add(bucket)
        return result

    def _prove_padding_is_ignored(self, arguments: Mapping[str, Any], length: int, bucket: int) -> None:
        def eager(inputs):
            with torch.no_grad():
                return self.module(**inputs)

        with_filler = _tensors(_narrow_outputs(eager(self._at_bucket(arguments, length, bucket, junk=False)),
                                               self.output_dim, bucket, length))
        with_junk = _tensors(_narrow_outputs(eager(self._at_bucket(arguments, length, bucket, junk=True)),
                                             self.output_dim, bucket, length))
        unpadded = _tensors(eager(dict(arguments)))
        if len(with_filler) != len(with_junk) or any(not torch.equal(a, b) for a, b in zip(with_filler, with_junk)):
            raise PaddingDependence("outputs at real positions change with the padding; "
                                    "this callable cannot run through padded buckets")
        if len(unpadded) != len(with_filler):
            raise PaddingDependence("padded and unpadded calls return different numbers of tensors")
        for plain, padded in zip(unpadded, with_filler):
            if plain.shape != padded.shape:
                raise PaddingDependence(f"padded output has shape {tuple(padded.shape)}, unpadded {tuple(plain.shape)}")
            if not plain.is_floating_point():
                if not torch.equal(plain, padded):
                    raise PaddingDependence(f"bucket {bucket}: padded eager differs from unpadded eager")
                continue
            scale = float(plain.float().norm())
            gap = float((padded.float() - plain.float()).norm())
            if scale > 0 and gap / scale > _RELATIVE_L2_LIMIT:
                raise PaddingDependence(f"bucket {bucket}: padded eager is {gap / scale:.3g} from unpadded eager")
