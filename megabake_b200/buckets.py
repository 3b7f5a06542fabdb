"""``bucketed``: variable-length calls through a few fixed-shape compiled kernels.

The kernel has static shapes; a serving engine sends prompts of any length.  Each call
pads its sequence arguments at the end up to the smallest bucket that holds them, runs
that bucket, and cuts the outputs back.  That is exact only if outputs at real positions
ignore the padding (true for causal decoders with the padding after the real tokens), and
this is checked on the first call of every bucket, not assumed.  Same contract as the
reference's ``megabake.bucketed`` (src/megabake/buckets.py:49-184).
"""

from __future__ import annotations

import inspect
from collections.abc import Callable, Mapping, Sequence
from typing import Any

import torch
from torch.utils import _pytree as pytree

DEFAULT_BUCKETS = (16, 32, 64, 128, 256, 512)
_RELATIVE_L2_LIMIT = 0.05  # padded vs unpadded eager differ by kernel choice; reading the padding differs outright


class PaddingDependence(ValueError):
    """Outputs at real positions change with the padding, so buckets are inexact."""


def _tensor_leaves(value: Any) -> list[torch.Tensor]:
    return [leaf for leaf in pytree.tree_leaves(value) if isinstance(leaf, torch.Tensor)]


class bucketed:
    """Call ``module`` at any sequence length up to ``max(buckets)``.

    ``sequence_args`` maps argument names to their sequence dimension; ``pad_values`` gives
    the padding value per argument (default 0); tensor outputs whose size along
    ``output_dim`` equals the bucket are cut back to the real length."""

    def __init__(self, module: torch.nn.Module | Callable[..., Any], *, backend: Any,
                 sequence_args: Mapping[str, int], pad_values: Mapping[str, int | float] | None = None,
                 buckets: Sequence[int] = DEFAULT_BUCKETS, output_dim: int = 1, verify: bool = True) -> None:
        if not sequence_args:
            raise ValueError("bucketed needs at least one sequence argument")
        if not buckets or any(size < 1 for size in buckets):
            raise ValueError("buckets must be positive lengths")
        self.module = module
        self.sequence_args = dict(sequence_args)
        self.pad_values = dict(pad_values or {})
        self.buckets = tuple(sorted(set(buckets)))
        self.output_dim = output_dim
        self.verify = verify
        target = module.forward if isinstance(module, torch.nn.Module) else module
        self._signature = inspect.signature(target)
        # Dynamo recompiles once per bucket shape on top of the first compile.
        torch._dynamo.config.recompile_limit = max(torch._dynamo.config.recompile_limit, len(self.buckets) + 1)
        self.compiled = torch.compile(module, backend=backend, fullgraph=True, dynamic=False)
        self.verified: set[int] = set()

    def bucket_for(self, length: int) -> int:
        for size in self.buckets:
            if length <= size:
                return size
        raise ValueError(f"length {length} exceeds the largest bucket {self.buckets[-1]}")

    def __call__(self, *args: Any, **kwargs: Any) -> Any:
        arguments = dict(self._signature.bind(*args, **kwargs).arguments)
        lengths = {name: arguments[name].shape[dim] for name, dim in self.sequence_args.items()
                   if isinstance(arguments.get(name), torch.Tensor)}
        if not lengths:
            raise ValueError("no sequence argument was passed")
        if len(set(lengths.values())) != 1:
            raise ValueError(f"sequence arguments disagree on the length: {lengths}")
        length = next(iter(lengths.values()))
        bucket = self.bucket_for(length)
        with torch.no_grad():
            output = self.compiled(**self._padded(arguments, length, bucket, seed=None))
        result = self._cut(output, length, bucket)
        if self.verify and bucket not in self.verified:
            self._verify(arguments, length, bucket)
            self.verified.add(bucket)
        return result

    def _padded(self, arguments: Mapping[str, Any], length: int, bucket: int, seed: int | None) -> dict[str, Any]:
        out = dict(arguments)
        if bucket == length:
            return out
        for name, dim in self.sequence_args.items():
            value = arguments.get(name)
            if not isinstance(value, torch.Tensor):
                continue
            shape = list(value.shape)
            shape[dim] = bucket - length
            if seed is None:
                tail = torch.full(shape, self.pad_values.get(name, 0), dtype=value.dtype, device=value.device)
            else:  # a second, different padding for the dependence check
                generator = torch.Generator(device="cpu").manual_seed(seed)
                tail = (torch.randn(shape, generator=generator) if value.dtype.is_floating_point
                        else torch.randint(0, 2, shape, generator=generator)).to(value)
            out[name] = torch.cat((value, tail), dim=dim)
        return out

    def _cut(self, output: Any, length: int, bucket: int) -> Any:
        dim = self.output_dim

        def trim(value: Any) -> Any:
            if (isinstance(value, torch.Tensor) and bucket != length and value.dim() > dim
                    and value.shape[dim] == bucket):
                return value.narrow(dim, 0, length)
            return value

        return pytree.tree_map(trim, output)

    def _verify(self, arguments: Mapping[str, Any], length: int, bucket: int) -> None:
        with torch.no_grad():
            first = self._cut(self.module(**self._padded(arguments, length, bucket, None)), length, bucket)
            second = self._cut(self.module(**self._padded(arguments, length, bucket, 1)), length, bucket)
            plain = self.module(**arguments)
        if not all(torch.equal(a, b) for a, b in zip(_tensor_leaves(first), _tensor_leaves(second), strict=True)):
            raise PaddingDependence("outputs at real positions change with the padding; "
                                    "this callable cannot run through padded buckets")
        for expected, padded in zip(_tensor_leaves(plain), _tensor_leaves(first), strict=True):
            if expected.shape != padded.shape:
                raise PaddingDependence(f"padded output has shape {tuple(padded.shape)}, unpadded {tuple(expected.shape)}")
            if expected.is_floating_point():
                norm = expected.float().norm()
                error = (padded.float() - expected.float()).norm() / norm if norm > 0 else 0.0
                if error > _RELATIVE_L2_LIMIT:
                    raise PaddingDependence(f"bucket {bucket}: padded eager is {float(error):.3g} from unpadded eager")
            elif not torch.equal(expected, padded):
                raise PaddingDependence(f"bucket {bucket}: padded eager differs from unpadded eager")
