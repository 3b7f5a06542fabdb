"""B200-native decoder megakernel behind MegaBake's backend surface.

    import megabake_b200 as megabake
    step = torch.compile(decoder, backend=megabake.make_backend(mode="decode"), fullgraph=True)

Public names follow the reference package (src/megabake/__init__.py:59-117) for the part
of its surface that the hot path needs.
"""

from .buckets import DEFAULT_BUCKETS, PaddingDependence, bucketed
from .diagnostics import CompilerDiagnostic, CompilerError
from .frontend import CaptureContext, make_backend, recognise_decoder
from .hf_attention import (DecodeStep, megabake_attention_forward, megabake_decode_attention,
                           register_transformers_attention)
from .models import ExplicitStateDecoder
from .ops import attention, kv_attention
from .synth import CONFIGS, DecoderConfig

__all__ = [
    "DEFAULT_BUCKETS", "PaddingDependence", "bucketed", "CompilerDiagnostic", "CompilerError",
    "CaptureContext", "make_backend", "recognise_decoder", "DecodeStep", "megabake_attention_forward",
    "megabake_decode_attention", "register_transformers_attention", "ExplicitStateDecoder", "attention",
    "kv_attention", "CONFIGS", "DecoderConfig", "DecoderKernel",
]


def __getattr__(name):
    if name == "DecoderKernel":  # imported lazily: it loads the CUDA library
        from .runtime import DecoderKernel

        return DecoderKernel
    raise AttributeError(name)
