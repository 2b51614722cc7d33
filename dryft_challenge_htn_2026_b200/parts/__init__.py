"""Parts a model is put together from: norms, position encodings, mixers, feed-forwards, blocks."""
from .base import ParamDecl, Part, Runtime, build_part, register_part
from . import norm, position, attention, attention_masked, linear_attention, parallel, feedforward, block  # noqa: F401  (register the built-in parts)
from .attention import GQAAttention
from .attention_masked import MaskedAttention
from .block import PreNormBlock
from .feedforward import DenseMLP, GatedMLP
from .linear_attention import LinearAttention
from .norm import RMSNorm, ScalarRMSNorm
from .parallel import ParallelMixer
from .position import RotaryHalf, Sinusoid

__all__ = ["ParamDecl", "Part", "Runtime", "build_part", "register_part", "GQAAttention", "PreNormBlock", "GatedMLP",
           "RMSNorm", "RotaryHalf", "MaskedAttention", "LinearAttention", "ParallelMixer", "DenseMLP", "ScalarRMSNorm",
           "Sinusoid"]
