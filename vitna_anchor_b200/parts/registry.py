"""Names of the kinds of parts, so that a configuration can choose them layer by layer.

A builder (see models/) turns a list of LayerSpec into blocks by looking the
names up here.  Registering a new kind is one call; nothing else changes.
"""
from __future__ import annotations

from typing import Callable, Dict

MIXERS: Dict[str, Callable] = {}
FEED_FORWARDS: Dict[str, Callable] = {}
NORMS: Dict[str, Callable] = {}
POSITION_ENCODINGS: Dict[str, Callable] = {}
BLOCKS: Dict[str, Callable] = {}

_KINDS = {"mixer": MIXERS, "feed_forward": FEED_FORWARDS, "norm": NORMS, "position": POSITION_ENCODINGS, "block": BLOCKS}


def register_part(kind: str, name: str, factory: Callable) -> None:
    """factory(**params) -> the part.  `kind` is one of mixer, feed_forward, norm, position, block."""
    if kind not in _KINDS:
        raise KeyError(f"unknown kind of part {kind!r}; kinds are {sorted(_KINDS)}")
    _KINDS[kind][name] = factory


def make_part(kind: str, name: str, **params):
    table = _KINDS[kind]
    if name not in table:
        raise KeyError(f"no {kind} named {name!r}; registered: {sorted(table)}")
    return table[name](**params)


def _register_builtin() -> None:
    from .attention import PagedAttention
    from .block import OutputNormBlock, PreNormBlock, SandwichNormBlock
    from .gla import GatedLinearAttention
    from .mixed_attention import MixedHeadAttention
    from .diff_attention import DiffAttention
    from .mlstm import MatrixLSTM
    from .delta import ChannelDeltaRule, GatedDeltaRule
    from .latent import LatentAttention
    from .feed_forward import ClampedGLU, DenseMLP, RoutedExperts, SwiGLU
    from .hyper import HyperBlock
    from .norms import LayerNorm, RMSNorm
    from .rotary import NoPositionEncoding, Rotary
    register_part("mixer", "attention", PagedAttention)
    register_part("mixer", "gated_delta", GatedDeltaRule)
    register_part("mixer", "channel_delta", ChannelDeltaRule)
    register_part("mixer", "latent_attention", LatentAttention.from_matrices)
    register_part("mixer", "diff_attention", DiffAttention)
    register_part("mixer", "mlstm", MatrixLSTM)
    register_part("mixer", "gla", GatedLinearAttention)
    register_part("mixer", "mixed_attention", MixedHeadAttention)
    register_part("feed_forward", "clamped_glu", ClampedGLU)
    register_part("feed_forward", "routed_experts", RoutedExperts)
    register_part("feed_forward", "swiglu", SwiGLU)
    register_part("feed_forward", "gated", SwiGLU)           # the same part; `activation` chooses the gate's function
    register_part("feed_forward", "dense", DenseMLP)
    register_part("norm", "rmsnorm", RMSNorm)
    register_part("norm", "layernorm", LayerNorm)
    register_part("position", "rotary", Rotary)
    register_part("position", "none", NoPositionEncoding)
    register_part("block", "pre_norm", PreNormBlock)
    register_part("block", "output_norm", OutputNormBlock)
    register_part("block", "sandwich_norm", SandwichNormBlock)
    register_part("block", "hyper", HyperBlock)


_register_builtin()
