"""Typed configuration of the Manatar decoder, read from config.json.

config.json gives every size and every constant that differs between models of the design:

    architecture      "Manatar"
    vocab, width
    norm.eps          eps of every RMS norm of the model (around the sublayers, inside the mixers, before the output matrix)
    residual_mult     m in  x <- x + m * norm(sublayer(x))
    embedding.bigram  {buckets, mul_prev, mul_cur}: a second embedding row, chosen by a hash of the previous and the current token
                      (absent: none)
    layers            a list; each entry has `type` (attention | mlstm), `mixer` (its sizes) and `mlp` (or null)

An attention mixer gives heads, kv_heads, dim, vdim, conv (taps of the short convolution), diff, scale, rot {base, dims, scaling
{factor, original, fast, slow}} and, optionally, kv_from (the layer whose cached keys and values it reads).  An mlstm mixer gives
heads, dim, vdim and gate_cap.  A feed-forward is {kind: dense, ff, limit} or {kind: moe, expert {ff}, router {experts, top},
shared {ff} (optional)}.  There is no limit on positions: nothing of the model is a table over them.  A key inside a layer that
this reader does not know is refused by name.
"""
from __future__ import annotations

import warnings
from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .errors import ConfigError
from .lupanex import _known, _number, _size
from .siparax import RotationSpec, _rotation

ARCHITECTURE = "Manatar"


@dataclass(frozen=True)
class BigramSpec:
    buckets: int
    mul_prev: int
    mul_cur: int


@dataclass(frozen=True)
class DiffAttentionSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int                       # taps of the short convolution on q, k and v (0: the key is absent, and so are the conv tensors)
    diff: float
    scale: float
    rot: Optional[RotationSpec]
    kv_from: Optional[int] = None

    kind = "attention"


@dataclass(frozen=True)
class MlstmSpec:
    heads: int
    dim: int
    vdim: int
    gate_cap: float

    kind = "mlstm"


@dataclass(frozen=True)
class DenseFFSpec:
    ff: int
    limit: float

    kind = "dense"


@dataclass(frozen=True)
class ExpertsFFSpec:
    ff: int                         # of one routed expert
    experts: int
    top: int
    shared_ff: Optional[int]        # of the expert every token uses (None: there is none)

    kind = "moe"


@dataclass(frozen=True)
class LayerSpec:
    mixer: Any                      # DiffAttentionSpec or MlstmSpec
    mlp: Any                        # DenseFFSpec, ExpertsFFSpec or None


def _mlp(entry: Any, where: str):
    if entry is None:
        return None
    if not isinstance(entry, Mapping):
        raise ConfigError(f"config.json: {where} is not an object")
    kind = entry.get("kind")
    if kind == "dense":
        _known(entry, where, ("kind", "ff", "limit"))
        limit = _number(entry, "limit", where + ".")
        if limit <= 0:
            raise ConfigError(f"config.json: {where}.limit is not positive")
        return DenseFFSpec(_size(entry, "ff", where + "."), limit)
    if kind == "moe":
        _known(entry, where, ("kind", "expert", "router", "shared"))
        _known(entry.get("expert"), where + ".expert", ("ff",))
        _known(entry.get("router"), where + ".router", ("experts", "top"))
        shared = None
        if entry.get("shared") is not None:
            _known(entry["shared"], where + ".shared", ("ff",))
            shared = _size(entry["shared"], "ff", where + ".shared.")
        experts, top = _size(entry["router"], "experts", where + ".router."), _size(entry["router"], "top", where + ".router.")
        if top > experts:
            raise ConfigError(f"config.json: {where}.router.top is larger than the number of experts")
        return ExpertsFFSpec(_size(entry["expert"], "ff", where + ".expert."), experts, top, shared)
    raise ConfigError(f"config.json: {where}.kind is {kind!r}; the kinds are dense and moe")


def _layer(i: int, entry: Mapping[str, Any]) -> LayerSpec:
    where = f"layers[{i}]."
    _known(entry, f"layers[{i}]", ("type", "mixer", "mlp"))
    kind, m = entry.get("type"), entry.get("mixer")
    if not isinstance(m, Mapping):
        raise ConfigError(f"config.json: {where}mixer is missing")
    s = lambda k, least=1: _size(m, k, where + "mixer.", least)
    if kind == "attention":
        _known(m, where + "mixer", ("heads", "kv_heads", "dim", "vdim", "conv", "diff", "scale", "rot", "kv_from"))
        heads = s("heads")
        kv = s("kv_heads") if m.get("kv_heads") is not None else heads
        if heads % kv:
            raise ConfigError(f"config.json: {where}mixer.heads do not divide into kv_heads groups")
        dim = s("dim")
        rot = None
        if m.get("rot") is not None:
            rot = _rotation(m["rot"], where + "mixer.rot")
            if rot.dims > dim:
                raise ConfigError(f"config.json: {where}mixer.rot.dims is larger than dim")
        diff = _number(m, "diff", where + "mixer.")
        mixer = DiffAttentionSpec(heads, kv, dim, s("vdim") if m.get("vdim") is not None else dim, s("conv") if m.get("conv") is not None else 0,
                                  diff, _number(m, "scale", where + "mixer."), rot, s("kv_from", 0) if m.get("kv_from") is not None else None)
    elif kind == "mlstm":
        _known(m, where + "mixer", ("heads", "dim", "vdim", "gate_cap"))
        cap = _number(m, "gate_cap", where + "mixer.")
        if cap <= 0:
            raise ConfigError(f"config.json: {where}mixer.gate_cap is not positive")
        dim = s("dim")
        mixer = MlstmSpec(s("heads"), dim, s("vdim") if m.get("vdim") is not None else dim, cap)
    else:
        raise ConfigError(f"config.json: {where}type is {kind!r}; the mixers are attention and mlstm")
    return LayerSpec(mixer, _mlp(entry.get("mlp"), f"layers[{i}].mlp"))


@dataclass(frozen=True)
class ManatarConfig:
    vocab: int
    width: int
    eps: float
    residual_mult: float
    bigram: Optional[BigramSpec]
    layers: Tuple[LayerSpec, ...]

    architecture = ARCHITECTURE

    @classmethod
    def from_dict(cls, cfg: Mapping[str, Any]) -> "ManatarConfig":
        top = ("architecture", "architectures", "vocab", "width", "norm", "residual_mult", "embedding", "layers")
        other = sorted(set(cfg) - set(top))
        if other:       # notes beside the model (a name, a seed) are no part of it; a key inside a layer is, and is refused
            warnings.warn(f"config.json: keys that are no part of the model are ignored: {', '.join(other)}", stacklevel=2)
        _known(cfg.get("norm"), "norm", ("eps",))
        eps = _number(cfg["norm"], "eps", "norm.")
        if eps < 0:
            raise ConfigError("config.json: norm.eps is negative")
        bigram = None
        emb = cfg.get("embedding")
        if emb is not None:
            _known(emb, "embedding", ("bigram",))
            if emb.get("bigram") is not None:
                b = emb["bigram"]
                _known(b, "embedding.bigram", ("buckets", "mul_prev", "mul_cur"))
                bigram = BigramSpec(_size(b, "buckets", "embedding.bigram."), _size(b, "mul_prev", "embedding.bigram.", 0),
                                    _size(b, "mul_cur", "embedding.bigram.", 0))
        entries = cfg.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json: layers is not a list of layers")
        layers = tuple(_layer(i, e) for i, e in enumerate(entries))
        for i, layer in enumerate(layers):
            m = layer.mixer
            if isinstance(m, DiffAttentionSpec) and m.kv_from is not None:
                src = layers[m.kv_from].mixer if m.kv_from < i else None
                if not isinstance(src, DiffAttentionSpec) or src.kv_from is not None:
                    raise ConfigError(f"config.json: layers[{i}].mixer.kv_from does not name an earlier attention layer with keys of its own")
                if (src.kv_heads, src.dim, src.vdim) != (m.kv_heads, m.dim, m.vdim):     # the rows are read as that layer wrote them
                    raise ConfigError(f"config.json: layers[{i}] and the layer it reads keys from differ in kv_heads, dim or vdim")
        return cls(vocab=_size(cfg, "vocab", ""), width=_size(cfg, "width", ""), eps=eps,
                   residual_mult=_number(cfg, "residual_mult", "") if cfg.get("residual_mult") is not None else 1.0, bigram=bigram, layers=layers)

    def to_dict(self) -> dict:
        """The config.json that reads back as this configuration."""
        def mixer(m):
            if isinstance(m, MlstmSpec):
                return dict(heads=m.heads, dim=m.dim, vdim=m.vdim, gate_cap=m.gate_cap)
            d = dict(heads=m.heads, kv_heads=m.kv_heads, dim=m.dim, vdim=m.vdim, diff=m.diff, scale=m.scale)
            if m.conv:
                d["conv"] = m.conv
            if m.rot is not None:
                rot = dict(base=m.rot.base, dims=m.rot.dims)
                if m.rot.scaling is not None:
                    rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), m.rot.scaling))
                d["rot"] = rot
            if m.kv_from is not None:
                d["kv_from"] = m.kv_from
            return d

        def mlp(f):
            if f is None:
                return None
            if isinstance(f, DenseFFSpec):
                return dict(kind="dense", ff=f.ff, limit=f.limit)
            d = dict(kind="moe", expert=dict(ff=f.ff), router=dict(experts=f.experts, top=f.top))
            if f.shared_ff is not None:
                d["shared"] = dict(ff=f.shared_ff)
            return d

        d = dict(architecture=ARCHITECTURE, vocab=self.vocab, width=self.width, norm=dict(eps=self.eps), residual_mult=self.residual_mult,
                 layers=[dict(type=l.mixer.kind, mixer=mixer(l.mixer), mlp=mlp(l.mlp)) for l in self.layers])
        if self.bigram is not None:
            d["embedding"] = dict(bigram=dict(buckets=self.bigram.buckets, mul_prev=self.bigram.mul_prev, mul_cur=self.bigram.mul_cur))
        return d
