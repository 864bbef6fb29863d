"""Typed configuration of the Tinevik decoder, read from config.json.

config.json gives every size and every constant that differs between models of the design:

    architecture      "Tinevik"
    vocab, width
    embedding.scale   the token rows are multiplied by it (absent: 1)
    norm.eps          eps of every norm of the model (the layer norms around the sublayers, the RMS norms inside the mixers)
    logit_scale       the logits are multiplied by it (absent: 1); the output matrix is the embedding table
    layers            a list; each entry has `type` (gla | attention | latent_attention), `mixer` (its sizes), `mlp` (or null) and,
                      optionally, `weights_of`: the layer whose tensors this layer runs with (with a cache or state of its own)

A gla mixer gives heads, dim, vdim and tau.  An attention mixer gives heads, kv_heads, dim, vdim, scale and, optionally, softcap
and rot {base, dims, scaling {factor}}.  A latent_attention mixer gives heads, dim, vdim, kv_rank, q_rank, scale and, optionally,
mask {size}.  A feed-forward is {kind: dense, ff} or {kind: moe, expert {ff, limit}, router {experts, top}}.  There is no limit on
positions: nothing of the model is a table over them.  A key inside a layer that this reader does not know is refused by name.
"""
from __future__ import annotations

import warnings
from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .errors import ConfigError
from .lupanex import _known, _number, _size

ARCHITECTURE = "Tinevik"


@dataclass(frozen=True)
class GlaSpec:
    heads: int
    dim: int
    vdim: int
    tau: float

    kind = "gla"


@dataclass(frozen=True)
class LinearRotation:
    base: float
    dims: int
    factor: Optional[float] = None      # every frequency is divided by it (None: by nothing)


@dataclass(frozen=True)
class MixedAttentionSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: Optional[float]
    rot: Optional[LinearRotation]

    kind = "attention"


@dataclass(frozen=True)
class WindowLatentSpec:
    heads: int
    dim: int
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    window: int                         # 0: every earlier position is seen

    kind = "latent_attention"


@dataclass(frozen=True)
class DenseFFSpec:
    ff: int

    kind = "dense"


@dataclass(frozen=True)
class TableExpertsSpec:
    ff: int
    limit: float
    experts: int
    top: int

    kind = "moe"


@dataclass(frozen=True)
class LayerSpec:
    mixer: Any                          # GlaSpec, MixedAttentionSpec or WindowLatentSpec
    mlp: Any                            # DenseFFSpec, TableExpertsSpec or None
    weights_of: Optional[int] = None    # the layer whose tensors this one runs with


def _mlp(entry: Any, where: str):
    if entry is None:
        return None
    if not isinstance(entry, Mapping):
        raise ConfigError(f"config.json: {where} is not an object")
    kind = entry.get("kind")
    if kind == "dense":
        _known(entry, where, ("kind", "ff"))
        return DenseFFSpec(_size(entry, "ff", where + "."))
    if kind == "moe":
        _known(entry, where, ("kind", "expert", "router"))
        _known(entry.get("expert"), where + ".expert", ("ff", "limit"))
        _known(entry.get("router"), where + ".router", ("experts", "top"))
        limit = _number(entry["expert"], "limit", where + ".expert.")
        if limit <= 0:
            raise ConfigError(f"config.json: {where}.expert.limit is not positive")
        experts, top = _size(entry["router"], "experts", where + ".router."), _size(entry["router"], "top", where + ".router.")
        if top > experts:
            raise ConfigError(f"config.json: {where}.router.top is larger than the number of experts")
        return TableExpertsSpec(_size(entry["expert"], "ff", where + ".expert."), limit, experts, top)
    raise ConfigError(f"config.json: {where}.kind is {kind!r}; the kinds are dense and moe")


def _layer(i: int, entry: Mapping[str, Any]) -> LayerSpec:
    where = f"layers[{i}]."
    _known(entry, f"layers[{i}]", ("type", "mixer", "mlp", "weights_of"))
    kind, m = entry.get("type"), entry.get("mixer")
    if not isinstance(m, Mapping):
        raise ConfigError(f"config.json: {where}mixer is missing")
    s = lambda k, least=1: _size(m, k, where + "mixer.", least)
    num = lambda k: _number(m, k, where + "mixer.")
    if kind == "gla":
        _known(m, where + "mixer", ("heads", "dim", "vdim", "tau"))
        tau = num("tau")
        if tau <= 0:
            raise ConfigError(f"config.json: {where}mixer.tau is not positive")
        dim = s("dim")
        mixer = GlaSpec(s("heads"), dim, s("vdim") if m.get("vdim") is not None else dim, tau)
    elif kind == "attention":
        _known(m, where + "mixer", ("heads", "kv_heads", "dim", "vdim", "scale", "softcap", "rot"))
        heads = s("heads")
        kv = s("kv_heads") if m.get("kv_heads") is not None else heads
        if heads % kv:
            raise ConfigError(f"config.json: {where}mixer.heads do not divide into kv_heads groups")
        dim = s("dim")
        vdim = s("vdim") if m.get("vdim") is not None else dim
        rot = None
        if m.get("rot") is not None:
            r = m["rot"]
            _known(r, where + "mixer.rot", ("base", "dims", "scaling"))
            factor = None
            if r.get("scaling") is not None:
                _known(r["scaling"], where + "mixer.rot.scaling", ("factor",))
                factor = _number(r["scaling"], "factor", where + "mixer.rot.scaling.")
                if factor <= 0:
                    raise ConfigError(f"config.json: {where}mixer.rot.scaling.factor is not positive")
            base, dims = _number(r, "base", where + "mixer.rot."), _size(r, "dims", where + "mixer.rot.", 0)
            if base <= 1 or dims % 2 or dims > dim:
                raise ConfigError(f"config.json: {where}mixer.rot needs a base above 1 and an even number of dims, at most dim")
            if vdim % 2:
                raise ConfigError(f"config.json: {where}mixer.vdim is odd, and the values are rotated in pairs")
            rot = LinearRotation(base, dims, factor)
        cap = None
        if m.get("softcap") is not None:
            cap = num("softcap")
            if cap <= 0:
                raise ConfigError(f"config.json: {where}mixer.softcap is not positive")
        mixer = MixedAttentionSpec(heads, kv, dim, vdim, num("scale"), cap, rot)
    elif kind == "latent_attention":
        _known(m, where + "mixer", ("heads", "dim", "vdim", "kv_rank", "q_rank", "scale", "mask"))
        window = 0
        if m.get("mask") is not None:
            _known(m["mask"], where + "mixer.mask", ("size",))
            window = _size(m["mask"], "size", where + "mixer.mask.")
        dim = s("dim")
        mixer = WindowLatentSpec(s("heads"), dim, s("vdim") if m.get("vdim") is not None else dim, s("kv_rank"), s("q_rank"), num("scale"), window)
    else:
        raise ConfigError(f"config.json: {where}type is {kind!r}; the mixers are gla, attention and latent_attention")
    weights_of = _size(entry, "weights_of", where, 0) if entry.get("weights_of") is not None else None
    return LayerSpec(mixer, _mlp(entry.get("mlp"), f"layers[{i}].mlp"), weights_of)


@dataclass(frozen=True)
class TinevikConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    logit_scale: float
    layers: Tuple[LayerSpec, ...]

    architecture = ARCHITECTURE

    def owner(self, i: int) -> int:
        """The layer whose tensors layer i runs with."""
        j = self.layers[i].weights_of
        return i if j is None else j

    @classmethod
    def from_dict(cls, cfg: Mapping[str, Any]) -> "TinevikConfig":
        top = ("architecture", "architectures", "vocab", "width", "norm", "embedding", "logit_scale", "layers")
        other = sorted(set(cfg) - set(top))
        if other:       # notes beside the model (a name, a seed) are no part of it; a key inside a layer is, and is refused
            warnings.warn(f"config.json: keys that are no part of the model are ignored: {', '.join(other)}", stacklevel=2)
        _known(cfg.get("norm"), "norm", ("eps",))
        eps = _number(cfg["norm"], "eps", "norm.")
        if eps < 0:
            raise ConfigError("config.json: norm.eps is negative")
        scale = 1.0
        if cfg.get("embedding") is not None:
            _known(cfg["embedding"], "embedding", ("scale",))
            if cfg["embedding"].get("scale") is not None:
                scale = _number(cfg["embedding"], "scale", "embedding.")
        entries = cfg.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError("config.json: layers is not a list of layers")
        layers = tuple(_layer(i, e) for i, e in enumerate(entries))
        for i, layer in enumerate(layers):
            j = layer.weights_of
            if j is None:
                continue
            if j >= len(layers) or j == i or layers[j].weights_of is not None:
                raise ConfigError(f"config.json: layers[{i}].weights_of does not name another layer with tensors of its own")
            if (layers[j].mixer, layers[j].mlp) != (layer.mixer, layer.mlp):
                raise ConfigError(f"config.json: layers[{i}] runs with the tensors of layers[{j}] but differs from it in type or sizes")
        return cls(vocab=_size(cfg, "vocab", ""), width=_size(cfg, "width", ""), eps=eps, embedding_scale=scale,
                   logit_scale=_number(cfg, "logit_scale", "") if cfg.get("logit_scale") is not None else 1.0, layers=layers)

    def to_dict(self) -> dict:
        """The config.json that reads back as this configuration."""
        def mixer(m):
            if isinstance(m, GlaSpec):
                return dict(heads=m.heads, dim=m.dim, vdim=m.vdim, tau=m.tau)
            if isinstance(m, WindowLatentSpec):
                d = dict(heads=m.heads, dim=m.dim, vdim=m.vdim, kv_rank=m.kv_rank, q_rank=m.q_rank, scale=m.scale)
                if m.window:
                    d["mask"] = dict(size=m.window)
                return d
            d = dict(heads=m.heads, kv_heads=m.kv_heads, dim=m.dim, vdim=m.vdim, scale=m.scale)
            if m.softcap is not None:
                d["softcap"] = m.softcap
            if m.rot is not None:
                d["rot"] = dict(base=m.rot.base, dims=m.rot.dims)
                if m.rot.factor is not None:
                    d["rot"]["scaling"] = dict(factor=m.rot.factor)
            return d

        def mlp(f):
            if f is None:
                return None
            if isinstance(f, DenseFFSpec):
                return dict(kind="dense", ff=f.ff)
            return dict(kind="moe", expert=dict(ff=f.ff, limit=f.limit), router=dict(experts=f.experts, top=f.top))

        def layer(l):
            d = dict(type=l.mixer.kind, mixer=mixer(l.mixer), mlp=mlp(l.mlp))
            if l.weights_of is not None:
                d["weights_of"] = l.weights_of
            return d

        return dict(architecture=ARCHITECTURE, vocab=self.vocab, width=self.width, norm=dict(eps=self.eps), embedding=dict(scale=self.embedding_scale),
                    logit_scale=self.logit_scale, layers=[layer(l) for l in self.layers])
