"""The Manatar decoder: manifest of its tensors and how its layers are built from the engine's parts.

A small decoder-only language model.  The embedding adds a second row chosen by a hash of the previous and the current token.  Every
layer is  x += m rms(mixer(x)) w1,  then (unless absent)  x += m rms(ff(x)) w2:  the sublayers read the residual stream itself and
the norm sits on what they give.  A layer's mixer is differential attention (two softmax maps a head over shared values, with a
short convolution, a norm per head and map and a rotation with rescaled frequencies in front, an output gate behind, optionally
reading another layer's cached keys and values) or the matrix memory with exponential gates; its feed-forward a clamped gated one or
routed experts with a shared expert.

Tensor names: embed, bigram, final.norm, head; layer i has l<i>.norm1, l<i>.norm2, l<i>.mix.* and l<i>.mlp.*.  Matrices are [out, in].
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..config.manatar import DenseFFSpec, DiffAttentionSpec, ExpertsFFSpec, ManatarConfig, MlstmSpec
from ..parts.diff_attention import DiffAttention
from ..parts.embedding import Embedding, HashedPairEmbedding, LMHead
from ..parts.registry import make_part
from ..parts.rotary import blended_frequencies
from ..weights.loader import WeightSpec
from .decoder import DecoderModel, LayerRun

UNBOUNDED_POSITIONS = 1 << 24       # nothing of the model is a table over positions; float32 holds these exactly


def manatar_manifest(cfg: ManatarConfig) -> List[WeightSpec]:
    W = cfg.width
    m = [WeightSpec("embed", (cfg.vocab, W))]
    if cfg.bigram is not None:
        m.append(WeightSpec("bigram", (cfg.bigram.buckets + 1, W)))
    for i, layer in enumerate(cfg.layers):
        p, mx = f"l{i}.", layer.mixer
        m.append(WeightSpec(p + "norm1", (W,)))
        if isinstance(mx, DiffAttentionSpec):
            qn, kn, vn = mx.heads * 2 * mx.dim, mx.kv_heads * 2 * mx.dim, mx.kv_heads * mx.vdim
            names = [("q", qn)] + ([("k", kn), ("v", vn)] if mx.kv_from is None else [])
            for name, rows in names:
                m += [WeightSpec(f"{p}mix.{name}", (rows, W)), WeightSpec(f"{p}mix.{name}.b", (rows,))]
                if mx.conv:
                    m.append(WeightSpec(f"{p}mix.{name}.conv", (rows, mx.conv)))
            m.append(WeightSpec(p + "mix.q.norm", (mx.dim,)))
            if mx.kv_from is None:
                m.append(WeightSpec(p + "mix.k.norm", (mx.dim,)))
            m += [WeightSpec(p + "mix." + n, (mx.dim,)) for n in ("lq1", "lk1", "lq2", "lk2")]
            m += [WeightSpec(p + "mix.g", (mx.heads * mx.vdim, W)), WeightSpec(p + "mix.o", (W, mx.heads * mx.vdim)), WeightSpec(p + "mix.o.b", (W,))]
        else:
            qk, v = mx.heads * mx.dim, mx.heads * mx.vdim
            m += [WeightSpec(p + "mix.q", (qk, W)), WeightSpec(p + "mix.k", (qk, W)), WeightSpec(p + "mix.v", (v, W)), WeightSpec(p + "mix.g", (v, W)),
                  WeightSpec(p + "mix.o", (W, v)), WeightSpec(p + "mix.norm", (v,)), WeightSpec(p + "mix.i", (mx.heads, W)),
                  WeightSpec(p + "mix.i.b", (mx.heads,)), WeightSpec(p + "mix.f", (mx.heads, W)), WeightSpec(p + "mix.f.b", (mx.heads,))]
        ff = layer.mlp
        if ff is None:
            continue
        m.append(WeightSpec(p + "norm2", (W,)))
        gated = lambda q, n: [WeightSpec(q + "gate", (n, W)), WeightSpec(q + "up", (n, W)), WeightSpec(q + "down", (W, n))]
        if isinstance(ff, DenseFFSpec):
            m += gated(p + "mlp.", ff.ff)
        else:
            for e in range(ff.experts):
                m += gated(f"{p}mlp.e{e}.", ff.ff)
            m += [WeightSpec(p + "mlp.router", (ff.experts, W)), WeightSpec(p + "mlp.router.b", (ff.experts,))]
            if ff.shared_ff is not None:
                m += gated(p + "mlp.shared.", ff.shared_ff)
    m += [WeightSpec("final.norm", (W,)), WeightSpec("head", (cfg.vocab, W))]
    return m


def is_norm_weight(name: str) -> bool:
    """Tensors that random initialisation makes 1 + noise instead of noise around 0."""
    return name.rsplit(".", 1)[-1] in ("norm1", "norm2", "norm")


def build_manatar(cfg: ManatarConfig, weights: Dict[str, torch.Tensor], dtype: torch.dtype, device) -> DecoderModel:
    """Matrices go to the device in the compute dtype; norms, biases, convolution weights, the gates' biases and the router are
    float32 in both paths."""
    dev = torch.device(device)
    W = cfg.width

    def mat(*names: str) -> torch.Tensor:
        parts = [weights[n].to(device=dev, dtype=dtype) for n in names]
        return parts[0].contiguous() if len(parts) == 1 else torch.cat(parts, dim=0).contiguous()

    def vec(*names: str) -> torch.Tensor:
        parts = [weights[n].to(device=dev, dtype=torch.float32) for n in names]
        return parts[0].contiguous() if len(parts) == 1 else torch.cat(parts, dim=0).contiguous()

    def norm(name: str):
        return make_part("norm", "rmsnorm", width=W, eps=cfg.eps, weight=vec(name))

    def gated(prefix: str, ff: int):
        return make_part("feed_forward", "swiglu", hidden=W, intermediate=ff, w_gate_up=mat(prefix + "gate", prefix + "up"), w_down=mat(prefix + "down"))

    blocks = []
    runs = []           # (cache layer of the pages or of the recurrent state, writes it, has a state beside its pages)
    for i, layer in enumerate(cfg.layers):
        p, mx = f"l{i}.", layer.mixer
        if isinstance(mx, DiffAttentionSpec):
            own = mx.kv_from is None
            names = ["q"] + (["k", "v"] if own else [])
            freq, mag, dims = None, 1.0, 0
            if mx.rot is not None and mx.rot.dims:
                f, mag = blended_frequencies(mx.rot.base, mx.rot.dims, mx.rot.scaling)
                freq, dims = torch.as_tensor(f).to(dev), mx.rot.dims
            b_in = torch.cat([vec(*[f"{p}mix.{n}.b" for n in names]), torch.zeros(mx.heads * mx.vdim, dtype=torch.float32, device=dev)])
            mixer = make_part("mixer", "diff_attention", hidden=W, num_heads=mx.heads, num_kv_heads=mx.kv_heads, dim=mx.dim, vdim=mx.vdim,
                              taps=mx.conv or 1, scale=mx.scale, diff=mx.diff,
                              lam=DiffAttention.lambda_of(*[weights[p + "mix." + n] for n in ("lq1", "lk1", "lq2", "lk2")], mx.diff),
                              eps=cfg.eps, w_in=mat(*[f"{p}mix.{n}" for n in names], p + "mix.g"), b_in=b_in,
                              conv=vec(*[f"{p}mix.{n}.conv" for n in names]) if mx.conv else None, q_norm=vec(p + "mix.q.norm"),
                              k_norm=vec(p + "mix.k.norm") if own else None, w_out=mat(p + "mix.o"), b_out=vec(p + "mix.o.b"), freq=freq, mag=mag,
                              rot_dims=dims, shares_kv=not own)
            runs.append((i if own else mx.kv_from, own, mixer.state_spec() is not None))
        else:
            mixer = make_part("mixer", "mlstm", hidden=W, num_heads=mx.heads, dim=mx.dim, vdim=mx.vdim, gate_cap=mx.gate_cap,
                              w_in=mat(p + "mix.q", p + "mix.k", p + "mix.v", p + "mix.g", p + "mix.i", p + "mix.f"),
                              gate_bias=vec(p + "mix.i.b", p + "mix.f.b"), norm_weight=vec(p + "mix.norm"), w_out=mat(p + "mix.o"), eps=cfg.eps)
            runs.append((i, True, False))
        ffn = ffn_norm = None
        ff = layer.mlp
        if isinstance(ff, DenseFFSpec):
            ffn = make_part("feed_forward", "clamped_glu", hidden=W, intermediate=ff.ff, w_gate_up=mat(p + "mlp.gate", p + "mlp.up"),
                            w_down=mat(p + "mlp.down"), limit=ff.limit, alpha=1.702)
        elif isinstance(ff, ExpertsFFSpec):
            gu = torch.stack([mat(f"{p}mlp.e{e}.gate", f"{p}mlp.e{e}.up") for e in range(ff.experts)]).contiguous()
            down = torch.stack([mat(f"{p}mlp.e{e}.down") for e in range(ff.experts)]).contiguous()
            ffn = make_part("feed_forward", "routed_experts", hidden=W, intermediate=ff.ff, experts=ff.experts, top=ff.top,
                            w_router=vec(p + "mlp.router"), b_router=vec(p + "mlp.router.b"), w_gate_up=gu, w_down=down,
                            shared=None if ff.shared_ff is None else gated(p + "mlp.shared.", ff.shared_ff), activation="silu")
        if ffn is not None:
            ffn_norm = norm(p + "norm2")
        blocks.append(make_part("block", "output_norm", mixer_norm=norm(p + "norm1"), mixer=mixer, ffn_norm=ffn_norm, ffn=ffn, mult=cfg.residual_mult))
    # cache layers are numbered without gaps: first those the runs name (a layer that reads another's rows has none), then the
    # states that attention layers keep beside their pages
    used = sorted({c for c, _, _ in runs})
    renumber = {c: n for n, c in enumerate(used)}
    schedule: List[LayerRun] = []
    extra = len(used)
    for i, (c, writes, beside) in enumerate(runs):
        schedule.append(LayerRun(block=i, cache=renumber[c], write_cache=writes, state=extra if beside else -1))
        extra += bool(beside)
    if cfg.bigram is not None:
        b = cfg.bigram
        embedding = HashedPairEmbedding(cfg.vocab, W, mat("embed"), mat("bigram"), b.buckets, b.mul_prev, b.mul_cur)
    else:
        embedding = Embedding(cfg.vocab, W, mat("embed"))
    return DecoderModel(embedding=embedding, blocks=blocks, schedule=schedule, final_norm=norm("final.norm"), lm_head=LMHead(cfg.vocab, W, mat("head")),
                        position=None, dtype=dtype, vocab_size=cfg.vocab, max_positions=UNBOUNDED_POSITIONS, config=cfg)
