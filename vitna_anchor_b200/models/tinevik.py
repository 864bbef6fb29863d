"""The Tinevik decoder: manifest of its tensors and how its layers are built from the engine's parts.

A small decoder-only language model.  x = scale * the token's row.  Every layer is  x += LN1b(mixer(LN1(x))),  then (unless absent)
x += LN2b(ff(LN2(x))),  with layer norms (weight and bias) before and behind each sublayer.  A layer's mixer is gated linear attention
(a matrix state that decays per key channel), an attention whose heads' scores are capped and mixed before the softmax and whose
values are rotated like its keys, or latent attention over a window with a gate on every value; its feed-forward a dense one with an
activation of two learned numbers, or experts that a table assigns to token ids.  A layer may run with another layer's tensors
(`weights_of`), with a cache or state of its own.  The logits are  c * E LN(x)  with the embedding table E itself.

Tensor names: embed, final.norm(.b); layer i has l<i>.norm1, norm1b, norm2, norm2b (each with .b), l<i>.mix.* and l<i>.mlp.*.
Matrices are [out, in].
"""
from __future__ import annotations

from typing import Dict, List

import numpy as np
import torch

from ..config.tinevik import DenseFFSpec, GlaSpec, MixedAttentionSpec, TableExpertsSpec, TinevikConfig, WindowLatentSpec
from ..parts.block import SandwichFlush
from ..parts.embedding import LMHead, ScaledEmbedding
from ..parts.registry import make_part
from ..weights.loader import WeightSpec
from .decoder import DecoderModel, LayerRun

UNBOUNDED_POSITIONS = 1 << 24       # nothing of the model is a table over positions; float32 holds these exactly


def tinevik_manifest(cfg: TinevikConfig) -> List[WeightSpec]:
    W = cfg.width
    norm = lambda name: [WeightSpec(name, (W,)), WeightSpec(name + ".b", (W,))]
    m = [WeightSpec("embed", (cfg.vocab, W))]
    for i, layer in enumerate(cfg.layers):
        if layer.weights_of is not None:
            continue
        p, mx = f"l{i}.", layer.mixer
        m += norm(p + "norm1") + norm(p + "norm1b")
        if isinstance(mx, GlaSpec):
            qk, v = mx.heads * mx.dim, mx.heads * mx.vdim
            m += [WeightSpec(p + "mix.q", (qk, W)), WeightSpec(p + "mix.k", (qk, W)), WeightSpec(p + "mix.v", (v, W)), WeightSpec(p + "mix.g", (v, W)),
                  WeightSpec(p + "mix.o", (W, v)), WeightSpec(p + "mix.norm", (mx.vdim,)), WeightSpec(p + "mix.a1", (None, W), free_size=16),
                  WeightSpec(p + "mix.a2", (qk, None), free_size=16), WeightSpec(p + "mix.a2.b", (qk,))]
        elif isinstance(mx, MixedAttentionSpec):
            m += [WeightSpec(p + "mix.q", (mx.heads * mx.dim, W)), WeightSpec(p + "mix.k", (mx.kv_heads * mx.dim, W)),
                  WeightSpec(p + "mix.v", (mx.kv_heads * mx.vdim, W)), WeightSpec(p + "mix.q.norm", (mx.dim,)), WeightSpec(p + "mix.k.norm", (mx.dim,)),
                  WeightSpec(p + "mix.talk", (mx.heads, mx.heads)), WeightSpec(p + "mix.o", (W, mx.heads * mx.vdim))]
        else:
            H = mx.heads
            m += [WeightSpec(p + "mix.dq", (mx.q_rank, W)), WeightSpec(p + "mix.dq.norm", (mx.q_rank,)), WeightSpec(p + "mix.uq", (H * mx.dim, mx.q_rank)),
                  WeightSpec(p + "mix.dkv", (mx.kv_rank, W)), WeightSpec(p + "mix.dkv.norm", (mx.kv_rank,)), WeightSpec(p + "mix.uk", (H * mx.dim, mx.kv_rank)),
                  WeightSpec(p + "mix.uv", (H * mx.vdim, mx.kv_rank)), WeightSpec(p + "mix.g", (H * mx.vdim, W)), WeightSpec(p + "mix.o", (W, H * mx.vdim))]
        ff = layer.mlp
        if ff is None:
            continue
        m += norm(p + "norm2") + norm(p + "norm2b")
        if isinstance(ff, DenseFFSpec):
            m += [WeightSpec(p + "mlp.up", (ff.ff, W)), WeightSpec(p + "mlp.down", (W, ff.ff)), WeightSpec(p + "mlp.act", (2,))]
        else:
            for e in range(ff.experts):
                q = f"{p}mlp.e{e}."
                m += [WeightSpec(q + "gate", (ff.ff, W)), WeightSpec(q + "up", (ff.ff, W)), WeightSpec(q + "down", (W, ff.ff))]
            m.append(WeightSpec(p + "mlp.table", (cfg.vocab, ff.top), floating=False, int_range=ff.experts))
    m += norm("final.norm")
    return m


def is_norm_weight(name: str):
    """Tensors that random initialisation makes 1 + noise instead of noise around 0 (the heads' mixing matrix: the identity + noise)."""
    last = name.rsplit(".", 1)[-1]
    if last == "talk":
        return "identity"
    return last in ("norm1", "norm2", "norm1b", "norm2b", "norm")


def _frequencies(base: float, dims: int, divide_by: float = 1.0) -> torch.Tensor:
    """f_i = base^(-2i/dims) / divide_by for i < dims / 2, worked out in float64 and rounded once."""
    f = np.power(float(base), -2.0 * np.arange(dims // 2, dtype=np.float64) / float(dims)) / float(divide_by)
    return torch.from_numpy(f.astype(np.float32))


def build_tinevik(cfg: TinevikConfig, weights: Dict[str, torch.Tensor], dtype: torch.dtype, device) -> DecoderModel:
    """Matrices go to the device in the compute dtype; norms, biases, the wide half of the decays' projection, the heads' mixing
    matrix and the activation's two numbers are float32 in both paths."""
    dev = torch.device(device)
    W = cfg.width

    def mat(*names: str) -> torch.Tensor:
        parts = [weights[n].to(device=dev, dtype=dtype) for n in names]
        return parts[0].contiguous() if len(parts) == 1 else torch.cat(parts, dim=0).contiguous()

    def vec(*names: str) -> torch.Tensor:
        parts = [weights[n].to(device=dev, dtype=torch.float32) for n in names]
        return parts[0].contiguous() if len(parts) == 1 else torch.cat(parts, dim=0).contiguous()

    def norm(name: str, mult: float = 1.0):
        return make_part("norm", "layernorm", width=W, eps=cfg.eps, weight=vec(name) * mult, bias=vec(name + ".b") * mult)

    blocks, block_of = [], {}
    for i, layer in enumerate(cfg.layers):
        if layer.weights_of is not None:
            continue
        p, mx = f"l{i}.", layer.mixer
        if isinstance(mx, GlaSpec):
            if weights[p + "mix.a1"].shape[0] != weights[p + "mix.a2"].shape[1]:
                raise ValueError(f"layer {i}: the two halves of the decays' projection differ in rank")
            mixer = make_part("mixer", "gla", hidden=W, num_heads=mx.heads, dim=mx.dim, vdim=mx.vdim, tau=mx.tau,
                              w_in=mat(p + "mix.q", p + "mix.k", p + "mix.v", p + "mix.g", p + "mix.a1"), w_a2=vec(p + "mix.a2"),
                              a_bias=vec(p + "mix.a2.b"), norm_weight=vec(p + "mix.norm"), w_out=mat(p + "mix.o"), eps=cfg.eps)
        elif isinstance(mx, MixedAttentionSpec):
            freq = v_freq = None
            dims = 0
            if mx.rot is not None:
                dims = mx.rot.dims
                freq = _frequencies(mx.rot.base, dims, mx.rot.factor or 1.0).to(dev) if dims else None
                v_freq = _frequencies(mx.rot.base, mx.vdim).to(dev)
            mixer = make_part("mixer", "mixed_attention", hidden=W, num_heads=mx.heads, num_kv_heads=mx.kv_heads, dim=mx.dim, vdim=mx.vdim,
                              scale=mx.scale, w_in=mat(p + "mix.q", p + "mix.k", p + "mix.v"), w_out=mat(p + "mix.o"), eps=cfg.eps,
                              q_norm=vec(p + "mix.q.norm"), k_norm=vec(p + "mix.k.norm"), softcap=mx.softcap, mix=vec(p + "mix.talk"),
                              freq=freq, rot_dims=dims, v_freq=v_freq)
        else:
            assert isinstance(mx, WindowLatentSpec)
            mixer = make_part("mixer", "latent_attention", hidden=W, num_heads=mx.heads, dim=mx.dim, rot_dim=0, v_dim=mx.vdim, kv_rank=mx.kv_rank,
                              q_rank=mx.q_rank, scale=mx.scale, eps=cfg.eps, w_dq=weights[p + "mix.dq"], q_norm=weights[p + "mix.dq.norm"],
                              w_uq=weights[p + "mix.uq"], w_dkv=weights[p + "mix.dkv"], kv_norm=weights[p + "mix.dkv.norm"], w_uk=weights[p + "mix.uk"],
                              w_uv=weights[p + "mix.uv"], w_o=weights[p + "mix.o"], w_gate=weights[p + "mix.g"], freq=np.zeros(0, dtype=np.float32),
                              mag=1.0, rot_dims=0, interleaved=False, dtype=dtype, device=dev, window=mx.window, gate_per_value=True)
        ffn = ffn_norm = ffn_post = None
        ff = layer.mlp
        if isinstance(ff, DenseFFSpec):
            ffn = make_part("feed_forward", "dense", hidden=W, intermediate=ff.ff, w_up=mat(p + "mlp.up"), w_down=mat(p + "mlp.down"),
                            activation="xielu", act_params=[float(v) for v in weights[p + "mlp.act"].to(torch.float32)])
        elif isinstance(ff, TableExpertsSpec):
            gu = torch.stack([mat(f"{p}mlp.e{e}.gate", f"{p}mlp.e{e}.up") for e in range(ff.experts)]).contiguous()
            down = torch.stack([mat(f"{p}mlp.e{e}.down") for e in range(ff.experts)]).contiguous()
            ffn = make_part("feed_forward", "routed_experts", hidden=W, intermediate=ff.ff, experts=ff.experts, top=ff.top, w_router=None,
                            b_router=None, w_gate_up=gu, w_down=down, activation="clamped", limit=ff.limit, alpha=1.702,
                            table=weights[p + "mlp.table"].to(device=dev, dtype=torch.int32))
        if ffn is not None:
            ffn_norm, ffn_post = norm(p + "norm2"), norm(p + "norm2b")
        block_of[i] = len(blocks)
        blocks.append(make_part("block", "sandwich_norm", mixer_norm=norm(p + "norm1"), mixer_post=norm(p + "norm1b"), mixer=mixer,
                                ffn_norm=ffn_norm, ffn_post=ffn_post, ffn=ffn))
    # every layer runs with a cache or state of its own, whoever's tensors it uses
    schedule = [LayerRun(block=block_of[cfg.owner(i)], cache=i) for i in range(len(cfg.layers))]
    embedding = ScaledEmbedding(cfg.vocab, W, mat("embed"), scale=cfg.embedding_scale)
    # logits = c * E LN(x): the factor rides on the last norm's weight and bias, so the output product is the plain one
    return DecoderModel(embedding=embedding, blocks=blocks, schedule=schedule, final_norm=norm("final.norm", cfg.logit_scale),
                        lm_head=LMHead(cfg.vocab, W, embedding.table), position=None, dtype=dtype, vocab_size=cfg.vocab,
                        max_positions=UNBOUNDED_POSITIONS, config=cfg, collect=SandwichFlush(cfg.eps))
