"""Attention whose heads' scores are capped and mixed before the softmax, with values that are rotated like keys.

With H query heads, G key-value heads (query head h reads key-value head h // (H / G)), keys of size dim and values of size vdim:

    q, k per head: x / rms(x) * w (w [dim], one for all heads; no norm without weights), then the first `rot_dims` values turned in
                   pairs (i, i + rot_dims / 2) by p * f_i
    v_j            turned over all its pairs (m, m + vdim / 2) by j * g_m, and cached so (no rotation of values without g)
    z_h(i, j)      = scale q_h(i) . k(j);  cap tanh(z / cap) (no cap: as it is);  z'_h = sum_g M[h, g] z_g (no M: as it is)
    o_h(i)         = sum_(j <= i) softmax_j(z'_h(i, .)) v_j,  turned back by -i * g_m;   out = W_o [heads side by side]

The frequencies f and g come from the host as float32 (any rescaling already in them); angles are float32 position times float32
frequency with accurate cos and sin.  The three projections are one product with float32 results, so the norm and the rotations
see unrounded sums; q and the cached k, v are in the compute dtype.  Because a head's softmax needs every head's score of the same
(query, key) pair, the attention kernel takes all heads of a query in one block.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..cache.manager import KVSpec, LayerCacheView
from .base import Mixer, StepContext


class MixedHeadAttention(Mixer):
    def __init__(self, hidden: int, num_heads: int, num_kv_heads: int, dim: int, vdim: int, scale: float, w_in: torch.Tensor, w_out: torch.Tensor,
                 eps: float = -1.0, q_norm: Optional[torch.Tensor] = None, k_norm: Optional[torch.Tensor] = None, softcap: Optional[float] = None,
                 mix: Optional[torch.Tensor] = None, freq: Optional[torch.Tensor] = None, rot_dims: int = 0, v_freq: Optional[torch.Tensor] = None,
                 window: int = 0):
        """w_in: W_q | W_k | W_v stacked by rows ([H dim + G dim + G vdim, hidden], compute dtype); freq float32 [rot_dims / 2];
        v_freq float32 [vdim / 2] (None: the values are cached and summed as they are); mix float32 [H, H]."""
        H, G = num_heads, num_kv_heads
        if H % G or w_in.shape != (H * dim + G * dim + G * vdim, hidden) or w_out.shape != (hidden, H * vdim):
            raise ValueError("the attention's weights do not fit the head counts")
        if (q_norm is None) != (k_norm is None) or (q_norm is not None and (q_norm.shape != (dim,) or k_norm.shape != (dim,))):
            raise ValueError("the queries' and keys' norm weights come together and have the keys' size")
        if rot_dims % 2 or rot_dims > dim or (rot_dims and (freq is None or freq.shape != (rot_dims // 2,))):
            raise ValueError("the rotation does not fit the keys")
        if v_freq is not None and v_freq.shape != (vdim // 2,):
            raise ValueError("the values' rotation does not fit their size")
        if mix is not None and mix.shape != (H, H):
            raise ValueError("the mixing matrix is not [heads, heads]")
        if softcap is not None and not softcap > 0:
            raise ValueError("the scores' cap is positive")
        self.hidden, self.H, self.G, self.dim, self.vdim, self.scale, self.eps = hidden, H, G, dim, vdim, float(scale), float(eps)
        self.cap, self.rot_dims, self.window = float(softcap or 0.0), int(rot_dims), int(window)
        f32 = lambda t: None if t is None else t.to(torch.float32).contiguous()
        self.w_in, self.w_out = w_in.contiguous(), w_out.contiguous()
        self.q_norm, self.k_norm, self.mix, self.freq, self.v_freq = f32(q_norm), f32(k_norm), f32(mix), f32(freq), f32(v_freq)
        if self.q_norm is None:
            self.eps = -1.0

    def tensors(self):
        return [t for t in (self.w_in, self.w_out, self.q_norm, self.k_norm, self.mix) if t is not None]

    def cache_spec(self):
        return KVSpec(self.G, self.dim, self.window, 0 if self.vdim == self.dim else self.vdim)

    def forward(self, xn: torch.Tensor, ctx: StepContext, cache: LayerCacheView, residual: torch.Tensor, write_cache: bool = True,
                norm=None) -> None:
        if not write_cache:
            raise ValueError("this attention writes the keys and values it reads")
        T, ws, H, G = ctx.num_tokens, ctx.workspace, self.H, self.G
        meta = ctx.groups[cache.group]
        ps = ops._page_size_of(cache.pages, G, self.dim, self.vdim)
        proj = ops.linear(xn, self.w_in, ws.rows("matt.proj", T, self.w_in.shape[0], torch.float32), ops.LINEAR_F32)
        q = ops.mixed_attn_prepare(proj, ctx.positions, meta.slot_mapping, self.q_norm, self.k_norm, self.eps, self.freq, self.rot_dims, self.v_freq,
                                   ws.rows("matt.q", T, H * self.dim, ctx.dtype), cache.pages, H, G, self.dim, self.vdim, ps)
        att = ops.attention_mixed(q, cache.pages, meta, ctx, ws.rows("matt.out", T, H * self.vdim, ctx.dtype), H, G, self.dim, self.vdim, ps,
                                  self.scale, self.cap, self.mix, self.v_freq, self.window)
        ops.linear(att, self.w_out, residual, ops.LINEAR_ACC_F32)
