"""Differential attention: two softmax score maps a head over one set of values, subtracted.

With H query heads, G key-value heads (query head h reads key-value head h // (H / G)), `dim` values per head and map for queries
and keys and vdim per head for values:

    q, k, v = conv(W_q x + b_q), conv(W_k x + b_k), conv(W_v x + b_v)      a short causal convolution a channel (taps weights,
                                                                           zeros before the sequence's start), straight after the product
    q, k     per head and map: RMS norm over dim with a weight shared by all heads and maps, then pairs (2i, 2i+1) of the first
             rot_dims values turned by position * f_i (f from the host, any rescaling already in it; cos and sin times `mag`)
    a1, a2   = softmax(scale q1 . k1) v,  softmax(scale q2 . k2) v          causal, per head, the same v for both maps
    o        = (a1 - lambda a2) / rms(a1 - lambda a2) * (1 - diff)          lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff, one number a layer
    out      = W_o (o * sigmoid(W_g x)) + b_o

It runs as ONE attention with 2H query heads, 2G key heads and G value heads over the paged cache (the attention kernels' form in
which neighbouring key heads read one value head), between two products and two small kernels.  The first product stacks W_q, W_k,
W_v and W_g and leaves float32; the convolution's memory (the last taps - 1 projected rows of a request) is a fixed-size state BESIDE
the pages.  A layer may read the keys and values that another layer cached (`shares_kv`: it has no W_k, W_v of its own, its run names
the other layer's cache and does not write it); its queries, and their convolution's memory, are its own.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import ops
from ..cache.manager import KVSpec, LayerCacheView, StateSpec
from .base import Mixer, StepContext


class DiffAttention(Mixer):
    def __init__(self, hidden: int, num_heads: int, num_kv_heads: int, dim: int, vdim: int, taps: int, scale: float, diff: float, lam: float,
                 eps: float, w_in: torch.Tensor, b_in: Optional[torch.Tensor], conv: Optional[torch.Tensor], q_norm: torch.Tensor,
                 k_norm: Optional[torch.Tensor], w_out: torch.Tensor, b_out: Optional[torch.Tensor], freq: Optional[torch.Tensor] = None,
                 mag: float = 1.0, rot_dims: int = 0, shares_kv: bool = False):
        """w_in: W_q | W_k | W_v (the last two unless shares_kv) | W_g stacked by rows, compute dtype; b_in float32 over the same rows
        (zeros under W_g) or None; conv float32 [channels of q, k, v; taps] or None (no convolution); freq float32 [rot_dims / 2]."""
        H, G = num_heads, num_kv_heads
        if H % G:
            raise ValueError("query heads do not divide into key-value heads")
        C = ops.diff_attn_channels(H, G, dim, vdim, not shares_kv)
        if w_in.shape != (C + H * vdim, hidden) or w_out.shape != (hidden, H * vdim):
            raise ValueError("differential attention weights do not fit the head counts")
        if q_norm.shape != (dim,) or (not shares_kv and (k_norm is None or k_norm.shape != (dim,))):
            raise ValueError("differential attention norm weights do not fit the head size")
        if conv is None:
            taps = 1
        elif taps < 1 or conv.shape != (C, taps):
            raise ValueError("the convolution's weights are not [channels, taps]")
        if rot_dims % 2 or rot_dims > dim or (rot_dims and (freq is None or freq.shape != (rot_dims // 2,))):
            raise ValueError("the rotation does not fit the head size")
        self.hidden, self.H, self.G, self.dim, self.vdim, self.taps = hidden, H, G, dim, vdim, int(taps)
        self.scale, self.diff, self.lam, self.eps, self.mag, self.rot_dims = float(scale), float(diff), float(lam), float(eps), float(mag), rot_dims
        self.shares_kv, self.channels = bool(shares_kv), C
        f32 = lambda t: None if t is None else t.to(torch.float32).contiguous()
        self.w_in, self.w_out = w_in.contiguous(), w_out.contiguous()
        self.b_in, self.b_out, self.conv, self.q_norm, self.k_norm, self.freq = f32(b_in), f32(b_out), f32(conv), f32(q_norm), f32(k_norm), f32(freq)
        if self.b_in is not None and self.b_in.shape != (C + H * vdim,):
            raise ValueError("the bias of the first product does not fit its rows")

    @staticmethod
    def lambda_of(lq1, lk1, lq2, lk2, diff: float) -> float:
        """exp(lq1 . lk1) - exp(lq2 . lk2) + diff, in float32 as the model's other scalars."""
        f = lambda t: t.detach().to(torch.float32).cpu()
        return float(torch.exp((f(lq1) * f(lk1)).sum()) - torch.exp((f(lq2) * f(lk2)).sum()) + torch.tensor(diff, dtype=torch.float32))

    def tensors(self):
        return [t for t in (self.w_in, self.b_in, self.conv, self.q_norm, self.k_norm, self.w_out, self.b_out) if t is not None]

    def cache_spec(self):
        return KVSpec(2 * self.G, self.dim, 0, self.vdim, v_share=2)

    def state_spec(self):
        if self.conv is None or self.taps <= 1:
            return None
        return StateSpec(((self.taps - 1) * self.channels,), torch.float32)

    def forward(self, xn: torch.Tensor, ctx: StepContext, cache: LayerCacheView, residual: torch.Tensor, write_cache: bool = True,
                norm=None) -> None:
        if write_cache == self.shares_kv:
            raise ValueError("a differential attention layer writes the cache exactly when it has keys and values of its own")
        T, ws, H, G, dim, vdim = ctx.num_tokens, ctx.workspace, self.H, self.G, self.dim, self.vdim
        meta = ctx.groups[cache.group]
        ps = ops._page_size_of(cache.pages, 2 * G, dim, vdim, 2)
        tail = cache.state if self.state_spec() is not None else None
        proj = ops.linear(xn, self.w_in, ws.rows("datt.proj", T, self.w_in.shape[0], torch.float32), ops.LINEAR_F32)
        q = ops.diff_attn_prepare(proj, self.b_in, self.conv, self.taps, tail, ctx, self.q_norm, self.k_norm, self.eps, self.freq, self.mag,
                                  self.rot_dims, H, G, dim, vdim, write_cache, meta.slot_mapping, cache.pages, ps,
                                  ws.rows("datt.q", T, 2 * H * dim, ctx.dtype), self.b_out, residual)
        att = ops.attention_biased(q, cache.pages, meta, ctx, ws.rows("datt.att", T, 2 * H * vdim, ctx.dtype), 2 * H, 2 * G, dim, vdim, ps,
                                   self.scale, 0, None, v_in_key=False, v_share=2)
        out = ops.diff_attn_combine(att, proj, self.channels, self.lam, self.diff, self.eps, H, G, vdim,
                                    ws.rows("datt.out", T, H * vdim, ctx.dtype), self.b_in, self.taps, self.channels, tail, ctx)
        ops.linear(out, self.w_out, residual, ops.LINEAR_ACC_F32)
