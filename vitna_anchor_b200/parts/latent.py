"""Latent attention: queries, keys and values pass through narrow latents, and only the key-value latent is cached.

With H heads, per head `dim` plain and `rot_dim` rotated query/key values and values of size vdim, a query latent of
q_rank and a key-value latent of kv_rank values:

    cq = rms(W_dq xn) * w_q                         q = W_uq cq, per head [dim plain | rot_dim rotated]
    [c_raw | kr_raw] = W_dkv xn                     c = rms(c_raw) * w_kv;  kr = rot(kr_raw), one part shared by all heads
    per head:  k = W_uk c,  v = W_uv c;   score(t, j) = scale (q_plain . k_j + rot(q_rot) . kr_j),  j <= t;  softmax
    out = W_o [heads' outputs side by side]         (gated: head h's output times sigmoid(W_g xn)_h first)

The cache keeps one row [c | kr] a token.  The keys' and values' expansions are folded into their neighbours once, at
load, in float64:  q_plain . (W_uk c) = (W_uk^T q_plain) . c,  so the query product is made with the rows
[W_uk_h^T W_uq_h,plain ; W_uq_h,rot] per head and gives [kv_rank + rot_dim] values a head that are dotted with the cached
row as it is; and  W_o,h (W_uv_h sum_j p_j c_j)  is made with W_o,h W_uv_h  on the weighted sum of the rows' c.  What runs is
an attention with ONE key-value head of size kv_rank + rot_dim whose values are the keys' first kv_rank values (the
framework's kernels for values of their own size, reading them inside the key rows, so that c is cached once), between
two ordinary products.  With a gate on every value instead of one a head (`w_uv` given: out = W_o (sigmoid(W_g xn) * [heads' v side by
side])) the values' expansion cannot be folded into W_o: it runs per head on the weighted sums of c, with the gate, in one kernel
between the attention and the output product.  `window` > 0: position i sees the keys i - window + 1 .. i.
A layer may read the rows that another layer wrote
(`shares_kv`: it has no W_dkv of its own; its run names the other layer's cache and does not write it).

The first product stacks W_dq, W_dkv and W_g and leaves float32; both RMS norms, the rotation's angles (float32 position
times a float32 frequency from the host, accurate cos and sin) and the gate are float32.
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from .. import ops
from ..cache.manager import KVSpec, LayerCacheView
from .base import Mixer, StepContext


class LatentAttention(Mixer):
    def __init__(self, hidden: int, num_heads: int, kv_rank: int, rot_dim: int, q_rank: int, scale: float, eps: float,
                 w_in: torch.Tensor, q_norm: torch.Tensor, kv_norm: Optional[torch.Tensor], w_q: torch.Tensor, w_out: torch.Tensor,
                 freq: torch.Tensor, mag: float, rot_dims: int, interleaved: bool, gated: bool = False, shares_kv: bool = False,
                 window: int = 0, w_uv: Optional[torch.Tensor] = None):
        """w_in: W_dq | W_dkv (unless shares_kv) | W_g (if gated) stacked by rows; w_q [H (kv_rank + rot_dim), q_rank] and
        w_out [hidden, H kv_rank]: the folded matrices (see from_matrices); freq float32 [rot_dims / 2].  With w_uv [H, kv_rank, v_dim]
        (the values' expansion, a head's matrix transposed) the gate has H v_dim values and w_out is the unfolded [hidden, H v_dim]."""
        H = num_heads
        v_dim = 0 if w_uv is None else w_uv.shape[2]
        n_gate = 0 if not gated else (H if w_uv is None else H * v_dim)
        n_in = q_rank + (0 if shares_kv else kv_rank + rot_dim) + n_gate
        if (w_in.shape != (n_in, hidden) or w_q.shape != (H * (kv_rank + rot_dim), q_rank)
                or w_out.shape != (hidden, H * (kv_rank if w_uv is None else v_dim)) or (w_uv is not None and w_uv.shape != (H, kv_rank, v_dim))):
            raise ValueError("latent attention weights do not fit the sizes")
        if window < 0:
            raise ValueError("a window is a number of positions")
        if q_norm.shape != (q_rank,) or (not shares_kv and (kv_norm is None or kv_norm.shape != (kv_rank,))):
            raise ValueError("latent attention norm weights do not fit the ranks")
        if rot_dims % 2 or rot_dims > rot_dim or freq.shape != (rot_dims // 2,):
            raise ValueError("the rotation does not fit the rotated part")
        self.hidden, self.H, self.kv_rank, self.rot_dim, self.q_rank = hidden, H, kv_rank, rot_dim, q_rank
        self.scale, self.eps, self.mag, self.rot_dims, self.interleaved = float(scale), float(eps), float(mag), rot_dims, bool(interleaved)
        self.gated, self.shares_kv = bool(gated), bool(shares_kv)
        self.w_in, self.w_q, self.w_out = w_in.contiguous(), w_q.contiguous(), w_out.contiguous()
        self.q_norm = q_norm.to(torch.float32).contiguous()
        self.kv_norm = None if kv_norm is None else kv_norm.to(torch.float32).contiguous()
        self.freq = freq.to(torch.float32).contiguous()
        self.kv_off = -1 if shares_kv else q_rank
        self.gate_off = n_in - n_gate if gated else -1
        self.window, self.v_dim = int(window), v_dim
        self.w_uv = None if w_uv is None else w_uv.contiguous()

    @classmethod
    def from_matrices(cls, *, hidden: int, num_heads: int, dim: int, rot_dim: int, v_dim: int, kv_rank: int, q_rank: int, scale: float,
                      eps: float, w_dq, q_norm, w_uq, w_dkv, kv_norm, w_uk, w_uv, w_o, w_gate, freq, mag: float, rot_dims: int,
                      interleaved: bool, dtype: torch.dtype, device, window: int = 0, gate_per_value: bool = False) -> "LatentAttention":
        """From the matrices as a checkpoint names them (host tensors; w_dkv None: the layer reads another layer's rows;
        w_gate None: no output gate; gate_per_value: w_gate has H v_dim rows, one for every value, instead of one a head).  The
        folding is done in float64 and rounded once to the compute dtype."""
        H = num_heads
        f64 = lambda t: t.to(torch.float64)
        if (w_uq.shape != (H * (dim + rot_dim), q_rank) or w_uk.shape != (H * dim, kv_rank) or w_uv.shape != (H * v_dim, kv_rank)
                or w_o.shape != (hidden, H * v_dim)):
            raise ValueError("latent attention matrices do not fit the head counts")
        uq = f64(w_uq).reshape(H, dim + rot_dim, q_rank)
        uk = f64(w_uk).reshape(H, dim, kv_rank)
        uv = f64(w_uv).reshape(H, v_dim, kv_rank)
        wo = f64(w_o).reshape(hidden, H, v_dim)
        w_q = torch.cat([torch.einsum("hdr,hdq->hrq", uk, uq[:, :dim]), uq[:, dim:]], dim=1).reshape(H * (kv_rank + rot_dim), q_rank)
        per_value = bool(gate_per_value) and w_gate is not None
        w_out = f64(w_o) if per_value else torch.einsum("whv,hvr->whr", wo, uv).reshape(hidden, H * kv_rank)
        w_in = torch.cat([f64(t) for t in (w_dq, w_dkv, w_gate) if t is not None], dim=0)
        put = lambda t: t.to(dtype=dtype).to(device)
        f32 = lambda t: None if t is None else t.to(torch.float32).to(device)
        return cls(hidden, H, kv_rank, rot_dim, q_rank, scale, eps, put(w_in), f32(q_norm), f32(kv_norm), put(w_q), put(w_out),
                   torch.as_tensor(np.asarray(freq, dtype=np.float32)).to(device), mag, rot_dims, interleaved, gated=w_gate is not None,
                   shares_kv=w_dkv is None, window=window, w_uv=put(uv.transpose(1, 2).contiguous()) if per_value else None)

    def tensors(self):
        return [self.w_in, self.w_q, self.w_out, self.q_norm] + [t for t in (self.kv_norm, self.w_uv) if t is not None]

    def cache_spec(self):
        return KVSpec(1, self.kv_rank + self.rot_dim, self.window, self.kv_rank, value_in_key=True)

    def forward(self, xn: torch.Tensor, ctx: StepContext, cache: LayerCacheView, residual: torch.Tensor, write_cache: bool = True,
                norm=None) -> None:
        if write_cache == self.shares_kv:
            raise ValueError("a latent attention layer writes the cache rows exactly when it has a key-value latent of its own")
        T, ws, H = ctx.num_tokens, ctx.workspace, self.H
        hd = self.kv_rank + self.rot_dim
        meta = ctx.groups[cache.group]
        ps = ops._page_size_of(cache.pages, 1, hd, 0)
        proj = ops.linear(xn, self.w_in, ws.rows("lat.proj", T, self.w_in.shape[0], torch.float32), ops.LINEAR_F32)
        cq = ops.latent_prepare(proj, self.q_rank, self.q_norm, ws.rows("lat.cq", T, self.q_rank, ctx.dtype), self.eps, ctx.positions,
                                self.freq, self.mag, self.rot_dims, self.interleaved, kv_off=self.kv_off, kv_rank=self.kv_rank,
                                rot_dim=self.rot_dim, kv_norm_w=self.kv_norm, slot_mapping=meta.slot_mapping,
                                cache_layer=cache.pages if write_cache else None, page_size=ps)
        q = ops.linear(cq, self.w_q, ws.rows("lat.q", T, H * hd, ctx.dtype), ops.LINEAR_SAME)
        ops.latent_rotate_q(q, ctx.positions, self.freq, self.mag, H, self.kv_rank, self.rot_dim, self.rot_dims, self.interleaved)
        att = ops.attention_biased(q, cache.pages, meta, ctx, ws.rows("lat.out", T, H * self.kv_rank, ctx.dtype), H, 1, hd, self.kv_rank, ps,
                                   self.scale, self.window, None, v_in_key=True)
        if self.w_uv is not None:
            att = ops.latent_expand_gate(att, self.w_uv, proj if self.gated else None, max(self.gate_off, 0), H, self.kv_rank, self.v_dim,
                                         ws.rows("lat.vals", T, H * self.v_dim, ctx.dtype))
        elif self.gated:
            ops.head_gate(att, proj, self.gate_off, H)
        ops.linear(att, self.w_out, residual, ops.LINEAR_ACC_F32)
