"""Gated linear attention: a recurrent mixer whose state per head is a matrix that decays per key channel.

With H heads, keys and queries of size dim and values of size vdim:

    q = W_q x * dim^-1/2,  k = W_k x,  v = W_v x
    a = sigmoid(W_a2 (W_a1 x) + b)^(1/tau)                      one decay per head and key channel (W_a1 narrow, W_a2 wide)
    S_t = diag(a_t) S_(t-1) + k_t v_t^T;   o_t = S_t^T q_t      S starts at zero
    out = W_o (o / rms(o) per head * w_norm * silu(W_g x))      w_norm [vdim], shared by the heads

The five projections q, k, v, g and W_a1 x are ONE product with float32 results; the wide half of the decays' projection, the
decays (through their logarithm), the state and the output's norm are float32.  A request's state lives in its state slot and is
carried from step to step; the recurrence runs token after token in both dtypes, so the result does not depend on how a prompt is
cut.  All launches depend on the step's counts and device arrays alone.
"""
from __future__ import annotations

import torch

from .. import ops
from ..cache.manager import LayerCacheView, StateSpec
from .base import Mixer, StepContext


class GatedLinearAttention(Mixer):
    def __init__(self, hidden: int, num_heads: int, dim: int, vdim: int, tau: float, w_in: torch.Tensor, w_a2: torch.Tensor, a_bias: torch.Tensor,
                 norm_weight: torch.Tensor, w_out: torch.Tensor, eps: float):
        """w_in: W_q | W_k | W_v | W_g | W_a1 stacked by rows ([2 H dim + 2 H vdim + rank, hidden], compute dtype); w_a2 [H dim, rank] and
        a_bias [H dim] (kept in float32); norm_weight [vdim]."""
        H = num_heads
        rank = w_a2.shape[1]
        if w_in.shape != (2 * H * dim + 2 * H * vdim + rank, hidden) or w_out.shape != (hidden, H * vdim) or w_a2.shape != (H * dim, rank):
            raise ValueError("the gated linear attention's weights do not fit the head counts")
        if a_bias.shape != (H * dim,) or norm_weight.shape != (vdim,):
            raise ValueError("the gated linear attention's vectors do not fit the head counts")
        if not tau > 0:
            raise ValueError("the decays' temperature is positive")
        if dim > ops.gla_max_dim():
            raise ValueError(f"keys of {dim} values: the recurrence keeps a column of the state in registers, up to {ops.gla_max_dim()} rows")
        self.hidden, self.H, self.dim, self.vdim, self.tau, self.eps, self.rank = hidden, H, dim, vdim, float(tau), float(eps), rank
        self.w_in, self.w_out = w_in.contiguous(), w_out.contiguous()
        self.a2t = w_a2.to(torch.float32).t().contiguous()          # [rank, H dim]: neighbouring threads read neighbouring channels
        self.a_bias = a_bias.to(torch.float32).contiguous()
        self.norm_weight = norm_weight.to(torch.float32).contiguous()
        self.gate_off = 2 * H * dim + H * vdim
        self.a_off = self.gate_off + H * vdim

    def tensors(self):
        return [self.w_in, self.a2t, self.a_bias, self.norm_weight, self.w_out]

    def cache_spec(self):
        return StateSpec((ops.gla_state_floats(self.H, self.dim, self.vdim),), torch.float32)

    def forward(self, xn: torch.Tensor, ctx: StepContext, cache: LayerCacheView, residual: torch.Tensor, write_cache: bool = True,
                norm=None) -> None:
        if not write_cache:
            raise ValueError("a recurrent mixer has no cache that another run could read")
        T, ws, HV = ctx.num_tokens, ctx.workspace, self.H * self.vdim
        proj = ops.linear(xn, self.w_in, ws.rows("gla.proj", T, self.w_in.shape[0], torch.float32), ops.LINEAR_F32)
        out = ops.gla(proj, self.a_off, self.a2t, self.a_bias, self.tau, self.norm_weight, self.eps, ctx, cache.state,
                      ws.rows("gla.decay", T, self.H * self.dim, torch.float32), ws.rows("gla.o", T, HV, torch.float32),
                      ws.rows("gla.out", T, HV, ctx.dtype), self.H, self.dim, self.vdim, self.gate_off)
        ops.linear(out, self.w_out, residual, ops.LINEAR_ACC_F32)
