"""The matrix memory with exponential gates (mLSTM): a recurrent mixer whose state per head is a matrix, a vector and a number.

With H heads, keys and queries of size dim and values of size vdim:

    q = W_q x * dim^-1/2,  k = W_k x,  v = W_v x
    i = cap tanh((W_i x + b_i) / cap),  f = log sigmoid(cap tanh((W_f x + b_f) / cap))          one each per head, logarithms of the gates
    m_t = max(f_t + m_(t-1), i_t);   S_t = e^(f_t + m_(t-1) - m_t) S_(t-1) + e^(i_t - m_t) k_t v_t^T;   n_t the same with k_t alone
    o_t = S_t^T q_t / (max(|n_t . q_t|, e^(-m_t)) + 1e-6)                                      S, n start at zero, m at 0
    out = W_o (o / rms(o) per head * w_norm * sigmoid(W_g x))                                  w_norm over all heads' values

The six projections are ONE product with float32 results; gates, the running maximum, the state and the output's norm are float32.
A request's state lives in its state slot and is carried from step to step; the recurrence runs token after token in both dtypes, so
the result does not depend on how a prompt is cut.  All launches depend on the step's counts and device arrays alone.
"""
from __future__ import annotations

import torch

from .. import ops
from ..cache.manager import LayerCacheView, StateSpec
from .base import Mixer, StepContext


class MatrixLSTM(Mixer):
    def __init__(self, hidden: int, num_heads: int, dim: int, vdim: int, gate_cap: float, w_in: torch.Tensor, gate_bias: torch.Tensor,
                 norm_weight: torch.Tensor, w_out: torch.Tensor, eps: float):
        """w_in: W_q | W_k | W_v | W_g | W_i | W_f stacked by rows ([2 H dim + 2 H vdim + 2 H, hidden], compute dtype); gate_bias: b_i | b_f."""
        H = num_heads
        if w_in.shape != (2 * H * dim + 2 * H * vdim + 2 * H, hidden) or w_out.shape != (hidden, H * vdim):
            raise ValueError("the matrix memory's weights do not fit the head counts")
        if gate_bias.shape != (2 * H,) or norm_weight.shape != (H * vdim,):
            raise ValueError("the matrix memory's vectors do not fit the head counts")
        if not gate_cap > 0:
            raise ValueError("the gates' cap is positive")
        if dim > ops.mlstm_max_dim():
            raise ValueError(f"keys of {dim} values: the recurrence keeps a column of the state in registers, up to {ops.mlstm_max_dim()} rows")
        self.hidden, self.H, self.dim, self.vdim, self.cap, self.eps = hidden, H, dim, vdim, float(gate_cap), float(eps)
        self.w_in, self.w_out = w_in.contiguous(), w_out.contiguous()
        self.gate_bias = gate_bias.to(torch.float32).contiguous()
        self.norm_weight = norm_weight.to(torch.float32).contiguous()

    def tensors(self):
        return [self.w_in, self.gate_bias, self.norm_weight, self.w_out]

    def cache_spec(self):
        return StateSpec((ops.mlstm_state_floats(self.H, self.dim, self.vdim),), torch.float32)

    def forward(self, xn: torch.Tensor, ctx: StepContext, cache: LayerCacheView, residual: torch.Tensor, write_cache: bool = True,
                norm=None) -> None:
        if not write_cache:
            raise ValueError("a recurrent mixer has no cache that another run could read")
        T, ws, HV = ctx.num_tokens, ctx.workspace, self.H * self.vdim
        proj = ops.linear(xn, self.w_in, ws.rows("mlstm.proj", T, self.w_in.shape[0], torch.float32), ops.LINEAR_F32)
        out = ops.mlstm(proj, self.gate_bias, self.cap, self.norm_weight, self.eps, ctx, cache.state, ws.rows("mlstm.o", T, self.H * (self.vdim + 2), torch.float32),
                        ws.rows("mlstm.out", T, HV, ctx.dtype), self.H, self.dim, self.vdim)
        ops.linear(out, self.w_out, residual, ops.LINEAR_ACC_F32)
