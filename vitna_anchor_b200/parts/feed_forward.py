"""SwiGLU feed-forward: y = W_down (silu(W_gate xn) * (W_up xn)), added into the residual stream
(engine/src/model.c:962-972; silu(g) = g / (1 + exp(-g)), engine/src/ops.c:283-288).
The gate and up matrices are stacked by rows so that one product reads xn once.

With another activation than silu (`activation`, one of ops.ACTIVATIONS) it is the same gated form, y = W_down (act(W_gate xn) * (W_up xn)).

The dense feed-forward: y = W_down act(W_up xn), act one of ops.ACTIVATIONS (the erf or the tanh form of gelu, silu), or "xielu":
act(z) = softplus(p) z^2 + z/2 for z > 0 and (1/2 + softplus(q)) (e^z - 1 - z) + z/2 otherwise, with the layer's two numbers (p, q).

The clamped gated feed-forward: g = min(W_gate xn, L), u = clamp(W_up xn, -L, L), y = W_down (g sigmoid(alpha g) (u + 1)).

The routed feed-forward: a router chooses `top` of E small gated feed-forwards per token (the largest logits; their weights
the softmax over the chosen logits alone); the weighted sum of their outputs, plus, if there is one, a feed-forward that every
token uses.  Instead of a router a table [vocab, top] may name the experts of every token id, each weighted 1 / top.  An expert's
gate is one of the gated epilogues' activations, or "clamped": the clamped gated form above with `limit` and `alpha`."""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import ops
from .base import FeedForward, StepContext


class SwiGLU(FeedForward):
    def __init__(self, hidden: int, intermediate: int, w_gate_up: torch.Tensor, w_down: torch.Tensor, activation: str = "silu"):
        if w_gate_up.shape != (2 * intermediate, hidden) or w_down.shape != (hidden, intermediate):
            raise ValueError("feed-forward weights do not fit the sizes")
        if activation not in ops.ACTIVATIONS:
            raise ValueError(f"activation {activation!r} is not one of {sorted(ops.ACTIVATIONS)}")
        self.hidden, self.intermediate, self.activation = hidden, intermediate, activation
        self.w_gate_up, self.w_down = w_gate_up.contiguous(), w_down.contiguous()

    def tensors(self):
        return [self.w_gate_up, self.w_down]

    def fuses_norm(self, norm, ctx: StepContext) -> bool:
        return (self.activation == "silu" and norm.as_rms() is not None
                and ops.fused_norm_takes(ctx.dtype, ctx.num_tokens, self.hidden, 2 * self.intermediate))

    def forward(self, xn: torch.Tensor, ctx: StepContext, residual: torch.Tensor, norm=None) -> None:
        T = ctx.num_tokens
        ws = ctx.workspace
        act_buf = ws.rows("ffn.act", T, self.intermediate, ctx.dtype)
        if self.activation != "silu":
            act = ops.linear_gated(xn, self.w_gate_up, ws.rows("ffn.gu", T, 2 * self.intermediate, ctx.dtype), act_buf, self.activation)
        elif norm is not None:
            # few rows: norm, gate and up, and silu(gate) * up in one launch
            nw, eps = norm.as_rms()
            act = ops.linear_skinny(xn, self.w_gate_up, act_buf, ops.EPI_SWIGLU, norm_weight=nw, eps=eps)
        elif (xn.stride(0) % 8 == 0 and xn.data_ptr() % 16 == 0
              and ops.skinny_takes(ctx.dtype, T, self.hidden, 2 * self.intermediate)):
            # a few dozen rows: the norm ran once for all of them; gate, up and silu(gate) * up in one launch
            act = ops.linear_skinny(xn, self.w_gate_up, act_buf, ops.EPI_SWIGLU)
        elif T > ops.SKINNY_MAX_ROWS and self.intermediate % 8 == 0 and ops.tcgen05_takes(xn, self.w_gate_up):
            # prompt-sized batch in bfloat16: gate, up and silu(gate) * up in one tcgen05 kernel
            act = ops.linear_tcgen05_swiglu(xn, self.w_gate_up, act_buf)
        else:
            gu = ops.linear(xn, self.w_gate_up, ws.rows("ffn.gu", T, 2 * self.intermediate, ctx.dtype), ops.LINEAR_SAME)
            act = ops.silu_mul(gu, act_buf)
        ops.linear(act, self.w_down, residual, ops.LINEAR_ACC_F32)


class DenseMLP(FeedForward):
    def __init__(self, hidden: int, intermediate: int, w_up: torch.Tensor, w_down: torch.Tensor, activation: str = "gelu", act_params=None):
        """act_params: for "xielu" the layer's two numbers (p, q) as the checkpoint holds them."""
        if w_up.shape != (intermediate, hidden) or w_down.shape != (hidden, intermediate):
            raise ValueError("feed-forward weights do not fit the sizes")
        if activation not in ops.ACTIVATIONS and activation != "xielu":
            raise ValueError(f"activation {activation!r} is not one of {sorted(ops.ACTIVATIONS) + ['xielu']}")
        self.hidden, self.intermediate, self.activation = hidden, intermediate, activation
        self.w_up, self.w_down = w_up.contiguous(), w_down.contiguous()
        self.a_pos = self.a_neg = 0.0
        if activation == "xielu":
            if act_params is None or len(act_params) != 2:
                raise ValueError("xielu takes the layer's two numbers")
            p, q = (float(v) for v in act_params)
            softplus = lambda z: max(z, 0.0) + math.log1p(math.exp(-abs(z)))
            self.a_pos, self.a_neg = softplus(p), 0.5 + softplus(q)

    def tensors(self):
        return [self.w_up, self.w_down]

    def forward(self, xn: torch.Tensor, ctx: StepContext, residual: torch.Tensor, norm=None) -> None:
        buf = ctx.workspace.rows("ffn.act", ctx.num_tokens, self.intermediate, ctx.dtype)
        if self.activation == "xielu":
            act = ops.linear_xielu(xn, self.w_up, buf, self.a_pos, self.a_neg)
        else:
            act = ops.linear_act(xn, self.w_up, buf, self.activation)
        ops.linear(act, self.w_down, residual, ops.LINEAR_ACC_F32)


class ClampedGLU(FeedForward):
    def __init__(self, hidden: int, intermediate: int, w_gate_up: torch.Tensor, w_down: torch.Tensor, limit: float, alpha: float = 1.702):
        if w_gate_up.shape != (2 * intermediate, hidden) or w_down.shape != (hidden, intermediate):
            raise ValueError("feed-forward weights do not fit the sizes")
        if not limit > 0:
            raise ValueError("the clamp's limit is positive")
        self.hidden, self.intermediate, self.limit, self.alpha = hidden, intermediate, float(limit), float(alpha)
        self.w_gate_up, self.w_down = w_gate_up.contiguous(), w_down.contiguous()

    def tensors(self):
        return [self.w_gate_up, self.w_down]

    def forward(self, xn: torch.Tensor, ctx: StepContext, residual: torch.Tensor, norm=None) -> None:
        T, ws = ctx.num_tokens, ctx.workspace
        act = ops.linear_glu_clamped(xn, self.w_gate_up, ws.rows("ffn.gu", T, 2 * self.intermediate, ctx.dtype),
                                     ws.rows("ffn.act", T, self.intermediate, ctx.dtype), self.limit, self.alpha)
        ops.linear(act, self.w_down, residual, ops.LINEAR_ACC_F32)


class RoutedExperts(FeedForward):
    """w_router float32 [E, hidden] (+ b_router [E]); w_gate_up [E, 2 ff, hidden] (an expert's gate rows, then its up rows) and
    w_down [E, hidden, ff] in the compute dtype; `shared`: a FeedForward every token passes as well (or None).  The router's
    logits are float32 sums over the (compute dtype) input.  Which experts run never comes to the host: the kernels read the
    choice on the device, so the part is replayed faithfully from a graph.  Steps with at least GROUPED_FROM (token, expert) pairs in
    bfloat16 run the experts as products of row groups on the tensor cores; shorter steps and float32 read each token's experts' rows
    directly."""

    GROUPED_FROM = 256

    def __init__(self, hidden: int, intermediate: int, experts: int, top: int, w_router: Optional[torch.Tensor], b_router: Optional[torch.Tensor],
                 w_gate_up: torch.Tensor, w_down: torch.Tensor, shared: Optional[FeedForward] = None, activation: str = "silu",
                 table: Optional[torch.Tensor] = None, limit: float = 0.0, alpha: float = 1.702):
        """Either w_router (float32 [E, hidden], with or without b_router) or table (int32 [vocab, >= top]: the experts of every token
        id, each weighted 1 / top).  activation: one of the gated epilogues' or "clamped" (with limit and alpha)."""
        E = experts
        if w_gate_up.shape != (E, 2 * intermediate, hidden) or w_down.shape != (E, hidden, intermediate):
            raise ValueError("the experts' weights do not fit the sizes")
        if (w_router is None) == (table is None):
            raise ValueError("the experts are chosen by a router or by a table, one of the two")
        if w_router is not None and w_router.shape != (E, hidden):
            raise ValueError("the router does not fit the experts")
        if b_router is not None and (w_router is None or b_router.shape != (E,)):
            raise ValueError("the router's bias does not fit the experts")
        if table is not None and (table.dim() != 2 or table.shape[1] < top or table.dtype != torch.int32):
            raise ValueError("the experts' table is int32 [vocab, top]")
        if not 1 <= top <= min(E, 32):
            raise ValueError("a token uses between one and min(experts, 32) experts")
        if activation == "clamped" and not limit > 0:
            raise ValueError("the clamp's limit is positive")
        self.hidden, self.intermediate, self.E, self.top, self.activation, self.shared = hidden, intermediate, E, int(top), activation, shared
        self.limit, self.alpha = float(limit), float(alpha)
        self.w_router = None if w_router is None else w_router.to(torch.float32).contiguous()
        self.b_router = None if b_router is None else b_router.to(torch.float32).contiguous()
        self.table = None if table is None else table.contiguous()
        self.w_gate_up, self.w_down = w_gate_up.contiguous(), w_down.contiguous()

    def tensors(self):
        return [t for t in (self.w_router, self.b_router, self.table, self.w_gate_up, self.w_down) if t is not None] + \
            ([] if self.shared is None else self.shared.tensors())

    def weight_bytes(self) -> int:
        """What one token reads: the router (or its row of the table), its `top` experts, the shared feed-forward."""
        one = (self.w_gate_up[0].numel() + self.w_down[0].numel()) * self.w_down.element_size()
        choose = self.w_router.numel() * 4 if self.w_router is not None else 4 * self.top
        return choose + self.top * one + (0 if self.shared is None else self.shared.weight_bytes())

    def forward(self, xn: torch.Tensor, ctx: StepContext, residual: torch.Tensor, norm=None) -> None:
        T, ws = ctx.num_tokens, ctx.workspace
        ids = ws.rows("moe.ids", T, self.top, torch.int32)
        wts = ws.rows("moe.wts", T, self.top, torch.float32)
        if self.table is not None:
            ops.experts_route_table(ctx.tokens, self.table, self.E, self.top, ids, wts)
        else:
            ops.experts_route(xn, self.w_router, self.b_router, self.top, ids, wts)
        if T * self.top >= self.GROUPED_FROM and ops.experts_grouped_takes(xn, self.w_gate_up, self.w_down):
            # a prompt's portion in bfloat16: the copies sorted expert by expert, two products of row groups on the tensor cores
            rows, rows_max = ops.experts_grouped_rows(T, self.top, self.E), ops.experts_grouped_rows(ws.max_tokens, self.top, self.E)
            key = f"{self.top}/{self.E}"
            xs = ws.flat(f"moe.xs/{key}/{self.hidden}", rows_max * self.hidden, ctx.dtype)[:rows * self.hidden].view(rows, self.hidden)
            act = ws.flat(f"moe.gact/{key}/{self.intermediate}", rows_max * self.intermediate, ctx.dtype)[:rows * self.intermediate].view(rows, self.intermediate)
            o = ws.flat(f"moe.o/{key}/{self.hidden}", rows_max * self.hidden, torch.float32)[:rows * self.hidden].view(rows, self.hidden)
            ops.experts_apply_grouped(xn, self.w_gate_up, self.w_down, ids, wts, ws.rows("moe.pos", T, self.top, torch.int32),
                                      ws.flat(f"moe.row_token/{key}", rows_max, torch.int32)[:rows],
                                      ws.flat(f"moe.tile_group/{key}", rows_max // 128, torch.int32)[:rows // 128], xs, act, o, residual, self.activation,
                                      self.limit, self.alpha,
                                      None if self.activation != "clamped" else
                                      ws.flat(f"moe.gu/{key}/{self.intermediate}", rows_max * 2 * self.intermediate, ctx.dtype)[:rows * 2 * self.intermediate].view(rows, 2 * self.intermediate))
        else:
            act = ws.flat(f"moe.act/{self.top}/{self.intermediate}", ws.max_tokens * self.top * self.intermediate, ctx.dtype)
            ops.experts_apply(xn, self.w_gate_up, self.w_down, ids, wts, act[:T * self.top * self.intermediate].view(T * self.top, self.intermediate),
                              residual, self.activation, self.limit, self.alpha)
        if self.shared is not None:
            self.shared.forward(xn, ctx, residual)
