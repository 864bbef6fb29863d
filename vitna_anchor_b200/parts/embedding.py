"""Token embedding and the output matrix.

x = the token's row, widened to float32, unscaled (engine/src/model.c:893-895);
logits = W_out xn in float32, where W_out is lm_head.weight or, when the model
ties them, the embedding table itself (engine/src/model.c:315-321, 975-978).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from .base import LogitsOutput, StepContext, TokenInput


class Embedding(TokenInput):
    def __init__(self, vocab: int, hidden: int, table: torch.Tensor):
        if table.shape != (vocab, hidden):
            raise ValueError("the embedding table does not fit the sizes")
        self.vocab, self.hidden, self.table = vocab, hidden, table.contiguous()

    def tensors(self):
        return [self.table]

    def forward(self, ctx: StepContext) -> torch.Tensor:
        x = ctx.workspace.rows("x", ctx.num_tokens, self.hidden, torch.float32)
        return ops.embed_rows(self.table, ctx.tokens, x)


class NormedEmbedding(Embedding):
    """x = norm(the token's row): the rows are normed in float32 where they lie.  `norm` is any norm with in_place()."""

    def __init__(self, vocab: int, hidden: int, table: torch.Tensor, norm):
        super().__init__(vocab, hidden, table)
        if not hasattr(norm, "in_place"):
            raise ValueError("the embedding's norm cannot norm float32 rows in place")
        self.norm = norm

    def tensors(self):
        return [self.table] + self.norm.tensors()

    def weight_bytes(self) -> int:
        return self.norm.weight_bytes()         # a row per token is read, not the table

    def forward(self, ctx: StepContext) -> torch.Tensor:
        return self.norm.in_place(super().forward(ctx))


class ScaledEmbedding(TokenInput):
    """x = scale * the token's row + a learned row for the token's position (unscaled), written `copies` times side by
    side: float32 [T, copies * hidden], the form a model with several residual streams starts from."""

    def __init__(self, vocab: int, hidden: int, table: torch.Tensor, scale: float = 1.0, positions: Optional[torch.Tensor] = None,
                 copies: int = 1):
        if table.shape != (vocab, hidden) or (positions is not None and (positions.dim() != 2 or positions.shape[1] != hidden)):
            raise ValueError("the embedding tables do not fit the sizes")
        self.vocab, self.hidden, self.scale, self.copies = vocab, hidden, float(scale), int(copies)
        self.table = table.contiguous()
        self.positions = None if positions is None else positions.to(torch.float32).contiguous()

    def tensors(self):
        return [self.table] + ([] if self.positions is None else [self.positions])

    def weight_bytes(self) -> int:
        return 0                     # a row per token is read, not the tables

    def forward(self, ctx: StepContext) -> torch.Tensor:
        x = ctx.workspace.rows("x", ctx.num_tokens, self.copies * self.hidden, torch.float32)
        return ops.embed_scaled(self.table, ctx.tokens, ctx.positions, self.positions, self.scale, x, self.copies)


class HashedPairEmbedding(TokenInput):
    """x = the token's row + a row of a second table chosen by a hash of the previous and the current token:
    row (prev * mul_prev + cur * mul_cur) mod buckets, and row `buckets` (the last) for a request's first token.  The token
    before a step's first one is one int32 word of the request's state slot (state_spec), moved on by the kernel."""

    def __init__(self, vocab: int, hidden: int, table: torch.Tensor, second: torch.Tensor, buckets: int, mul_prev: int, mul_cur: int):
        if table.shape != (vocab, hidden) or second.shape != (buckets + 1, hidden) or buckets < 1:
            raise ValueError("the embedding tables do not fit the sizes")
        self.vocab, self.hidden, self.buckets, self.mul_prev, self.mul_cur = vocab, hidden, int(buckets), int(mul_prev), int(mul_cur)
        self.table, self.second = table.contiguous(), second.contiguous()

    def tensors(self):
        return [self.table, self.second]

    def weight_bytes(self) -> int:
        return 0                     # two rows per token are read, not the tables

    def state_spec(self):
        from ..cache.manager import StateSpec
        return StateSpec((1,), torch.int32)

    def forward(self, ctx: StepContext, state: Optional[torch.Tensor] = None) -> torch.Tensor:
        if state is None:
            raise ValueError("the hashed embedding needs its word of the requests' state slots")
        x = ctx.workspace.rows("x", ctx.num_tokens, self.hidden, torch.float32)
        return ops.embed_hashed(self.table, self.second, ctx.tokens, ctx.positions, ctx.token_seg, ctx.seg_starts, ctx.seg_slots, state, x, None,
                                self.buckets, self.mul_prev, self.mul_cur)


class LMHead(LogitsOutput):
    def __init__(self, vocab: int, hidden: int, weight: torch.Tensor):
        if weight.shape != (vocab, hidden):
            raise ValueError("the output matrix does not fit the sizes")
        self.vocab, self.hidden, self.weight = vocab, hidden, weight.contiguous()

    def tensors(self):
        return [self.weight]

    def _out(self, rows: int, out: Optional[torch.Tensor], device) -> torch.Tensor:
        if out is None:
            return torch.empty((rows, self.vocab), dtype=torch.float32, device=device)
        if out.shape != (rows, self.vocab) or out.dtype != torch.float32 or not out.is_contiguous():
            raise ValueError("the logits buffer is not a contiguous float32 [rows, vocab]")
        return out

    def forward(self, xn: torch.Tensor, ctx: StepContext, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """xn [R, hidden] in the compute dtype -> float32 logits [R, vocab] (in `out`, or a new tensor)."""
        return ops.linear(xn, self.weight, self._out(xn.shape[0], out, xn.device), ops.LINEAR_F32)

    def fuses_norm(self, norm, ctx: StepContext, rows: int) -> bool:
        return norm.as_rms() is not None and ops.fused_norm_takes(ctx.dtype, rows, self.hidden, self.vocab)

    def forward_normed(self, x: torch.Tensor, rows: torch.Tensor, norm, ctx: StepContext,
                       out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """logits of rmsnorm(x[rows]) in one launch (few rows); x is the float32 residual stream."""
        nw, eps = norm.as_rms()
        return ops.linear_skinny(x, self.weight, self._out(rows.shape[0], out, x.device), ops.EPI_F32, norm_weight=nw, eps=eps, rows=rows)


class CappedLMHead(LMHead):
    """logits <- cap * tanh(logits / cap) after the output matrix (float32, in place)."""

    def __init__(self, vocab: int, hidden: int, weight: torch.Tensor, cap: float):
        super().__init__(vocab, hidden, weight)
        if not cap > 0:
            raise ValueError("the soft cap of the logits is positive")
        self.cap = float(cap)

    def forward(self, xn: torch.Tensor, ctx: StepContext, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        return ops.softcap(super().forward(xn, ctx, out), self.cap)

    def forward_normed(self, x: torch.Tensor, rows: torch.Tensor, norm, ctx: StepContext, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        return ops.softcap(super().forward_normed(x, rows, norm, ctx, out), self.cap)
