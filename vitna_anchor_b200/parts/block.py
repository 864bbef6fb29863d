"""Pre-norm residual block: x += mixer(norm1(x)); x += feed_forward(norm2(x))
(engine/src/model.c:906-972).

Output-norm residual block: x += m * norm1(mixer(x)); x += m * norm2(feed_forward(x)): the sublayers read the residual
stream as it is and the norm sits on what they give.

Sandwich-norm residual block: x += post1(mixer(pre1(x))); x += post2(feed_forward(pre2(x))), the four norms layer norms with weight
and bias."""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops

from ..cache.manager import LayerCacheView
from .base import Block, FeedForward, Mixer, Norm, Part, StepContext


class PreNormBlock(Block):
    def __init__(self, mixer_norm: Norm, mixer: Mixer, ffn_norm: Optional[Norm] = None, ffn: Optional[FeedForward] = None):
        """A layer without a feed-forward is the mixer's half alone."""
        if (ffn is None) != (ffn_norm is None):
            raise ValueError("a feed-forward and its norm come together")
        self.mixer_norm, self.mixer, self.ffn_norm, self.ffn = mixer_norm, mixer, ffn_norm, ffn

    def tensors(self):
        return [t for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn) if p is not None for t in p.tensors()]

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: Optional[LayerCacheView], write_cache: bool = True) -> None:
        if self.mixer.fuses_norm(self.mixer_norm, ctx):
            self.mixer.forward(x, ctx, cache, x, write_cache, norm=self.mixer_norm)
        else:
            self.mixer.forward(self.mixer_norm.forward(x, ctx, "block.xn"), ctx, cache, x, write_cache)
        if self.ffn is None:
            return
        if self.ffn.fuses_norm(self.ffn_norm, ctx):
            self.ffn.forward(x, ctx, x, norm=self.ffn_norm)
        else:
            self.ffn.forward(self.ffn_norm.forward(x, ctx, "block.xn"), ctx, x)


class OutputNormBlock(Block):
    """x <- x + mult * norm(sublayer(x)) for the mixer and then (unless absent) the feed-forward; the norms have the RMS form.

    The sublayers keep the framework's contract (they ADD their result into a float32 buffer), only that the buffer is not
    the residual stream but a zeroed row y; one kernel then norms y, scales it, sums it into the float32 residual row, zeroes
    y again and writes the next sublayer's input in the compute dtype.  The first block of a pass writes that input and zeroes
    y itself (a pass is numbered in ctx.extra["pass"] by the decoder), so a step that was given up half-way leaves nothing
    behind.  In float32 the sublayers read the residual stream itself."""

    def __init__(self, mixer_norm: Norm, mixer: Mixer, ffn_norm: Optional[Norm] = None, ffn: Optional[FeedForward] = None, mult: float = 1.0):
        if (ffn is None) != (ffn_norm is None):
            raise ValueError("a feed-forward and its norm come together")
        if mixer_norm.as_rms() is None or (ffn_norm is not None and ffn_norm.as_rms() is None):
            raise ValueError("the norms on the sublayers' outputs have the RMS form")
        self.mixer_norm, self.mixer, self.ffn_norm, self.ffn, self.mult = mixer_norm, mixer, ffn_norm, ffn, float(mult)

    def tensors(self):
        return [t for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn) if p is not None for t in p.tensors()]

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: Optional[LayerCacheView], write_cache: bool = True) -> None:
        T, W, ws = ctx.num_tokens, x.shape[1], ctx.workspace
        y = ws.flat(f"outnorm.y/{W}", ws.max_tokens * W, torch.float32, zero=True)[:T * W].view(T, W)
        xc = x if ctx.dtype == torch.float32 else ws.rows("outnorm.xc", T, W, ctx.dtype)
        copy = None if xc is x else xc
        this_pass = ctx.extra.get("pass", 0)
        if ctx.extra.get("outnorm.begun") != this_pass:
            ops.residual_norm_step(x, y, None, copy)
            ctx.extra["outnorm.begun"] = this_pass
        self.mixer.forward(xc, ctx, cache, y, write_cache)
        w, eps = self.mixer_norm.as_rms()
        ops.residual_norm_step(x, y, w, copy, eps, self.mult)
        if self.ffn is None:
            return
        self.ffn.forward(xc, ctx, y)
        w, eps = self.ffn_norm.as_rms()
        ops.residual_norm_step(x, y, w, copy, eps, self.mult)


class SandwichNormBlock(Block):
    """x <- x + post(sublayer(pre(x))) for the mixer and then (unless absent) the feed-forward; the four norms are layer norms with
    weight and bias (anything with .weight, .bias and .eps of the LayerNorm part).

    The sublayers do what they do everywhere in the framework (they ADD their result into a float32 buffer): the buffer is a zeroed row
    y, and ONE kernel between two sublayers norms y, sums it into the float32 residual row, zeroes y again and norms the new row for the
    next sublayer.  A block leaves its last sum pending for the next block's first kernel (two launches a layer instead of three); behind
    the last block SandwichFlush, the decoder's `collect` part, does what is left.  While something looks at the residual rows
    between the runs of the schedule (ctx.after_run), every block finishes its own sum."""

    PENDING = "sandwich.pending"

    def __init__(self, mixer_norm: Norm, mixer_post: Norm, mixer: Mixer, ffn_norm: Optional[Norm] = None, ffn_post: Optional[Norm] = None,
                 ffn: Optional[FeedForward] = None):
        if not ((ffn is None) == (ffn_norm is None) == (ffn_post is None)):
            raise ValueError("a feed-forward and its two norms come together")
        for n in (mixer_norm, mixer_post, ffn_norm, ffn_post):
            if n is not None and not (hasattr(n, "weight") and hasattr(n, "bias") and hasattr(n, "eps")):
                raise ValueError("the norms of this block are layer norms with weight and bias")
        self.mixer_norm, self.mixer_post, self.mixer, self.ffn_norm, self.ffn_post, self.ffn = mixer_norm, mixer_post, mixer, ffn_norm, ffn_post, ffn

    def tensors(self):
        return [t for p in (self.mixer_norm, self.mixer_post, self.mixer, self.ffn_norm, self.ffn_post, self.ffn) if p is not None for t in p.tensors()]

    @staticmethod
    def buffer(x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        T, W, ws = ctx.num_tokens, x.shape[1], ctx.workspace
        return ws.flat(f"sandwich.y/{W}", ws.max_tokens * W, torch.float32, zero=True)[:T * W].view(T, W)

    @classmethod
    def take_pending(cls, ctx: StepContext):
        """The (weight, bias) of a sum that the block before left to do, if it did so in this pass."""
        left = ctx.extra.pop(cls.PENDING, None)
        return left[1] if left is not None and left[0] == ctx.extra.get("pass", 0) else None

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: Optional[LayerCacheView], write_cache: bool = True) -> None:
        T, W, ws = ctx.num_tokens, x.shape[1], ctx.workspace
        y = self.buffer(x, ctx)
        xn = ws.rows("block.xn", T, W, ctx.dtype)
        pair = lambda n: (n.weight, n.bias)
        eps = self.mixer_norm.eps
        ops.sandwich_step(x, y, self.take_pending(ctx), pair(self.mixer_norm), xn, eps)
        self.mixer.forward(xn, ctx, cache, y, write_cache)
        last = self.mixer_post
        if self.ffn is not None:
            ops.sandwich_step(x, y, pair(self.mixer_post), pair(self.ffn_norm), xn, eps)
            self.ffn.forward(xn, ctx, y)
            last = self.ffn_post
        if ctx.after_run is not None:
            ops.sandwich_step(x, y, pair(last), None, None, eps)
        else:
            ctx.extra[self.PENDING] = (ctx.extra.get("pass", 0), pair(last))


class SandwichFlush(Part):
    """Behind the last SandwichNormBlock: the sum that it left pending.  Used as a decoder's `collect` part."""

    def __init__(self, eps: float):
        self.eps = float(eps)

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        post = SandwichNormBlock.take_pending(ctx)
        if post is not None:
            ops.sandwich_step(x, SandwichNormBlock.buffer(x, ctx), post, None, None, self.eps)
        return x
