"""Arrangements of a layer's parts.

`PreNormBlock`, the reference's decoder layer (src/paged/qwen3.rs:932-939):
    h = norm1(x); x = x + mixer(h); h = norm2(x); x = x + feed_forward(h)

The residual stream x is float32.  A sublayer's output is not added at once:
it travels as `delta` to the next norm, whose kernel forms x + delta in float32,
stores it and norms it in one pass.  A block therefore takes (residual, delta)
and returns (residual, delta); the model adds the last delta in its final norm.

`SandwichNormBlock`: a norm before AND after each sublayer, and a multiplier m on both branches:
    x = x + m * norm1b(mixer(norm1(x)));  x = x + m * norm2b(feed_forward(norm2(x)))
(the second line falls away in a layer without a feed-forward).  The norm after a sublayer, the scaled
residual update and the norm before the next sublayer are one kernel; a mixer made of two members
(`forward_branches`) has its members' norms and their sum done there too.  The residual is complete when the
block returns, so it hands on no delta.

`PostNormBlock`: a norm on each sublayer's OUTPUT only; the sublayers read the stream itself:
    x = x + norm1(mixer(x));  x = x + norm2(feed_forward(x))
(the second line falls away in a layer without a feed-forward).  The sublayers' input is the float32 stream
rounded to the engine's element type; the kernel that norms a sublayer's output and updates the residual
also writes that rounding for the next sublayer, and the last one of a block leaves it in `ctx.rounded` for
the next block.

`ParallelSublayersBlock`: ONE norm, whose output both sublayers read:
    h = norm(x);  x = x + mixer(h) + feed_forward(h)
(the last term falls away in a layer without a feed-forward).  The sublayers' outputs are not added at once: they
travel as a `PendingSum` to whoever norms the stream next (the next block of this kind, or the model before another
block or the final norm), whose one kernel adds them to the float32 residual, with their coefficients, and norms the
sum.  A mixer made of members side by side hands its members over unmerged with their coefficients
(`forward_terms`), so their weighted sum is formed in float32 in that same kernel.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Tuple

import torch

from ..csrc import ops
from .base import Block


@dataclass
class PendingSum:
    """What is still to be added to the float32 residual: up to three (tensor, coefficient) terms in the engine's
    element type, float32 rows of the residual's shape, and a float32 vector added to every row."""
    terms: List[Tuple[torch.Tensor, float]] = field(default_factory=list)
    rows: Optional[torch.Tensor] = None
    vector: Optional[torch.Tensor] = None

    def add_to(self, residual: torch.Tensor, weight=None, eps: float = 0.0, out_dtype=None):
        """Adds everything to `residual` in place; with a weight returns the RMS norm of the sum."""
        terms = list(self.terms)
        while len(terms) > 3:   # (more terms than the kernel takes: the first ones go ahead)
            ops.sum_add_rmsnorm(residual, terms[:3])
            terms = terms[3:]
        return ops.sum_add_rmsnorm(residual, terms, self.rows, self.vector, weight, eps, out_dtype)


class PreNormBlock(Block):
    norm_names = ("mixer", "feed_forward")

    def forward(self, residual, delta, ctx, cache):
        h = self.norms["mixer"].add_norm(residual, delta)
        a = self.mixer.forward(h, ctx, cache)
        h = self.norms["feed_forward"].add_norm(residual, a)
        f = self.feed_forward.forward(h, ctx)
        return residual, f


class PostNormBlock(Block):
    needs_feed_forward = False
    leaves_rounded = True

    def __init__(self, mixer, feed_forward, norms):
        self.norm_names = ("mixer_out",) + (("feed_forward_out",) if feed_forward is not None else ())
        super().__init__(mixer, feed_forward, norms)
        for name, n in self.norms.items():
            if not hasattr(n, "weight") or not hasattr(n, "eps"):
                raise ValueError("PostNormBlock fuses its norms into the residual update and takes RMS norms; %r is %s"
                                 % (name, type(n).__name__))

    def forward(self, residual, delta, ctx, cache):
        n = self.norms
        dtype = self.mixer.runtime.dtype
        if delta is not None:   # (a block before this one left a sublayer's output to be added)
            residual.add_(delta)
            ctx.rounded = None
        carried = ctx.rounded
        if carried is not None and carried[0] is residual and carried[1].dtype == dtype:
            h = carried[1]
        else:
            h = ops.cast_rows(residual, dtype)
        y = self.mixer.forward(h, ctx, cache)
        h = ops.merge_norm_add_norm(residual, y, n["mixer_out"].weight, 1.0, n["mixer_out"].eps, rounded=True)
        if self.feed_forward is not None:
            f = self.feed_forward.forward(h, ctx)
            h = ops.merge_norm_add_norm(residual, f, n["feed_forward_out"].weight, 1.0, n["feed_forward_out"].eps, rounded=True)
        ctx.rounded = (residual, h)
        return residual, None


class SandwichNormBlock(Block):
    needs_feed_forward = False

    def __init__(self, mixer, feed_forward, norms, residual_mult: float = 1.0):
        self.norm_names = ("mixer", "mixer_out") + (("feed_forward", "feed_forward_out") if feed_forward is not None else ())
        super().__init__(mixer, feed_forward, norms)
        self.residual_mult = float(residual_mult)
        for name, n in self.norms.items():
            if not hasattr(n, "weight") or not hasattr(n, "eps"):
                raise ValueError("SandwichNormBlock fuses its norms into one kernel and takes RMS norms; %r is %s"
                                 % (name, type(n).__name__))

    def forward(self, residual, delta, ctx, cache):
        n, m = self.norms, self.residual_mult
        h = n["mixer"].add_norm(residual, delta)
        after, eps = n["mixer_out"], n["mixer_out"].eps
        w_next = n["feed_forward"].weight if self.feed_forward is not None else None
        if hasattr(self.mixer, "forward_branches") and getattr(self.mixer, "eps", eps) == eps:
            (y0, w0, c0), (y1, w1, c1) = self.mixer.forward_branches(h, ctx, cache)
            h = ops.merge_norm_add_norm(residual, y0, after.weight, m, eps, w0, c0, y1, w1, c1, w_next=w_next)
        else:
            h = ops.merge_norm_add_norm(residual, self.mixer.forward(h, ctx, cache), after.weight, m, eps, w_next=w_next)
        if self.feed_forward is not None:
            f = self.feed_forward.forward(h, ctx)
            ops.merge_norm_add_norm(residual, f, n["feed_forward_out"].weight, m, n["feed_forward_out"].eps)
        return residual, None


class ParallelSublayersBlock(Block):
    norm_names = ("shared",)
    needs_feed_forward = False
    takes_pending = True

    def __init__(self, mixer, feed_forward, norms):
        super().__init__(mixer, feed_forward, norms)
        n = self.norms["shared"]
        if not hasattr(n, "weight") or not hasattr(n, "eps"):
            raise ValueError("ParallelSublayersBlock fuses its norm into the residual update and takes an RMS norm; got %s"
                             % type(n).__name__)

    def forward(self, residual, delta, ctx, cache):
        n = self.norms["shared"]
        dtype = self.mixer.runtime.dtype
        if isinstance(delta, PendingSum):
            h = delta.add_to(residual, n.weight, n.eps, dtype)
        else:
            h = n.add_norm(residual, delta)
        if hasattr(self.mixer, "forward_terms"):
            terms = list(self.mixer.forward_terms(h, ctx, cache))
        else:
            terms = [(self.mixer.forward(h, ctx, cache), 1.0)]
        if self.feed_forward is not None:
            terms.append((self.feed_forward.forward(h, ctx), 1.0))
        return residual, PendingSum(terms)
