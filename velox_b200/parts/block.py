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

`HyperConnectionBlock`: the stream is kept in n copies x_1 .. x_n (all equal to the embedding's output at first).  A
sublayer reads a weighted sum of them and writes to all of them while they are mixed among themselves:
    u = sum_s in[s] x_s;   y = ls (.) sublayer(norm(u));   x_t <- sum_s mix[s, t] x_s + m out[t] y   (all t from the old x_s)
with `in`, `out` [n], `mix` [n, n] (indexed [from, to]) and the channel-wise layer scale `ls` [hidden] being tensors of the
sublayer, and m a constant of the model.  With `streams` = 0 there is one copy and no mixing tensors: the plain pre-norm
layer with a layer scale, x <- x + m ls (.) sublayer(norm(x)).  The update of one sublayer and the weighted sum and norm
of the next are one kernel (`ops.stream_update`); the last update of a block travels as a `PendingStreams` to the next
block of this kind, whose first norm it is fused with, or is applied by whoever reads the stream next.  The residual
between such blocks is [tokens, n * hidden] float32; a `LayerNorm(streams=n)` reads the sum of the copies at the end.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Tuple

import torch

from ..csrc import ops
from .base import Block, Part, TensorSpec


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


class PendingStreams(PendingSum):
    """A sublayer's output that is still to be written into the copies of the stream: x_t <- sum_s mix[s][t] x_s +
    mult * out[t] * layer_scale (.) y.  `add_to` applies it (and, given the next reader's coefficients and norm weight,
    returns that reader's normed input from the same kernel)."""

    def __init__(self, y, streams: int, mix, out, mult: float, layer_scale):
        super().__init__([(y, 1.0)])
        self.y, self.streams, self.mix, self.out, self.mult, self.layer_scale = y, int(streams), mix, out, float(mult), layer_scale

    def add_to(self, residual, weight=None, eps: float = 0.0, out_dtype=None, in_next=None, rms: bool = False):
        if self.rows is not None or self.vector is not None or len(self.terms) != 1:
            raise ValueError("a stream kept in several copies takes no inputs between its layers")
        return ops.stream_update(residual, self.streams, self.mix, self.out, self.mult, self.layer_scale, self.y,
                                 in_next, weight, eps, rms)


class StreamCoefficients(Part):
    """The tensors of one sublayer's connection to the copies of the stream: `in`, `out` [n], `mix` [n, n] (kept as host
    numbers: they are parameters of the stream kernels) and the layer scale [hidden] (float32 on the device)."""
    cuda_graph_safe = True

    def __init__(self, prefix: str, streams: int, hidden_size: int, names=("in", "out", "mix"), scale_name: str = ""):
        super().__init__(prefix)
        self.streams, self.hidden_size = int(streams), int(hidden_size)
        self.names = tuple(prefix + n for n in names)
        self.scale_name = scale_name
        self.into = self.out = self.mix = self.layer_scale = None

    def tensor_specs(self):
        n, specs = self.streams, []
        if n:
            specs += [TensorSpec(self.names[0], (n,), "norm"), TensorSpec(self.names[1], (n,), "norm"),
                      TensorSpec(self.names[2], (n, n), "mixing")]
        if self.scale_name:
            specs.append(TensorSpec(self.scale_name, (self.hidden_size,), "norm"))
        return specs

    def bind(self, tensors, runtime):
        super().bind(tensors, runtime)
        if self.streams:
            self.into = tensors[self.names[0]].to(torch.float32).cpu().tolist()
            self.out = tensors[self.names[1]].to(torch.float32).cpu().tolist()
            self.mix = tensors[self.names[2]].to(torch.float32).cpu().tolist()
        if self.scale_name:
            self.layer_scale = tensors[self.scale_name].to(torch.float32).contiguous()


class HyperConnectionBlock(Block):
    needs_feed_forward = False
    takes_pending = True

    def __init__(self, mixer, feed_forward, norms, hidden_size: int, streams: int = 0, residual_mult: float = 1.0,
                 prefix: str = "", connection_names=("hc1.", "hc2."), scale_names=("ls1", "ls2"), coefficient_names=("in", "out", "mix")):
        self.norm_names = ("mixer",) + (("feed_forward",) if feed_forward is not None else ())
        super().__init__(mixer, feed_forward, norms)
        self.hidden_size, self.streams, self.residual_mult = int(hidden_size), int(streams), float(residual_mult)
        if not 0 <= self.streams <= ops.STREAMS_MAX:
            raise ValueError("%sa stream in %d copies: the stream kernels take up to %d" % (prefix, self.streams, ops.STREAMS_MAX))
        if not 0 < self.hidden_size <= ops.STREAM_MAX_WIDTH:
            raise ValueError("%sa stream of width %d: the stream kernels take up to %d" % (prefix, self.hidden_size, ops.STREAM_MAX_WIDTH))
        for name, n in self.norms.items():
            if not hasattr(n, "weight") or not hasattr(n, "eps") or getattr(n, "streams", 1) != 1:
                raise ValueError("HyperConnectionBlock fuses its norms into the stream's update and takes layer or RMS norms of one "
                                 "row; %r is %s" % (name, type(n).__name__))
        self.links = [StreamCoefficients(prefix + connection_names[q], self.streams, self.hidden_size, coefficient_names,
                                         prefix + scale_names[q] if scale_names and scale_names[q] else "")
                      for q in range(2 if feed_forward is not None else 1)]

    @property
    def copies(self) -> int:
        return max(self.streams, 1)

    def parts(self):
        return super().parts() + list(self.links)

    @staticmethod
    def _rms(norm) -> bool:
        return not hasattr(norm, "streams")   # (an RMS norm of this package; the layer norm says how many copies it reads)

    def forward(self, residual, delta, ctx, cache):
        n, E = self.copies, self.hidden_size
        norm, link = self.norms["mixer"], self.links[0]
        dtype = self.mixer.runtime.dtype
        plain = residual.shape[1] == E and (n > 1 or not isinstance(delta, PendingStreams))
        if plain:
            # the embedding's output (or a plain stream left by another kind of block): the copies start equal to it
            if isinstance(delta, PendingSum):
                delta.add_to(residual)
            elif delta is not None:
                ops.sum_add_rmsnorm(residual, [(delta, 1.0)])
            copies = torch.empty((residual.shape[0], n * E), dtype=torch.float32, device=residual.device) if n > 1 else None
            h = ops.stream_norm(None, n, link.into, norm.weight, norm.eps, dtype, single=residual, copies=copies, rms=self._rms(norm))
            if copies is not None:
                residual = copies
        elif isinstance(delta, PendingStreams):
            h = delta.add_to(residual, norm.weight, norm.eps, dtype, in_next=link.into, rms=self._rms(norm))
        else:
            if delta is not None:
                raise ValueError("a stream kept in several copies cannot take a sublayer output that names no copies")
            h = ops.stream_norm(residual, n, link.into, norm.weight, norm.eps, dtype, rms=self._rms(norm))
        y = self.mixer.forward(h, ctx, cache)
        pending = PendingStreams(y, n, link.mix, link.out, self.residual_mult, link.layer_scale)
        if self.feed_forward is not None:
            norm, link = self.norms["feed_forward"], self.links[1]
            h = pending.add_to(residual, norm.weight, norm.eps, dtype, in_next=link.into, rms=self._rms(norm))
            y = self.feed_forward.forward(h, ctx)
            pending = PendingStreams(y, n, link.mix, link.out, self.residual_mult, link.layer_scale)
        return residual, pending
