"""A decoder put together from a `ModelPlan`: embedding, blocks in the plan's
running order, final norm, output head.  Which architecture the plan came from
is not known here.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..parts.base import Part, Runtime, TensorSpec
from ..parts.block import PendingSum
from ..parts.plan import ModelPlan
from ..parts.registry import build_part, part_class


class StreamInputs(Part):
    """What a plan adds to the stream between layers (`ModelPlan.stream_inputs`): holds the tensors of vectors
    (float32) and says, per place, what is to be added."""
    cuda_graph_safe = True

    def __init__(self, inputs, hidden_size: int):
        super().__init__("")
        self.hidden_size = int(hidden_size)
        self.by_place = {x.place: x for x in inputs}
        self.shapes = {}
        for x in inputs:
            if x.tensor is not None:
                if self.shapes.setdefault(x.tensor, x.rows) != x.rows:
                    raise ValueError("stream inputs disagree about the rows of %r" % x.tensor)
        self.vectors = {}

    @property
    def needs_embedding(self) -> bool:
        return any(x.embedding for x in self.by_place.values())

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(name, (rows, self.hidden_size), "bias") for name, rows in self.shapes.items()]

    def bind(self, tensors: Dict[str, torch.Tensor], runtime: Runtime) -> None:
        super().bind(tensors, runtime)
        self.vectors = {name: tensors[name].to(torch.float32).contiguous() for name in self.shapes}

    def at(self, place: int, embedded):
        """(float32 rows or None, float32 vector or None) that the stream takes before `place`."""
        x = self.by_place.get(place)
        if x is None:
            return None, None
        return (embedded if x.embedding else None), (self.vectors[x.tensor][x.row] if x.tensor is not None else None)


class DecoderModel:
    def __init__(self, plan: ModelPlan):
        plan.validate()
        self.plan = plan
        self.embedding = build_part("embedding", plan.embedding)
        self.blocks = []
        for spec in plan.layers:
            block_cls = part_class("block", spec.block)
            self.blocks.append(block_cls(
                build_part("mixer", spec.mixer) if spec.mixer is not None else None,
                build_part("feed_forward", spec.feed_forward) if spec.feed_forward is not None else None,
                {name: build_part("norm", n) for name, n in spec.norms.items()}, **spec.block_params))
        self.final_norm = build_part("norm", plan.final_norm)
        self.head = build_part("head", plan.head)
        self.order = plan.running_order()
        self.stream_inputs = StreamInputs(plan.stream_inputs, plan.hidden_size) if plan.stream_inputs else None
        # called as probe(place, stream [tokens, hidden] float32) after every place of the running order (tests, tools)
        self.probe = None
        self.runtime: Optional[Runtime] = None

    # -- weights -------------------------------------------------------------
    def parts(self) -> List[Part]:
        out: List[Part] = [self.embedding]
        for b in self.blocks:
            out.extend(b.parts())
        out.extend([self.final_norm, self.head])
        if self.stream_inputs is not None:
            out.append(self.stream_inputs)
        return out

    def tensor_specs(self) -> List[TensorSpec]:
        return [s for p in self.parts() for s in p.tensor_specs()]

    def ignored_tensors(self) -> List[str]:
        return [n for p in self.parts() for n in p.ignored_tensors()] + list(self.plan.ignored_tensors)

    def bind(self, tensors: Dict[str, torch.Tensor], runtime: Runtime) -> None:
        self.runtime = runtime
        for p in self.parts():
            p.bind(tensors, runtime)
        if getattr(self.head, "tied", False):
            self.head.tie(self.embedding.weight)

    # -- cache ---------------------------------------------------------------
    # Caches belong to the places of the running order, not to layers: a layer
    # that the order names twice shares its weights between the two places, but
    # each place keeps keys, values or state of its own, so that a position's
    # result does not depend on how the tokens were cut into steps.
    # An embedding that keeps something per request has one more place, after the last
    # of the running order.
    def cache_specs(self) -> list:
        """Per place of the running order: the mixer's cache need, or None for a
        place without a cache of its own (none at all, or another's); then the
        embedding's need, if it has one."""
        specs = [None if self.plan.layers[i].cache_of is not None or self.blocks[i].mixer is None
                 else self.blocks[i].mixer.cache_spec() for i in self.order]
        return specs + ([self.embedding.cache_spec()] if self._embedding_keeps_state() else [])

    def _embedding_keeps_state(self) -> bool:
        return getattr(self.embedding, "cache_spec", None) is not None and self.embedding.cache_spec() is not None

    def cache_sources(self) -> list:
        """Per place of the running order: None, or the earlier place whose cache
        it reads (the latest earlier run of layer `cache_of`)."""
        out = []
        for k, i in enumerate(self.order):
            j = self.plan.layers[i].cache_of
            if j is None:
                out.append(None)
                continue
            earlier = [m for m in range(k) if self.order[m] == j]
            if not earlier:
                raise ValueError("layer %d reads the cache of layer %d, which has not run before it" % (i, j))
            out.append(earlier[-1])
        return out + ([None] if self._embedding_keeps_state() else [])

    # -- step ----------------------------------------------------------------
    def forward_hidden(self, ctx, cache):
        """Runs the step's tokens through every layer; returns (residual, delta),
        whose sum is the last layer's output [tokens, hidden]."""
        ctx.rounded = None
        if self._embedding_keeps_state():
            residual = self.embedding.forward(ctx, cache.layer(len(self.order)))
        else:
            residual = self.embedding.forward(ctx)
        delta = None
        inputs = self.stream_inputs
        embedded = residual.clone() if inputs is not None and inputs.needs_embedding else None
        for place, i in enumerate(self.order):
            block = self.blocks[i]
            if inputs is not None:
                rows, vector = inputs.at(place, embedded)
                if rows is not None or vector is not None:
                    # added with whatever the last block left to be added, by the kernel that norms the stream next
                    if not isinstance(delta, PendingSum):
                        delta = PendingSum([(delta, 1.0)] if delta is not None else [])
                    delta.rows, delta.vector = rows, vector
                    ctx.rounded = None
            if isinstance(delta, PendingSum) and not getattr(block, "takes_pending", False):
                delta.add_to(residual)
                delta = None
            residual, delta = block.forward(residual, delta, ctx, cache.layer(place))
            if not getattr(block, "leaves_rounded", False):
                ctx.rounded = None   # (a rounded copy of the stream is good for the block right after its maker)
            if self.probe is not None:
                done = residual.clone()
                if isinstance(delta, PendingSum):
                    delta.add_to(done)
                elif delta is not None:
                    done += delta
                self.probe(place, done)
        return residual, delta

    def logits(self, residual, delta, rows: torch.Tensor) -> torch.Tensor:
        """float32 logits [len(rows), vocab] at the given token rows (int32)."""
        if isinstance(delta, PendingSum):
            delta.add_to(residual)
            delta = None
        h = self.final_norm.add_norm(residual, delta, rows=rows)
        return self.head.forward(h)
