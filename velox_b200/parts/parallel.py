"""Two mixers side by side: both read the same input, each one's output is RMS-normed over the model width
with a weight of its own, and the result is their weighted sum (by default the mean).  Without norm names
(`out_norm_names=None`) the members' outputs are not normed: the result is the plain weighted sum, and a block
that adds a sublayer's output to the stream itself takes the members unmerged with their coefficients
(`forward_terms`).

The members are any registered mixers, given as `PartSpec`s; each keeps the cache it asks for (the mixer's
need is a `CacheParts` of the members' needs, and it hands each member its part).  A block that norms a
sublayer's output anyway can take the members' outputs unmerged (`forward_branches`) and do the members'
norms, the sum, its own norm and the residual update in one kernel.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from ..csrc import ops
from .base import CacheParts, Mixer, Runtime, TensorSpec
from .plan import PartSpec
from .registry import build_part


class ParallelMixer(Mixer):
    @property
    def cuda_graph_safe(self) -> bool:
        return all(bool(m.cuda_graph_safe) for m in self.members)

    @property
    def short_rows_up_to(self) -> int:
        return max(int(getattr(m, "short_rows_up_to", 1)) for m in self.members)

    def __init__(self, prefix: str, hidden_size: int, members: Sequence[PartSpec], out_norm_names: Optional[Sequence[str]],
                 eps: float = 1e-6, coefficients: Optional[Sequence[float]] = None):
        super().__init__(prefix)
        self.normed = out_norm_names is not None
        out_norm_names = out_norm_names if self.normed else ("", "")
        if len(members) != 2 or len(out_norm_names) != 2:
            raise ValueError("%sa parallel mixer has two members (got %d)" % (prefix, len(members)))
        self.hidden_size, self.eps = int(hidden_size), float(eps)
        self.members = [build_part("mixer", m) for m in members]
        self.norm_names = [prefix + n for n in out_norm_names]
        self.coefficients = [float(c) for c in coefficients] if coefficients is not None else [0.5, 0.5]
        self.norm_weights: List[Optional[torch.Tensor]] = [None, None]

    def tensor_specs(self) -> List[TensorSpec]:
        specs = [s for m in self.members for s in m.tensor_specs()]
        return specs + ([TensorSpec(n, (self.hidden_size,), "norm") for n in self.norm_names] if self.normed else [])

    def ignored_tensors(self) -> List[str]:
        return [n for m in self.members for n in m.ignored_tensors()]

    def bind(self, tensors: Dict[str, torch.Tensor], runtime: Runtime) -> None:
        super().bind(tensors, runtime)
        for m in self.members:
            m.bind(tensors, runtime)
        self.norm_weights = [tensors[n] for n in self.norm_names] if self.normed else [None, None]

    def cache_spec(self):
        return CacheParts(tuple(m.cache_spec() for m in self.members))

    def forward_branches(self, h: torch.Tensor, ctx, cache):
        """[(member's output, its norm's weight, its coefficient)] for a block that merges them itself."""
        parts = cache.parts if cache.parts is not None else [cache for _ in self.members]
        return [(m.forward(h, ctx, c), w, k) for m, c, w, k in zip(self.members, parts, self.norm_weights, self.coefficients)]

    def forward_terms(self, h: torch.Tensor, ctx, cache):
        """[(member's output, its coefficient)] of a mixer without member norms, for a block that adds them itself."""
        if self.normed:
            return [(self.forward(h, ctx, cache), 1.0)]
        return [(y, c) for y, _, c in self.forward_branches(h, ctx, cache)]

    def forward(self, h: torch.Tensor, ctx, cache) -> torch.Tensor:
        (y0, w0, c0), (y1, w1, c1) = self.forward_branches(h, ctx, cache)
        if not self.normed:
            # the weighted sum in float32, rounded once (through the kernel that adds terms to a float32 row)
            acc = torch.zeros(y0.shape, dtype=torch.float32, device=y0.device)
            ops.sum_add_rmsnorm(acc, [(y0, c0), (y1, c1)])
            return ops.cast_rows(acc, y0.dtype)
        return ops.merge_norms(y0, w0, c0, y1, w1, c1, self.eps)
