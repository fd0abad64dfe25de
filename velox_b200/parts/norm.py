"""RMSNorm: x * rsqrt(mean(x^2) + eps) * weight, statistics in float32.

The reference calls its tensor library's rms_norm with `rms_norm_eps`
(src/paged/qwen3.rs:923-928, 933, 936); the weight multiplies, with no offset.
With `one_plus` the stored tensor is the multiplier's offset from one: the multiplier is 1 + tensor
(formed once in float32 when the weights are bound).

`LayerNorm`: (x - mean) / sqrt(mean((x - mean)^2) + eps) * weight, no bias; statistics in float32, the variance taken
from the deviations.  With `streams` n > 1 the stream it reads is kept in n copies side by side
([tokens, n * size] float32) and the norm is taken of their sum: the last norm of a model with several streams.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..csrc import ops
from .base import Norm, Runtime, TensorSpec


class RMSNorm(Norm):
    cuda_graph_safe = True  # reads nothing of a step but device tensors and sizes fixed per graph

    def __init__(self, prefix: str, size: int, eps: float, weight_name: str = "weight", one_plus: bool = False):
        super().__init__(prefix)
        self.size, self.eps, self.one_plus = int(size), float(eps), bool(one_plus)
        self.weight_name = prefix + weight_name   # (a checkpoint may name the tensor by the prefix alone: "")
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self.weight_name, (self.size,), "bias" if self.one_plus else "norm")]

    def bind(self, tensors: Dict[str, torch.Tensor], runtime: Runtime) -> None:
        super().bind(tensors, runtime)
        self.weight = tensors[self.weight_name]
        if self.one_plus:
            self.weight = (self.weight.to(torch.float32) + 1.0).contiguous()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.rmsnorm(x, self.weight, self.eps)

    def add_norm(self, residual, delta, rows=None):
        return ops.add_rmsnorm(residual, delta, self.weight, self.eps, self.runtime.dtype, rows=rows)


class LayerNorm(Norm):
    cuda_graph_safe = True

    def __init__(self, prefix: str, size: int, eps: float, weight_name: str = "weight", streams: int = 1):
        super().__init__(prefix)
        self.size, self.eps, self.streams = int(size), float(eps), int(streams)
        if not 0 < self.streams <= ops.STREAMS_MAX:
            raise ValueError("%slayer norm over %d streams: 1 to %d" % (prefix, self.streams, ops.STREAMS_MAX))
        self.weight_name = prefix + weight_name
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self.weight_name, (self.size,), "norm")]

    def bind(self, tensors: Dict[str, torch.Tensor], runtime: Runtime) -> None:
        super().bind(tensors, runtime)
        self.weight = tensors[self.weight_name]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x32 = x if x.dtype == torch.float32 else ops.cast_rows(x, torch.float32)
        return ops.stream_norm(x32, self.streams, None, self.weight, self.eps, x.dtype)

    def add_norm(self, residual, delta, rows=None):
        if delta is not None:
            if self.streams != 1:
                raise ValueError("a layer norm over several streams takes the streams complete, without a pending sublayer output")
            ops.sum_add_rmsnorm(residual, [(delta, 1.0)])
        if residual.shape[1] == self.size and self.streams > 1:   # (a model without layers: the copies are all the input)
            return ops.stream_norm(None, self.streams, None, self.weight, self.eps, self.runtime.dtype, rows=rows, single=residual)
        return ops.stream_norm(residual, self.streams, None, self.weight, self.eps, self.runtime.dtype, rows=rows)
