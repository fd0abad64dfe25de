"""Token embedding and output head.

x[t] = embed_tokens.weight[id[t]] (src/paged/qwen3.rs:958, 998); logits =
rows W^T with W the head's own matrix, or the embedding table when the two are
tied (src/paged/qwen3.rs:966-976).  The embedding feeds the float32 residual
stream; logits are always float32 (the reference leaves them in the model's
element type, src/paged/qwen3.rs:1015).  Two multipliers for designs that have them:
`TokenEmbedding(scale=)` on the rows that enter the stream, `OutputHead(logit_scale=)`
on the float32 logits; and a bound, `OutputHead(logit_softcap=c)`: logits become c tanh(logits / c).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..csrc import ops
from .base import Embedding, FixedState, Part, Runtime, TensorSpec
from .linear import matmul


class TokenEmbedding(Embedding):
    cuda_graph_safe = True  # reads nothing of a step but device tensors and sizes fixed per graph

    def __init__(self, prefix: str, vocab_size: int, hidden_size: int, scale: float = 1.0, weight_name: str = "weight",
                 leaves_rounded: bool = False):
        super().__init__(prefix)
        self.vocab_size, self.hidden_size, self.scale = int(vocab_size), int(hidden_size), float(scale)
        self.weight_name = prefix + weight_name
        # for a first block whose sublayers read the stream itself: the rows also go to `ctx.rounded`
        # in the engine's element type, from the same kernel
        self.leaves_rounded = bool(leaves_rounded)
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self.weight_name, (self.vocab_size, self.hidden_size), "table")]

    def bind(self, tensors: Dict[str, torch.Tensor], runtime: Runtime) -> None:
        super().bind(tensors, runtime)
        self.weight = tensors[self.weight_name]

    def forward(self, ctx) -> torch.Tensor:
        if not self.leaves_rounded:
            return ops.embedding(ctx.token_ids, self.weight, scale=self.scale)
        rounded = torch.empty((ctx.token_ids.numel(), self.hidden_size), dtype=self.weight.dtype, device=self.weight.device)
        x = ops.embedding(ctx.token_ids, self.weight, scale=self.scale, rounded=rounded)
        ctx.rounded = (x, rounded)
        return x


class PairHashEmbedding(Embedding):
    """x[t] = table[id[t]] + pair_table[(id[t-1] * mul_prev + id[t] * mul_cur) mod buckets]: the token's row
    plus a row picked by the pair (previous token, token).  A request's first token has no previous one and
    takes the pair table's last row (number `buckets`).  The token before a step's first is part of the
    request's state: one int32 per state slot, read and advanced on the device."""
    cuda_graph_safe = True

    def __init__(self, prefix: str, vocab_size: int, hidden_size: int, buckets: int, mul_prev: int, mul_cur: int,
                 table_name: str = "embed", pair_table_name: str = "bigram"):
        super().__init__(prefix)
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.buckets, self.mul_prev, self.mul_cur = int(buckets), int(mul_prev), int(mul_cur)
        if self.buckets <= 0 or self.mul_prev < 0 or self.mul_cur < 0:
            raise ValueError("pair embedding: buckets must be positive and the multipliers not negative")
        self.table_name, self.pair_table_name = prefix + table_name, prefix + pair_table_name
        self.weight: Optional[torch.Tensor] = None
        self.pair_weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self.table_name, (self.vocab_size, self.hidden_size), "table"),
                TensorSpec(self.pair_table_name, (self.buckets + 1, self.hidden_size), "table")]

    def bind(self, tensors: Dict[str, torch.Tensor], runtime: Runtime) -> None:
        super().bind(tensors, runtime)
        self.weight, self.pair_weight = tensors[self.table_name], tensors[self.pair_table_name]

    def cache_spec(self):
        return FixedState((1,), "int32")

    def forward(self, ctx, cache=None) -> torch.Tensor:
        return ops.embedding_pair(ctx.token_ids, ctx.positions, ctx.seq_of_token, ctx.cu_seqlens, ctx.state_slots,
                                  cache.state.view(-1), self.weight, self.pair_weight, self.buckets, self.mul_prev,
                                  self.mul_cur)


class OutputHead(Part):
    cuda_graph_safe = True  # reads nothing of a step but device tensors and sizes fixed per graph

    def __init__(self, prefix: str, vocab_size: int, hidden_size: int, tied: bool = False, weight_name: str = "weight",
                 logit_scale: float = 1.0, logit_softcap: float = 0.0):
        super().__init__(prefix)
        self.logit_softcap = float(logit_softcap)
        self.vocab_size, self.hidden_size, self.tied = int(vocab_size), int(hidden_size), bool(tied)
        self.logit_scale = float(logit_scale)
        self.weight_name = prefix + weight_name
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> List[TensorSpec]:
        if self.tied:
            return []
        return [TensorSpec(self.weight_name, (self.vocab_size, self.hidden_size), "matrix")]

    def ignored_tensors(self) -> List[str]:
        # a tied checkpoint may still carry a copy of the head
        return [self.weight_name] if self.tied else []

    def bind(self, tensors: Dict[str, torch.Tensor], runtime: Runtime) -> None:
        super().bind(tensors, runtime)
        if not self.tied:
            self.weight = tensors[self.weight_name]

    def tie(self, table: torch.Tensor) -> None:
        self.weight = table

    def forward(self, rows: torch.Tensor) -> torch.Tensor:
        logits = matmul(rows, self.weight, None, torch.float32)
        if self.logit_scale != 1.0:
            logits = ops.scale_rows(logits, self.logit_scale)
        return ops.softcap_rows(logits, self.logit_softcap) if self.logit_softcap > 0 else logits
