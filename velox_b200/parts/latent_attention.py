"""Attention whose keys and values are raised from one latent vector per position.

    q        = W_q h                          per head: `head_dim` channels that stay, then `rot_dim` rotated ones
    [c; r]   = W_dkv h                        c: `kv_rank` channels, RMS-normed with a plain weight; r: `rot_dim`
                                              channels, rotated, one key part shared by all heads
    k_h      = [W_uk,h c ; r],  v_h = W_uv,h c
    score    = q_h . k_h * scale,  causal softmax,  output W_o on the joined heads

Only [c; r] is kept per position (`PagedLatent`: one row of kv_rank + rot_dim elements in the page).  The keys are
never formed: since q_h . (W_uk,h c) = (W_uk,h^T q_h) . c, a step folds W_uk into its queries (one small product per
head), attends over the cached rows as ONE key/value head of width kv_rank + rot_dim whose value is the row's first
kv_rank elements (`ops.latent_attention`: a tile of rows is staged once for eight heads), and raises the attended latent
vector through W_uv afterwards (again one product per head).
A step that brings a prompt portion of `RAISE_MIN_TOKENS` tokens or more (bfloat16, key and value sizes the tensor-core
kernel takes) goes the other way round: the cached rows of its requests are copied out of their pages into one matrix, ONE
product with [W_uk,h 0; 0 I; W_uv,h 0] per head leaves every head's key [W_uk,h c ; r] and value side by side, and the
tensor-core prompt kernel (`ops.raised_attention`) reads them there with the queries as the projection left them.
Angles, the latent norm, scores and the softmax are float32.  The rotation takes either layout of the position part.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from ..csrc import ops
from .base import Mixer, PagedLatent, Runtime, TensorSpec
from .linear import Linear
from .plan import PartSpec
from .registry import build_part


RAISE_MIN_TOKENS = 16        # longest portion of a step from which keys and values are raised for the tensor-core kernel
RAISE_MAX_BYTES = 2 << 30    # the most that the raised keys and values of a step may take


class LatentAttention(Mixer):
    @property
    def cuda_graph_safe(self) -> bool:
        return bool(self.position.cuda_graph_safe)

    def __init__(self, prefix: str, hidden_size: int, num_heads: int, head_dim: int, rot_dim: int, v_head_dim: int,
                 kv_rank: int, scale: float, position: PartSpec, eps: float = 1e-6,
                 names: Sequence[str] = ("q", "dkv", "dkv.norm", "uk", "uv", "o")):
        super().__init__(prefix)
        self.hidden_size, self.num_heads, self.head_dim = int(hidden_size), int(num_heads), int(head_dim)
        self.rot_dim, self.v_head_dim, self.kv_rank = int(rot_dim), int(v_head_dim), int(kv_rank)
        self.scale, self.eps = float(scale), float(eps)
        if min(self.num_heads, self.head_dim, self.v_head_dim, self.kv_rank) <= 0 or self.rot_dim < 0 or self.rot_dim % 2:
            raise ValueError("%slatent attention: sizes must be positive and rot_dim even" % prefix)
        if self.kv_rank + self.rot_dim > ops.LATENT_ATTENTION_MAX_ROW:
            raise ValueError("%skv_rank + rot_dim = %d: the latent attention kernel takes rows up to %d"
                             % (prefix, self.kv_rank + self.rot_dim, ops.LATENT_ATTENTION_MAX_ROW))
        self.position = build_part("position", position)
        table = self.position.rotary_table("cpu")
        if table is None or table[1] != self.rot_dim:
            raise ValueError("%sthe rotated part has %d channels and the position encoding must turn all of them" % (prefix, self.rot_dim))
        self.names = dict(zip(("q", "dkv", "norm", "uk", "uv", "o"), (prefix + n for n in names)))
        self.proj: Optional[Linear] = None
        self.out: Optional[Linear] = None
        self.norm_weight = self.uk_t = self.uv = self.rotary = self.raise_w = None

    @property
    def row(self) -> int:
        return self.kv_rank + self.rot_dim

    def tensor_specs(self) -> List[TensorSpec]:
        e, H, n = self.hidden_size, self.num_heads, self.names
        return [TensorSpec(n["q"], (H * (self.head_dim + self.rot_dim), e), "matrix"),
                TensorSpec(n["dkv"], (self.row, e), "matrix"), TensorSpec(n["norm"], (self.kv_rank,), "norm"),
                TensorSpec(n["uk"], (H * self.head_dim, self.kv_rank), "matrix"),
                TensorSpec(n["uv"], (H * self.v_head_dim, self.kv_rank), "matrix"),
                TensorSpec(n["o"], (e, H * self.v_head_dim), "matrix")] + self.position.tensor_specs()

    def bind(self, tensors: Dict[str, torch.Tensor], runtime: Runtime) -> None:
        super().bind(tensors, runtime)
        n, H = self.names, self.num_heads
        self.proj = Linear(torch.cat([tensors[n["q"]], tensors[n["dkv"]]], dim=0).contiguous())
        self.norm_weight = tensors[n["norm"]]
        # W_uk per head, transposed: [H, kv_rank, head_dim], the matrix of the product that folds it into a query
        self.uk_t = tensors[n["uk"]].view(H, self.head_dim, self.kv_rank).transpose(1, 2).contiguous()
        self.uv = tensors[n["uv"]].view(H, self.v_head_dim, self.kv_rank).contiguous()
        self.out = Linear(tensors[n["o"]])
        D, R, C, Dv = self.head_dim, self.rot_dim, self.kv_rank, self.v_head_dim
        if ops.raised_attention_supported(tensors[n["uk"]].dtype, D + R, Dv):
            # per head: D rows [W_uk,h | 0], R rows [0 | I] (the shared rotated part), Dv rows [W_uv,h | 0]
            w = torch.zeros((H, D + R + Dv, C + R), dtype=tensors[n["uk"]].dtype, device=tensors[n["uk"]].device)
            w[:, :D, :C] = tensors[n["uk"]].view(H, D, C)
            w[:, D:D + R, C:] = torch.eye(R, dtype=w.dtype, device=w.device)
            w[:, D + R:, :C] = tensors[n["uv"]].view(H, Dv, C)
            self.raise_w = Linear(w.view(H * (D + R + Dv), C + R))
        self.position.bind(tensors, runtime)
        self.rotary = self.position.rotary_table(runtime.device)

    def cache_spec(self):
        return PagedLatent(self.row)

    def forward(self, h: torch.Tensor, ctx, cache) -> torch.Tensor:
        H, D, R, C, Dv = self.num_heads, self.head_dim, self.rot_dim, self.kv_rank, self.v_head_dim
        t = h.shape[0]
        group = ctx.groups[cache.group]
        x = self.proj(h)                       # [tokens, H (D + R) | C + R]
        q, down = x[:, :H * (D + R)], x[:, H * (D + R):]
        interleaved = bool(getattr(self.position, "interleaved", False))
        if (self.raise_w is not None and ctx.max_new >= RAISE_MIN_TOKENS and len(ctx.new_lens) == ctx.n_seqs
                and len(ctx.offsets) == ctx.n_seqs and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0):
            plan = getattr(ctx, "raised_rows", None)   # (made by the step's first latent layer, kept on its context)
            if plan is None:
                plan = ctx.raised_rows = ops.RaisedPlan([a + b for a, b in zip(ctx.offsets, ctx.new_lens)], x.device)
            if plan.rows * H * (D + R + Dv) * 2 <= RAISE_MAX_BYTES:
                ops.latent_prep(down, q, None, self.norm_weight, self.eps, self.rotary[0], interleaved, ctx.positions,
                                group.slot_mapping if cache.writes else None, cache.pages, H, D, R, C)
                kv = self.raise_w(ops.latent_gather(cache.pages, group.block_table, ctx.cu_seqlens, ctx.kv_offsets, plan))
                o = ops.raised_attention(x, x.shape[1], kv, ctx.cu_seqlens, ctx.kv_offsets, plan, self.scale, H, D + R, Dv,
                                         ctx.max_new)
                return self.out(o)
        qa = torch.empty((t, H, C + R), dtype=x.dtype, device=x.device)   # folded queries: [W_uk^T q | rotated part]
        ops.latent_prep(down, q, qa, self.norm_weight, self.eps, self.rotary[0], interleaved,
                        ctx.positions, group.slot_mapping if cache.writes else None, cache.pages, H, D, R, C)
        ops.gemm_heads(q.view(t, H, D + R)[:, :, :D], self.uk_t, qa[:, :, :C])
        latent = ops.latent_attention(qa, cache.pages, group.block_table, ctx.seq_of_token, ctx.positions, self.scale, H, C, R,
                                      max_kv=ctx.max_kv)
        o = torch.empty((t, H, Dv), dtype=x.dtype, device=x.device)
        ops.gemm_heads(latent, self.uv, o)
        return self.out(o.view(t, H * Dv))
