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

Four more, for designs that have them:
`q_rank` r > 0: the queries go through a latent vector of their own, q = W_uq rmsnorm(W_dq h) (a plain weight, the
layer's eps); W_dq rides in the fused projection and W_uq is a second product;
`window` w > 0: position i sees only j with 0 <= i - j < w.  The folded kernel starts at the window's first tile; the
raised way gathers and raises only the rows from the window of the step's first query on (`cache_window`, at least
`window`, is how long the cache keeps a row: the longest window of this layer and of the layers that borrow its rows);
`output_gate`: the joined heads are multiplied element by element by sigmoid(W_g h) before the output projection; W_g rides
in the fused projection;
`own_rows=False`: the layer has no W_dkv and no norm weight of its own and reads the rows that another layer wrote (the
plan's `cache_of`), with its own W_uk, W_uv, queries and window.
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
                 names: Sequence[str] = ("q", "dkv", "dkv.norm", "uk", "uv", "o"), q_rank: int = 0, window: int = 0,
                 cache_window: Optional[int] = None, output_gate: bool = False, own_rows: bool = True,
                 query_names: Sequence[str] = ("dq", "dq.norm", "uq"), gate_name: str = "g"):
        super().__init__(prefix)
        self.q_rank, self.window, self.output_gate, self.own_rows = int(q_rank), int(window), bool(output_gate), bool(own_rows)
        self.cache_window = self.window if cache_window is None else int(cache_window)
        if self.q_rank < 0 or self.window < 0 or (self.cache_window and self.cache_window < self.window) \
                or (self.window == 0 and self.cache_window):
            raise ValueError("%slatent attention: q_rank and window must not be negative, and the cache must keep a row at "
                             "least as long as the window" % prefix)
        self.query_names = tuple(prefix + n for n in query_names)
        self.gate_name = prefix + gate_name
        self.q_norm_weight = self.uq = None
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
        if getattr(self.position, "magnitude", 1.0) != 1.0:
            raise ValueError("%slatent attention rotates without a multiplier of cosines and sines; the position asks for %g"
                             % (prefix, self.position.magnitude))
        self.names = dict(zip(("q", "dkv", "norm", "uk", "uv", "o"), (prefix + n for n in names)))
        self.proj: Optional[Linear] = None
        self.out: Optional[Linear] = None
        self.norm_weight = self.uk_t = self.uv = self.rotary = self.raise_w = None

    @property
    def row(self) -> int:
        return self.kv_rank + self.rot_dim

    def tensor_specs(self) -> List[TensorSpec]:
        e, H, n = self.hidden_size, self.num_heads, self.names
        q_rows = H * (self.head_dim + self.rot_dim)
        if self.q_rank:
            dq, dq_norm, uq = self.query_names
            specs = [TensorSpec(dq, (self.q_rank, e), "matrix"), TensorSpec(dq_norm, (self.q_rank,), "norm"),
                     TensorSpec(uq, (q_rows, self.q_rank), "matrix")]
        else:
            specs = [TensorSpec(n["q"], (q_rows, e), "matrix")]
        if self.own_rows:
            specs += [TensorSpec(n["dkv"], (self.row, e), "matrix"), TensorSpec(n["norm"], (self.kv_rank,), "norm")]
        if self.output_gate:
            specs.append(TensorSpec(self.gate_name, (H * self.v_head_dim, e), "matrix"))
        return specs + [TensorSpec(n["uk"], (H * self.head_dim, self.kv_rank), "matrix"),
                        TensorSpec(n["uv"], (H * self.v_head_dim, self.kv_rank), "matrix"),
                        TensorSpec(n["o"], (e, H * self.v_head_dim), "matrix")] + self.position.tensor_specs()

    def bind(self, tensors: Dict[str, torch.Tensor], runtime: Runtime) -> None:
        super().bind(tensors, runtime)
        n, H = self.names, self.num_heads
        # one projection of the layer's input: [W_q or W_dq; W_dkv; W_g], every block on a multiple of 8 rows so that the
        # slices of its output start on 16-byte addresses
        mats, self.cols, at = [], {}, 0
        first = tensors[self.query_names[0]] if self.q_rank else tensors[n["q"]]
        for key, w in (("q", first), ("dkv", tensors[n["dkv"]] if self.own_rows else None),
                       ("g", tensors[self.gate_name] if self.output_gate else None)):
            if w is None:
                continue
            self.cols[key] = at
            pad = (-w.shape[0]) % 8
            mats += [w] + ([torch.zeros((pad, w.shape[1]), dtype=w.dtype, device=w.device)] if pad else [])
            at += w.shape[0] + pad
        self.proj = Linear(torch.cat(mats, dim=0).contiguous() if len(mats) > 1 else mats[0])
        del mats, first
        if self.q_rank:
            self.q_norm_weight = tensors[self.query_names[1]]
            self.uq = Linear(tensors[self.query_names[2]])
        self.norm_weight = tensors[n["norm"]] if self.own_rows else None
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
        if not self.own_rows:
            return None
        return PagedLatent(self.row, self.cache_window)

    def _gated(self, o: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
        if not self.output_gate:
            return o
        g = self.cols["g"]
        return ops.sigmoid_gate(o, x[:, g:g + o.shape[1]])

    def forward(self, h: torch.Tensor, ctx, cache) -> torch.Tensor:
        H, D, R, C, Dv = self.num_heads, self.head_dim, self.rot_dim, self.kv_rank, self.v_head_dim
        t = h.shape[0]
        group = ctx.groups[cache.group]
        x = self.proj(h)                       # [tokens, H (D + R) or q_rank | C + R | H Dv], each block padded to 8 columns
        if self.q_rank:
            q = self.uq(ops.rmsnorm(x[:, :self.q_rank], self.q_norm_weight, self.eps))
        else:
            q = x[:, :H * (D + R)]
        writes = cache.writes and self.own_rows
        down = x[:, self.cols["dkv"]:self.cols["dkv"] + C + R] if self.own_rows else None
        slots = group.slot_mapping if writes else None
        interleaved = bool(getattr(self.position, "interleaved", False))
        if (self.raise_w is not None and ctx.max_new >= RAISE_MIN_TOKENS and len(ctx.new_lens) == ctx.n_seqs
                and len(ctx.offsets) == ctx.n_seqs and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0):
            plans = getattr(ctx, "raised_rows", None)   # (made by the step's first latent layer of a window, kept on its context)
            if plans is None:
                plans = ctx.raised_rows = {}
            plan = plans.get(self.window)
            if plan is None:
                plan = plans[self.window] = ops.RaisedPlan([a + b for a, b in zip(ctx.offsets, ctx.new_lens)], x.device,
                                                           ctx.offsets, self.window)
            if plan.rows * H * (D + R + Dv) * 2 <= RAISE_MAX_BYTES:
                ops.latent_prep(down, q, None, self.norm_weight, self.eps, self.rotary[0], interleaved, ctx.positions,
                                slots, cache.pages, H, D, R, C)
                kv = self.raise_w(ops.latent_gather(cache.pages, group.block_table, ctx.cu_seqlens, ctx.kv_offsets, plan))
                o = ops.raised_attention(q, q.stride(0), kv, ctx.cu_seqlens, ctx.kv_offsets, plan, self.scale, H, D + R, Dv,
                                         ctx.max_new)
                return self.out(self._gated(o, x))
        qa = torch.empty((t, H, C + R), dtype=x.dtype, device=x.device)   # folded queries: [W_uk^T q | rotated part]
        ops.latent_prep(down, q, qa, self.norm_weight, self.eps, self.rotary[0], interleaved,
                        ctx.positions, slots, cache.pages, H, D, R, C)
        ops.gemm_heads(q.view(t, H, D + R)[:, :, :D], self.uk_t, qa[:, :, :C])
        latent = ops.latent_attention(qa, cache.pages, group.block_table, ctx.seq_of_token, ctx.positions, self.scale, H, C, R,
                                      max_kv=ctx.max_kv, window=self.window)
        o = torch.empty((t, H, Dv), dtype=x.dtype, device=x.device)
        ops.gemm_heads(latent, self.uv, o)
        return self.out(self._gated(o.view(t, H * Dv), x))
