"""Differential attention: every head takes TWO softmax maps over the same values and keeps their difference.

    q = W_q h   [heads, 2, head_dim]     k = W_k h   [kv_heads, 2, head_dim]     v = W_v h   [kv_heads, v_head_dim]
    per head and map: RMS norm over head_dim (one weight for all queries, one for all keys), then the rotation
    a_m = softmax(q_m . k_m * scale) v   over the visible keys, m = 1, 2 (query head h reads key/value head h // group)
    o   = a_1 - lambda a_2,   lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff   (one number for the layer)
    o   <- o / sqrt(mean(o^2) + eps) * (1 - diff)   over the head's values, times sigmoid(W_g h)_h, then W_o.

In this engine the two maps are 2 * heads query heads over 2 * kv_heads key heads of head_dim channels whose values are
shared by pairs of key heads: the paged cache keeps the key heads [kv head, map] and ONE value head per kv head
(`PagedKV(num_v_heads=kv_heads)`), and the attention kernels take `v_share = 2`.  The rows of W_q are reordered when they
are bound, per kv head all its heads' first maps and then all their second maps, so that the query heads of one key head
lie side by side as the grouped kernels want them.  The projections are one matrix [W_q; W_k; W_v; W_g; zero rows to a
multiple of 8].  The maps come back in float32; `ops.diff_combine` takes the difference, the norm and the gate in float32.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch

from ..csrc import ops
from .base import Mixer, PagedKV, Runtime, TensorSpec
from .linear import Linear
from .plan import PartSpec
from .registry import build_part


class DifferentialAttention(Mixer):
    @property
    def cuda_graph_safe(self) -> bool:
        return self.position is None or bool(self.position.cuda_graph_safe)

    def __init__(self, prefix: str, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, v_head_dim: int,
                 diff: float, scale: Optional[float] = None, eps: float = 1e-6, window: int = 0,
                 position: Optional[PartSpec] = None, qk_norm: bool = True, output_gate: bool = True,
                 names: Sequence[str] = ("q", "k", "v", "o"), norm_names: Sequence[str] = ("q.norm", "k.norm"),
                 lambda_names: Sequence[str] = ("lq1", "lk1", "lq2", "lk2"), gate_name: str = "g"):
        super().__init__(prefix)
        self.hidden_size, self.num_heads, self.num_kv_heads = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.head_dim, self.v_head_dim = int(head_dim), int(v_head_dim)
        if min(self.num_heads, self.num_kv_heads, self.head_dim, self.v_head_dim) <= 0 or self.num_heads % self.num_kv_heads:
            raise ValueError("%sdifferential attention: sizes must be positive and heads a multiple of kv_heads" % prefix)
        if max(self.head_dim, self.v_head_dim) > ops.ATTENTION_MAX_HEAD_DIM or (position is not None and self.head_dim % 2):
            raise ValueError("%shead sizes %d / %d: the attention kernels take even sizes up to %d"
                             % (prefix, self.head_dim, self.v_head_dim, ops.ATTENTION_MAX_HEAD_DIM))
        self.diff, self.eps, self.window = float(diff), float(eps), int(window)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.head_dim)
        self.qk_norm, self.output_gate = bool(qk_norm), bool(output_gate)
        self.position = build_part("position", position) if position is not None else None
        if self.position is not None and self.position.rotary_table("cpu") is None:
            raise ValueError("%sdifferential attention rotates inside its fused kernel and takes a rotary position" % prefix)
        self.names = dict(zip(("q", "k", "v", "o"), (prefix + n for n in names)))
        self.norm_names = tuple(prefix + n for n in norm_names)
        self.lambda_names = tuple(prefix + n for n in lambda_names)
        self.gate_name = prefix + gate_name
        self.qkv: Optional[Linear] = None
        self.out: Optional[Linear] = None
        self.q_norm_weight = self.k_norm_weight = None
        self.lam = 0.0

    @property
    def per_group(self) -> int:
        return self.num_heads // self.num_kv_heads

    @property
    def gate_col(self) -> int:
        if not self.output_gate:
            return -1
        return 2 * (self.num_heads + self.num_kv_heads) * self.head_dim + self.num_kv_heads * self.v_head_dim

    def tensor_specs(self) -> List[TensorSpec]:
        e, H, G, D, Dv, n = self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim, self.v_head_dim, self.names
        specs = [TensorSpec(n["q"], (H * 2 * D, e), "matrix"), TensorSpec(n["k"], (G * 2 * D, e), "matrix"),
                 TensorSpec(n["v"], (G * Dv, e), "matrix"), TensorSpec(n["o"], (e, H * Dv), "matrix")]
        if self.qk_norm:
            specs += [TensorSpec(self.norm_names[0], (D,), "norm"), TensorSpec(self.norm_names[1], (D,), "norm")]
        specs += [TensorSpec(name, (D,), "bias") for name in self.lambda_names]
        if self.output_gate:
            specs.append(TensorSpec(self.gate_name, (H, e), "matrix"))
        if self.position is not None:
            specs.extend(self.position.tensor_specs())
        return specs

    def ignored_tensors(self) -> List[str]:
        return self.position.ignored_tensors() if self.position is not None else []

    def bind(self, tensors: Dict[str, torch.Tensor], runtime: Runtime) -> None:
        super().bind(tensors, runtime)
        H, G, D, per, n = self.num_heads, self.num_kv_heads, self.head_dim, self.per_group, self.names
        wq = tensors[n["q"]].view(G, per, 2, D, self.hidden_size)
        # [kv head, head of the group, map] -> [kv head, map, head of the group]: the query heads of a key head side by side
        mats = [wq.transpose(1, 2).reshape(H * 2 * D, self.hidden_size), tensors[n["k"]], tensors[n["v"]]]
        del wq
        rows = sum(m.shape[0] for m in mats)
        if self.output_gate:
            mats.append(tensors[self.gate_name])
            rows += H
        mats.append(torch.zeros(((-rows) % 8, self.hidden_size), dtype=mats[0].dtype, device=mats[0].device))
        self.qkv = Linear(torch.cat(mats, dim=0).contiguous())
        del mats
        self.out = Linear(tensors[n["o"]])
        if self.qk_norm:
            self.q_norm_weight, self.k_norm_weight = tensors[self.norm_names[0]], tensors[self.norm_names[1]]
        lq1, lk1, lq2, lk2 = (tensors[name].to(torch.float64).cpu() for name in self.lambda_names)
        self.lam = math.exp(float((lq1 * lk1).sum())) - math.exp(float((lq2 * lk2).sum())) + self.diff
        if self.position is not None:
            self.position.bind(tensors, runtime)

    def cache_spec(self):
        return PagedKV(2 * self.num_kv_heads, self.head_dim, self.window,
                       self.v_head_dim if self.v_head_dim != self.head_dim else 0, 0, self.num_kv_heads)

    def forward(self, h: torch.Tensor, ctx, cache) -> torch.Tensor:
        H, G, D, Dv = self.num_heads, self.num_kv_heads, self.head_dim, self.v_head_dim
        group = ctx.groups[cache.group]
        qkv = self.qkv(h)
        inv_freq, rot = self.position.rotary_table(h.device) if self.position is not None else (None, 0)
        ops.qk_norm_rope_kv(qkv, self.q_norm_weight, self.k_norm_weight, self.eps, inv_freq, rot, ctx.positions,
                            group.slot_mapping if cache.writes else None, cache.k_pool, cache.v_pool, 2 * H, 2 * G, D, Dv,
                            interleaved=bool(getattr(self.position, "interleaved", False)), num_v_heads=G,
                            magnitude=float(getattr(self.position, "magnitude", 1.0)))
        maps = self._maps(qkv, ctx, cache, group)
        o = ops.diff_combine(maps, qkv, self.gate_col, self.lam, 1.0 - self.diff, self.eps, H, self.per_group, Dv, qkv.dtype)
        return self.out(o)

    def _maps(self, qkv, ctx, cache, group) -> torch.Tensor:
        """Both maps of every head, [tokens, 2 * heads * v_head_dim]: per kv head its heads' first maps, then their second."""
        H, G, D, Dv = self.num_heads, self.num_kv_heads, self.head_dim, self.v_head_dim
        if ops.biased_attention_supported(qkv.dtype, D, Dv, cache.k_pool.shape[2]):
            # bfloat16 and sizes the tensor-core kernels take (softmax weights in two bfloat16 halves): a step of single tokens
            # has every row's keys dealt to the warps of a block, any other step runs the portion kernel
            if ctx.decode_only:
                return ops.biased_decode_attention(qkv, qkv.shape[1], cache.k_pool, cache.v_pool, group.block_table,
                                                   ctx.seq_of_token, ctx.positions, self.scale, self.window, 0, 0.0, 2 * H, 2 * G, D,
                                                   Dv, qkv.shape[0], max_kv=ctx.max_kv, v_share=2, out_float32=True)
            return ops.biased_prefill_attention(qkv, qkv.shape[1], cache.k_pool, cache.v_pool, group.block_table, ctx.cu_seqlens,
                                                ctx.kv_offsets, self.scale, self.window, 0, 0.0, 2 * H, 2 * G, D, Dv, ctx.n_seqs,
                                                ctx.max_new, qkv.shape[0], v_share=2, out_float32=True)
        return ops.paged_attention_generic(qkv, qkv.shape[1], cache.k_pool, cache.v_pool, group.block_table, ctx.seq_of_token,
                                           ctx.positions, self.scale, self.window, 2 * H, 2 * G, D, qkv.shape[0], v_head_dim=Dv,
                                           v_share=2, out_float32=True)
