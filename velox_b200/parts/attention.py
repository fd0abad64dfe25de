"""Attention over a paged cache of keys and values: the mixer of Qwen3.

In the reference's order (src/paged/qwen3.rs:428-448, 584-642):
q/k/v projections -> RMSNorm of each q and k head over head_dim (before the
rotation, not on v) -> rotation at position kv_offset + t -> new k (normed,
rotated) and v (raw) written into the pages -> causal attention over the
request's pages, scale 1/sqrt(head_dim), grouped heads -> output projection
whose input width is heads * head_dim.  The three projections are one matrix
here ([Wq; Wk; Wv], rows in that order), which the reference keeps apart
(src/paged/qwen3.rs:428-430).

Everything is a parameter: head counts, head size, whether q/k are normed,
whether projections are biased, the window (0: all keys), the scale, and the
position encoding (a `PartSpec` of category "position").

Three more, for designs that put positions into the scores instead of rotating:
`v_head_dim` (values of another size than keys; the output projection then takes
heads * v_head_dim), `keep_first` (with a window, the first positions stay visible
to every later query, at their true distances), and `distance_bias_exponent` b > 0
(head h's scores lose 2^(-b (h+1) / heads) * (query position - key position) before
the softmax; 0: no bias).  With any of them the step's keys and values are written by
the plain store kernel (by the q/k norm's kernel, if q and k are normed or rotated: it takes a
value size of its own) and the attention runs in the kernels that know them
(`csrc/attention_biased.cu` for bfloat16, the general kernel otherwise).  `names` renames the four matrices
and `norm_names` the two q/k norm weights.

Two more, for designs that let a head attend to nothing and gate what it found:
`sink` (a learned float32 per query head, tensor `sink_name`): the softmax's denominator also holds
exp(sink_h), an entry without key or value that is not scaled, so a row's weights sum to less than one;
`output_gate` (a matrix [heads, hidden], tensor `gate_name`): head h's output is multiplied by
sigmoid(W_g x)_h before the output projection; W_g reads the mixer's input and rides as further rows of the
fused projection matrix ([Wq; Wk; Wv; Wg], zero rows up to a multiple of 8), and the attention kernels apply
the gate as they write a head's output.

And two for designs that bound their scores and rotate neighbours: `score_softcap` c > 0 (a scaled score s becomes
c tanh(s / c) before the softmax) and a rotary position whose `layout` is "interleaved" (channel 2i paired with
2i + 1; the q/k kernel takes the layout as a flag).  `weights_32bit` asks for the kernels that keep the softmax weights
in 32 bits (two bfloat16 halves on the tensor cores) also where nothing else of the layer needs them.
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


TC_PREFILL_MIN_TOKENS = 32   # longest portion of a step from which the tcgen05 kernel is used


class PagedAttention(Mixer):
    # Requests that bring fewer tokens than the tcgen05 kernel's shortest portion are listed token by
    # token in the step's description (`single_rows`): every token goes to the decode kernel as a query
    # of its own, its request's keys cut into pieces of 256 that many warps share.  A prompt kernel gives
    # such a portion one block per kv head that walks ALL the request's keys alone: 16 tokens on top of
    # 4,000 cached keys took 300 us a layer that way.
    short_rows_up_to = TC_PREFILL_MIN_TOKENS - 1

    @property
    def cuda_graph_safe(self) -> bool:
        # reads nothing of a step but device tensors and sizes fixed per graph; a position
        # encoding of its own kind has to say the same of itself
        return self.position is None or bool(self.position.cuda_graph_safe)

    def __init__(self, prefix: str, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 bias: bool = False, qk_norm: bool = True, eps: float = 1e-6, window: int = 0,
                 position: Optional[PartSpec] = None, scale: Optional[float] = None, v_head_dim: int = 0,
                 keep_first: int = 0, distance_bias_exponent: float = 0.0,
                 names: Sequence[str] = ("q_proj.weight", "k_proj.weight", "v_proj.weight", "o_proj.weight"),
                 norm_names: Sequence[str] = ("q_norm.weight", "k_norm.weight"), sink: bool = False,
                 output_gate: bool = False, sink_name: str = "sink", gate_name: str = "g", score_softcap: float = 0.0,
                 weights_32bit: bool = False):
        super().__init__(prefix)
        self.softcap = float(score_softcap)
        self.weights_32bit = bool(weights_32bit)
        if self.softcap < 0:
            raise ValueError("%sscore_softcap must not be negative" % prefix)
        self.names = dict(zip(("q_proj", "k_proj", "v_proj", "o_proj"), names))
        self.norm_names = (prefix + norm_names[0], prefix + norm_names[1])
        self.sink, self.output_gate = bool(sink), bool(output_gate)
        self.sink_name, self.gate_name = prefix + sink_name, prefix + gate_name
        self.sinks = None
        if num_heads % num_kv_heads:
            raise ValueError("num_heads %d is not a multiple of num_kv_heads %d" % (num_heads, num_kv_heads))
        plain = position is None   # (no rotation: the norm and the general attention kernel take odd sizes too)
        if not (ops.attention_head_dim_supported(int(head_dim)) or (plain and 0 < int(head_dim) <= ops.ATTENTION_MAX_HEAD_DIM)):
            raise ValueError("%shead_dim %d: the attention kernels take even head sizes up to %d"
                             % (prefix, head_dim, ops.ATTENTION_MAX_HEAD_DIM))
        self.v_head_dim = int(v_head_dim) or int(head_dim)
        self.keep_first, self.bias_exponent = int(keep_first), float(distance_bias_exponent)
        if self.keep_first < 0 or self.bias_exponent < 0:
            raise ValueError("%skeep_first and distance_bias_exponent must not be negative" % prefix)
        if not 0 < self.v_head_dim <= ops.ATTENTION_MAX_HEAD_DIM:
            raise ValueError("%sv_head_dim %d: the attention kernels take sizes up to %d"
                             % (prefix, self.v_head_dim, ops.ATTENTION_MAX_HEAD_DIM))
        self.hidden_size, self.num_heads, self.num_kv_heads = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.head_dim, self.bias, self.qk_norm = int(head_dim), bool(bias), bool(qk_norm)
        self.eps, self.window = float(eps), int(window)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.head_dim)
        self.position = build_part("position", position) if position is not None else None
        self.qkv: Optional[Linear] = None
        self.out: Optional[Linear] = None
        self.q_norm_weight = self.k_norm_weight = None

    # -- weights -------------------------------------------------------------
    def _proj_rows(self):
        d = self.head_dim
        return {"q_proj": self.num_heads * d, "k_proj": self.num_kv_heads * d, "v_proj": self.num_kv_heads * self.v_head_dim}

    def _w(self, name: str) -> str:
        return self.prefix + self.names[name]

    @property
    def extended(self) -> bool:
        """True if the layer uses what only the kernels for biased, unequal or kept-first attention know."""
        return (self.v_head_dim != self.head_dim or self.keep_first > 0 or self.bias_exponent > 0 or self.sink
                or self.output_gate or self.softcap > 0 or self.weights_32bit)

    @property
    def gate_col(self) -> int:
        """The column of head 0's gate in a row of the fused projection, or -1."""
        if not self.output_gate:
            return -1
        return (self.num_heads + self.num_kv_heads) * self.head_dim + self.num_kv_heads * self.v_head_dim


    def tensor_specs(self) -> List[TensorSpec]:
        p, specs = self.prefix, []
        for name, rows in self._proj_rows().items():
            specs.append(TensorSpec(self._w(name), (rows, self.hidden_size), "matrix"))
            if self.bias:
                specs.append(TensorSpec(p + name + ".bias", (rows,), "bias"))
        specs.append(TensorSpec(self._w("o_proj"), (self.hidden_size, self.num_heads * self.v_head_dim), "matrix"))
        if self.bias:
            specs.append(TensorSpec(p + "o_proj.bias", (self.hidden_size,), "bias"))
        if self.qk_norm:
            specs.append(TensorSpec(self.norm_names[0], (self.head_dim,), "norm"))
            specs.append(TensorSpec(self.norm_names[1], (self.head_dim,), "norm"))
        if self.sink:
            specs.append(TensorSpec(self.sink_name, (self.num_heads,), "bias"))
        if self.output_gate:
            specs.append(TensorSpec(self.gate_name, (self.num_heads, self.hidden_size), "matrix"))
        if self.position is not None:
            specs.extend(self.position.tensor_specs())
        return specs

    def ignored_tensors(self) -> List[str]:
        return self.position.ignored_tensors() if self.position is not None else []

    def bind(self, tensors: Dict[str, torch.Tensor], runtime: Runtime) -> None:
        super().bind(tensors, runtime)
        p = self.prefix
        mats = [tensors[self._w(n)] for n in ("q_proj", "k_proj", "v_proj")]
        biases = [tensors[p + n + ".bias"] for n in ("q_proj", "k_proj", "v_proj")] if self.bias else None
        if self.output_gate:
            # the gates' rows, then zero rows up to a multiple of 8 (rows of the projection stay 16-byte aligned)
            g = tensors[self.gate_name]
            rows = sum(m.shape[0] for m in mats) + g.shape[0]
            mats += [g, torch.zeros(((-rows) % 8, self.hidden_size), dtype=g.dtype, device=g.device)]
            if biases is not None:
                biases.append(torch.zeros(mats[-2].shape[0] + mats[-1].shape[0], dtype=biases[0].dtype, device=g.device))
        w = torch.cat(mats, dim=0).contiguous()
        b = torch.cat(biases).contiguous() if biases is not None else None
        del mats
        self.qkv = Linear(w, b)
        if self.sink:
            self.sinks = tensors[self.sink_name].to(torch.float32).contiguous()
        self.out = Linear(tensors[self._w("o_proj")], tensors[p + "o_proj.bias"] if self.bias else None)
        if self.qk_norm:
            self.q_norm_weight, self.k_norm_weight = tensors[self.norm_names[0]], tensors[self.norm_names[1]]
        if self.position is not None:
            self.position.bind(tensors, runtime)

    # -- cache ---------------------------------------------------------------
    def cache_spec(self):
        if not self.extended:
            return PagedKV(self.num_kv_heads, self.head_dim, self.window)
        return PagedKV(self.num_kv_heads, self.head_dim, self.window,
                       self.v_head_dim if self.v_head_dim != self.head_dim else 0, self.keep_first if self.window else 0)

    # -- step ----------------------------------------------------------------
    def forward(self, h: torch.Tensor, ctx, cache) -> torch.Tensor:
        H, Hk, D = self.num_heads, self.num_kv_heads, self.head_dim
        group = ctx.groups[cache.group]
        qkv = self.qkv(h)
        slots = group.slot_mapping if cache.writes else None
        if self.extended and not self.qk_norm and self.position is None:
            # plain projections: nothing to norm or rotate, the step's keys and values go into their pages as they are
            if slots is not None:
                ops.kv_store(qkv, H * D, (H + Hk) * D, slots, cache.k_pool, cache.v_pool)
            return self.out(self._attend_extended(qkv, ctx, cache, group))
        rotary = self.position.rotary_table(h.device) if self.position is not None else None
        qw, kw = self.q_norm_weight, self.k_norm_weight
        if self.position is None or rotary is not None:
            inv_freq, rot = rotary if rotary is not None else (None, 0)
            ops.qk_norm_rope_kv(qkv, qw, kw, self.eps, inv_freq, rot, ctx.positions, slots,
                                cache.k_pool, cache.v_pool, H, Hk, D, self.v_head_dim,
                                interleaved=bool(getattr(self.position, "interleaved", False)),
                                magnitude=float(getattr(self.position, "magnitude", 1.0)))
        else:
            # An encoding the fused kernel does not know: norm in place, let the
            # part encode q and k in place, then write the cache.
            t = qkv.shape[0]
            ops.qk_norm_rope_kv(qkv, qw, kw, self.eps, None, 0, ctx.positions, None, None, None, H, Hk, D, self.v_head_dim)
            q, k = qkv[:, : H * D].view(t, H, D), qkv[:, H * D : (H + Hk) * D].view(t, Hk, D)
            q2, k2 = self.position.apply(q, k, ctx.positions)
            if q2 is not q:
                q.copy_(q2)
            if k2 is not k:
                k.copy_(k2)
            ops.qk_norm_rope_kv(qkv, None, None, self.eps, None, 0, ctx.positions, slots,
                                cache.k_pool, cache.v_pool, H, Hk, D, self.v_head_dim)
        attn = self._attend_extended(qkv, ctx, cache, group) if self.extended else self._attend(qkv, ctx, cache, group)
        return self.out(attn)

    def _attend_extended(self, qkv, ctx, cache, group) -> torch.Tensor:
        H, Hk, D = self.num_heads, self.num_kv_heads, self.head_dim
        more = dict(sinks=self.sinks, gate_col=self.gate_col)
        capped = dict(more, softcap=self.softcap)
        page = cache.k_pool.shape[2]
        if (not ctx.decode_only and ctx.max_new >= TC_PREFILL_MIN_TOKENS and self.keep_first == 0 and self.bias_exponent == 0
                and self.softcap == 0 and self.v_head_dim == D and ops.prefill_attention_tc_supported(qkv.dtype, D, page, H // Hk)):
            # prompt portions of heads of 128 without a bias by distance: the tcgen05 kernel, with the probabilities in two
            # bfloat16 halves (this path's softmax weights are 32-bit), the sink and the gate in its epilogue
            return ops.paged_prefill_attention_tc(qkv, qkv.shape[1], cache.k_pool, cache.v_pool, group.block_table, ctx.cu_seqlens,
                                                  ctx.kv_offsets, self.scale, self.window, H, Hk, D, ctx.n_seqs, ctx.max_new,
                                                  qkv.shape[0], max_kv=ctx.max_kv, halves=True, **more)
        if ops.biased_attention_supported(qkv.dtype, D, self.v_head_dim, cache.k_pool.shape[2]):
            # a step of single tokens: every row with its own position, its keys dealt to the warps of a block
            if ctx.decode_only:
                return ops.biased_decode_attention(qkv, qkv.shape[1], cache.k_pool, cache.v_pool, group.block_table,
                                                   ctx.seq_of_token, ctx.positions, self.scale, self.window,
                                                   self.keep_first, self.bias_exponent, H, Hk, D, self.v_head_dim,
                                                   qkv.shape[0], max_kv=ctx.max_kv, **capped)
            return ops.biased_prefill_attention(qkv, qkv.shape[1], cache.k_pool, cache.v_pool, group.block_table,
                                                ctx.cu_seqlens, ctx.kv_offsets, self.scale, self.window, self.keep_first,
                                                self.bias_exponent, H, Hk, D, self.v_head_dim, ctx.n_seqs, ctx.max_new,
                                                qkv.shape[0], **capped)
        return ops.paged_attention_generic(qkv, qkv.shape[1], cache.k_pool, cache.v_pool, group.block_table,
                                           ctx.seq_of_token, ctx.positions, self.scale, self.window, H, Hk, D,
                                           qkv.shape[0], v_head_dim=self.v_head_dim, keep_first=self.keep_first,
                                           bias_exponent=self.bias_exponent, softcap=self.softcap, **more)

    def _attend(self, qkv, ctx, cache, group) -> torch.Tensor:
        H, Hk, D = self.num_heads, self.num_kv_heads, self.head_dim
        if ctx.decode_only and ops.decode_attention_supported(qkv.dtype, D, cache.k_pool.shape[2], H // Hk):
            # one token per request: token row i is request i
            return ops.paged_decode_attention(qkv, qkv.shape[1], cache.k_pool, cache.v_pool, group.block_table,
                                              ctx.seq_of_token, ctx.positions, self.scale, self.window, H, Hk, D,
                                              ctx.n_seqs, ctx.max_kv)
        page = cache.k_pool.shape[2]
        use_tc = ctx.max_new >= TC_PREFILL_MIN_TOKENS and ops.prefill_attention_tc_supported(qkv.dtype, D, page, H // Hk)
        if use_tc or ops.prefill_attention_supported(qkv.dtype, D, page):
            prefill = ops.paged_prefill_attention_tc if use_tc else ops.paged_prefill_attention  # tcgen05 | mma.sync
            out, seqs, n = None, None, ctx.n_seqs
            if ctx.n_single and ops.decode_attention_supported(qkv.dtype, D, page, H // Hk):
                # A mixed step: the tokens of requests that bring one token, or a few, go to the
                # decode kernel (a warp per 256 keys), not into a query tile of their own; the
                # kernels write disjoint rows.  A decoded token's result is then the same bits
                # whether or not prompt portions ride in its step.
                out = torch.empty((qkv.shape[0], H * D), dtype=qkv.dtype, device=qkv.device)
                ops.paged_decode_attention(qkv, qkv.shape[1], cache.k_pool, cache.v_pool, group.block_table,
                                           ctx.seq_of_token, ctx.positions, self.scale, self.window, H, Hk, D,
                                           ctx.n_single, ctx.max_kv_single, token_rows=ctx.single_rows, out=out,
                                           single_tokens=ctx.max_short <= 1)
                if ctx.n_portions == 0:
                    return out
                seqs, n = ctx.portion_seqs, ctx.n_portions
            more = dict(max_kv=ctx.max_kv) if use_tc else {}   # (short portions on many keys: cut into runs of key tiles)
            return prefill(qkv, qkv.shape[1], cache.k_pool, cache.v_pool, group.block_table, ctx.cu_seqlens,
                           ctx.kv_offsets, self.scale, self.window, H, Hk, D, n, ctx.max_new, qkv.shape[0],
                           seq_list=seqs, out=out, **more)
        return ops.paged_attention_generic(qkv, qkv.shape[1], cache.k_pool, cache.v_pool, group.block_table,
                                           ctx.seq_of_token, ctx.positions, self.scale, self.window, H, Hk, D,
                                           qkv.shape[0])
