"""Linear attention as a recurrence: per head a state S [dim, vdim] with
S_p = a_p (.) S_(p-1) + k_p v_p^T and o_p = S_p^T q_p.  Two mixers share the frame:

`DecayedLinearAttention`: the decay a is a fixed number per head.  q, k = act(W_q h), act(W_k h), v = act(W_v h)
(act: silu or nothing).  Optional, for designs that have them: a rotation of q and k by position (`position`, a
`PartSpec` of a rotary encoding, either layout), multipliers on q and k after it (`q_scale`, `k_scale`), the norm of
the outputs taken per head instead of over the joined heads (`norm="per_head"`, with a weight [vdim] shared by the
heads or none), and silu instead of sigmoid on the gate.  The outputs are normed, multiplied by gate(W_g h) and
projected by W_o.

`GatedLinearAttention`: the decay is a number per key channel and position, a = sigmoid(z)^(1/tau) with
z = W_a2 (W_a1 h) + b, a projection through a narrow middle.  q is multiplied by `q_scale`; the norm is per head with a
weight [vdim] shared by the heads.

The state is float32, starts at zero and lives in the request's state slot (`FixedState`), so a step runs
only the tokens it brings.  The input projections are one matrix here ([W_q; W_k; W_v; W_g (; W_a1)]).  The plain
fixed-decay form has three kernels (`ops.linear_attention`, `csrc/linear_attention.cu`): the recurrence token by
token, chunks of 64 tokens on the tensor cores one after the other, and all chunks side by side with a scan.  With a
rotation, multipliers or a decay per channel the recurrence of `csrc/state_mixers.cu` runs (`ops.linear_attention_walk`):
rotation angles, multipliers, decays (through their logarithm), state and outputs are float32 there, q, k, v enter as
the projection left them.  A step with a portion of 128 tokens or more cuts its rows into stretches (64 tokens, longer in
long steps) that are walked side by side: once from zero for what each adds to the state, a scan over a request's stretches
for the state at the start of each, once more for the outputs (`ops.StretchPlan`).  Norms and gates are float32.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from ..csrc import ops
from .base import FixedState, Mixer, Runtime, TensorSpec
from .linear import Linear
from .plan import PartSpec
from .registry import build_part


class _LinearAttention(Mixer):
    cuda_graph_safe = True  # reads nothing of a step but device tensors and sizes fixed per graph
    KEYS = ("q", "k", "v", "g", "o", "norm")

    def __init__(self, prefix: str, hidden_size: int, num_heads: int, head_dim: int, v_head_dim: int, eps: float,
                 names: Sequence[str], norm: str, norm_weight: bool, gate_activation: str):
        super().__init__(prefix)
        self.hidden_size, self.num_heads = int(hidden_size), int(num_heads)
        self.head_dim, self.v_head_dim, self.eps = int(head_dim), int(v_head_dim), float(eps)
        if not 0 < self.head_dim <= ops.LINEAR_ATTENTION_MAX_DIM:
            raise ValueError("%shead_dim %d: the recurrence kernel takes up to %d" % (prefix, head_dim, ops.LINEAR_ATTENTION_MAX_DIM))
        if norm not in ("joined", "per_head") or gate_activation not in ("sigmoid", "silu"):
            raise ValueError("%snorm is 'joined' or 'per_head' and the gate passes through 'sigmoid' or 'silu'" % prefix)
        if norm == "joined" and (gate_activation != "sigmoid" or not norm_weight):
            raise ValueError("%sthe norm over the joined heads has a weight and a sigmoid gate" % prefix)
        self.norm, self.has_norm_weight, self.gate_activation = norm, bool(norm_weight), gate_activation
        self.names = dict(zip(self.KEYS, (prefix + n for n in names)))
        self.proj: Optional[Linear] = None
        self.out: Optional[Linear] = None
        self.norm_weight = None

    def _input_names(self) -> Sequence[str]:
        return ("q", "k", "v", "g")

    def tensor_specs(self) -> List[TensorSpec]:
        e, qk, vv = self.hidden_size, self.num_heads * self.head_dim, self.num_heads * self.v_head_dim
        n = self.names
        specs = [TensorSpec(n["q"], (qk, e), "matrix"), TensorSpec(n["k"], (qk, e), "matrix"),
                 TensorSpec(n["v"], (vv, e), "matrix"), TensorSpec(n["g"], (vv, e), "matrix"),
                 TensorSpec(n["o"], (e, vv), "matrix")]
        if self.has_norm_weight:
            specs.append(TensorSpec(n["norm"], (vv if self.norm == "joined" else self.v_head_dim,), "norm"))
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor], runtime: Runtime) -> None:
        super().bind(tensors, runtime)
        n = self.names
        self.proj = Linear(torch.cat([tensors[n[x]] for x in self._input_names()], dim=0).contiguous())
        self.out = Linear(tensors[n["o"]])
        self.norm_weight = tensors[n["norm"]] if self.has_norm_weight else None

    def cache_spec(self):
        return FixedState((self.num_heads, self.head_dim, self.v_head_dim), "float32")

    @staticmethod
    def _stretches(ctx):
        """The step's rows cut into stretches that the recurrence walks side by side, from a portion of
        `ops.STRETCH_MIN_TOKENS` rows on; made once a step and kept on its context."""
        if ctx.max_new < ops.STRETCH_MIN_TOKENS or len(ctx.new_lens) != ctx.n_seqs:
            return None
        plan = getattr(ctx, "walk_stretches", None)
        if plan is None:
            plan = ctx.walk_stretches = ops.StretchPlan(ctx.new_lens, ctx.positions.device)
        return plan

    def _finish(self, o: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
        """o float32 [tokens, heads * vdim] -> normed, gated, projected."""
        if self.norm == "joined":
            y = ops.gated_rmsnorm(o, gate, self.norm_weight, self.eps)
        else:
            y = ops.head_norm_gate(o, gate, self.norm_weight, self.num_heads, self.eps, self.gate_activation)
        return self.out(y)


class DecayedLinearAttention(_LinearAttention):
    def __init__(self, prefix: str, hidden_size: int, num_heads: int, head_dim: int, v_head_dim: int,
                 decay: Sequence[float], eps: float = 1e-6, activation: str = "silu",
                 names: Sequence[str] = ("q", "k", "v", "g", "o", "norm"), position: Optional[PartSpec] = None,
                 q_scale: float = 1.0, k_scale: float = 1.0, norm: str = "joined", norm_weight: bool = True,
                 gate_activation: str = "sigmoid"):
        super().__init__(prefix, hidden_size, num_heads, head_dim, v_head_dim, eps, names, norm, norm_weight, gate_activation)
        self.decay_values = [float(d) for d in decay]
        if len(self.decay_values) != self.num_heads:
            raise ValueError("%s%d decays for %d heads" % (prefix, len(self.decay_values), self.num_heads))
        if activation not in ("silu", "none"):
            raise ValueError("%sthe recurrence kernel applies silu or nothing to q, k, v; got %r" % (prefix, activation))
        self.activation = activation
        self.q_scale, self.k_scale = float(q_scale), float(k_scale)
        self.position = build_part("position", position) if position is not None else None
        self.rotary = None
        if self.position is not None:
            if activation != "none":
                raise ValueError("%sa rotation of q and k goes with no activation on them" % prefix)
            if getattr(self.position, "magnitude", 1.0) != 1.0:
                raise ValueError("%sthe state walk rotates without a multiplier of cosines and sines; the position asks for %g"
                                 % (prefix, self.position.magnitude))
            if self.position.rotary_table("cpu") is None:
                raise ValueError("%sthe recurrence kernel rotates by a rotary table; %s has none"
                                 % (prefix, type(self.position).__name__))
        self.decay = None

    @property
    def plain(self) -> bool:
        return self.position is None and self.q_scale == 1.0 and self.k_scale == 1.0

    def tensor_specs(self) -> List[TensorSpec]:
        return super().tensor_specs() + (self.position.tensor_specs() if self.position is not None else [])

    def bind(self, tensors: Dict[str, torch.Tensor], runtime: Runtime) -> None:
        super().bind(tensors, runtime)
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=runtime.device)
        if self.position is not None:
            self.position.bind(tensors, runtime)
            self.rotary = self.position.rotary_table(runtime.device)

    def forward(self, h: torch.Tensor, ctx, cache) -> torch.Tensor:
        H, D, Dv = self.num_heads, self.head_dim, self.v_head_dim
        x = self.proj(h)   # [tokens, q | k | v | g]
        if self.plain:
            o = ops.linear_attention(x, 0, H * D, 2 * H * D, self.decay, cache.state, ctx.cu_seqlens, ctx.state_slots,
                                     ctx.n_seqs, ctx.max_new, H, D, Dv, silu=self.activation == "silu")
        else:
            inv_freq, rot = self.rotary if self.rotary is not None else (None, 0)
            o = ops.linear_attention_walk(x, 0, H * D, 2 * H * D, cache.state, ctx.cu_seqlens, ctx.state_slots, ctx.n_seqs,
                                          H, D, Dv, decay=self.decay, inv_freq=inv_freq, rot_dim=rot,
                                          interleaved=bool(getattr(self.position, "interleaved", False)),
                                          positions=ctx.positions, q_mul=self.q_scale, k_mul=self.k_scale,
                                          stretches=self._stretches(ctx))
        return self._finish(o, x[:, 2 * H * D + H * Dv:2 * H * D + 2 * H * Dv])


class GatedLinearAttention(_LinearAttention):
    KEYS = ("q", "k", "v", "g", "o", "norm", "a1", "a2", "a2_bias")

    def __init__(self, prefix: str, hidden_size: int, num_heads: int, head_dim: int, v_head_dim: int, tau: float,
                 eps: float = 1e-6, q_scale: float = 1.0, decay_rank: Optional[int] = None,
                 names: Sequence[str] = ("q", "k", "v", "g", "o", "norm", "a1", "a2", "a2.b"), norm_weight: bool = True,
                 gate_activation: str = "silu"):
        super().__init__(prefix, hidden_size, num_heads, head_dim, v_head_dim, eps, names, "per_head", norm_weight,
                         gate_activation)
        self.tau, self.q_scale = float(tau), float(q_scale)
        if not self.tau > 0:
            raise ValueError("%stau must be positive, got %r" % (prefix, tau))
        # rows of W_a1; None: read off the tensor when it is bound
        self.decay_rank: Optional[int] = int(decay_rank) if decay_rank else None
        self.decay_up: Optional[Linear] = None

    def _input_names(self) -> Sequence[str]:
        return ("q", "k", "v", "g", "a1")

    def tensor_specs(self) -> List[TensorSpec]:
        n, qk = self.names, self.num_heads * self.head_dim
        r = self.decay_rank or -1   # (not given: whatever the file holds)
        return super().tensor_specs() + [TensorSpec(n["a1"], (r, self.hidden_size), "matrix"),
                                         TensorSpec(n["a2"], (qk, r), "matrix"), TensorSpec(n["a2_bias"], (qk,), "bias")]

    def bind(self, tensors: Dict[str, torch.Tensor], runtime: Runtime) -> None:
        super().bind(tensors, runtime)
        n = self.names
        a2 = tensors[n["a2"]]
        self.decay_rank = int(a2.shape[1])
        if self.proj.weight.shape[0] != 2 * self.num_heads * (self.head_dim + self.v_head_dim) + self.decay_rank:
            raise ValueError("%s and %s disagree about the middle width of the decay's projection" % (n["a1"], n["a2"]))
        self.decay_up = Linear(a2.contiguous(), tensors[n["a2_bias"]])

    def forward(self, h: torch.Tensor, ctx, cache) -> torch.Tensor:
        H, D, Dv = self.num_heads, self.head_dim, self.v_head_dim
        x = self.proj(h)   # [tokens, q | k | v | g | a1]
        g0 = 2 * H * D + H * Dv
        z = self.decay_up(x[:, g0 + H * Dv:g0 + H * Dv + self.decay_rank], torch.float32)   # float32 sums plus the bias
        o = ops.linear_attention_walk(x, 0, H * D, 2 * H * D, cache.state, ctx.cu_seqlens, ctx.state_slots, ctx.n_seqs,
                                      H, D, Dv, gate=z, gate_mul=1.0 / self.tau, q_mul=self.q_scale, stretches=self._stretches(ctx))
        return self._finish(o, x[:, g0:g0 + H * Dv])
