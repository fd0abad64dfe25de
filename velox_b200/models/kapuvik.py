"""Kapuvik as a plan of parts.

Input: the token's row times a multiplier.  Every layer has ONE norm (its multiplier one plus the stored tensor) whose
output the mixer and the feed-forward both read; their outputs are added to the stream together
(`parallel_sublayers`).  The mixer is, layer by layer as config.json lists them, one of
  * two members side by side, summed with a coefficient each: softmax attention over a paged cache (grouped
    key/value heads, values of a size of their own, q and k rotated on their first channels with neighbours paired, a
    score multiplier and a tanh bound on the scores), and linear attention with a fixed decay per head (q and k rotated
    with halves paired, k divided by sqrt(dim), every head's output divided by its root mean square, a silu gate);
  * latent attention: keys and values raised from one normed latent vector per position, plus a rotated key part that
    the heads share; only those two are cached;
  * linear attention with a decay per key channel and position (q divided by sqrt(dim), per-head norm with a weight
    shared by the heads, a silu gate).
The feed-forward is gated with bounds and biases, or absent.  A run of layers may be gone through several times in a row
with the same tensors: the plan's running order names those layers again, each place with a cache or state of its own;
before every pass the stream takes a vector of that pass, and before every pass but the first also the embedding's
output once more.  Output: norm, head, logits bounded by c tanh(logits / c).
Tensor names: `l<i>.` plus `norm1 | mix.left.{q,k,v,o} | mix.right.{q,k,v,g,o} | mix.{q,dkv,dkv.norm,uk,uv,o} |
mix.{q,k,v,g,o,norm,a1,a2,a2.b} | mlp.{gate,up,down}{,.b}`, `embed`, `loop.step`, `final.norm`, `head`.
"""
from __future__ import annotations

from ..config.model_config import KapuvikConfig
from ..config.registry import register_architecture
from ..parts.plan import LayerSpec, ModelPlan, PartSpec, StreamInput

# the feed-forward's activation is g * sigmoid(1.702 g): fixed by the design
FEED_FORWARD_SLOPE = 1.702


def _rotary(rot, head_dim: int, layout: str):
    if not rot:
        return None
    return PartSpec("rotary", "", dict(head_dim=head_dim, theta=float(rot["base"]), rotary_dim=int(rot.get("dims", head_dim)),
                                       layout=layout))


def _mixer(cfg: KapuvikConfig, layer: dict, p: str) -> PartSpec:
    m, kind = layer["mixer"], layer["type"]
    if kind == "parallel":
        left, right = m["left"], m["right"]
        members = [
            PartSpec("paged_attention", p + "left.", dict(
                hidden_size=cfg.width, num_heads=left["heads"], num_kv_heads=left["kv_heads"], head_dim=left["dim"],
                v_head_dim=left["vdim"], bias=False, qk_norm=False, eps=cfg.norm_eps, scale=float(left["scale"]),
                score_softcap=float(left.get("softcap") or 0.0), position=_rotary(left.get("rot"), left["dim"], "interleaved"),
                names=("q", "k", "v", "o"), weights_32bit=True)),
            PartSpec("decayed_linear_attention", p + "right.", dict(
                hidden_size=cfg.width, num_heads=right["heads"], head_dim=right["dim"], v_head_dim=right["vdim"],
                decay=list(right["decay"]), eps=cfg.norm_eps, activation="none", position=_rotary(right.get("rot"), right["dim"], "half"),
                k_scale=float(right["dim"]) ** -0.5, norm="per_head", norm_weight=False, gate_activation="silu")),
        ]
        return PartSpec("parallel", p, dict(hidden_size=cfg.width, members=members, out_norm_names=None, eps=cfg.norm_eps,
                                            coefficients=(float(m.get("left_scale", 1.0)), float(m.get("right_scale", 1.0)))))
    if kind == "latent_attention":
        return PartSpec("latent_attention", p, dict(
            hidden_size=cfg.width, num_heads=m["heads"], head_dim=m["dim"], rot_dim=m["rot_dim"], v_head_dim=m["vdim"],
            kv_rank=m["kv_rank"], scale=float(m["scale"]), eps=cfg.norm_eps,
            position=_rotary(dict(base=m["rot"]["base"], dims=m["rot_dim"]), m["rot_dim"], "interleaved")))
    return PartSpec("gated_linear_attention", p, dict(
        hidden_size=cfg.width, num_heads=m["heads"], head_dim=m["dim"], v_head_dim=m["vdim"], tau=float(m["tau"]),
        eps=cfg.norm_eps, q_scale=float(m["dim"]) ** -0.5, decay_rank=m.get("rank")))


def _feed_forward(cfg: KapuvikConfig, mlp, p: str):
    if mlp is None:
        return None
    return PartSpec("capped_gated_mlp", p, dict(hidden_size=cfg.width, intermediate_size=mlp["ff"], limit=float(mlp["limit"]),
                                                slope=FEED_FORWARD_SLOPE, bias=True))


def kapuvik_plan(cfg: KapuvikConfig) -> ModelPlan:
    norm = lambda name: PartSpec("rms_norm", name, dict(size=cfg.width, eps=cfg.norm_eps, weight_name="", one_plus=True))
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = "l%d." % i
        layers.append(LayerSpec(mixer=_mixer(cfg, layer, p + "mix."), feed_forward=_feed_forward(cfg, layer.get("mlp"), p + "mlp."),
                                norms={"shared": norm(p + "norm1")}, block="parallel_sublayers"))
    n = len(layers)
    order, inputs = list(range(n)), []
    if cfg.looped:
        a, b, times = cfg.loop_start, cfg.loop_stop, cfg.loop_times
        order = list(range(a))
        for t in range(times):
            inputs.append(StreamInput(place=len(order), embedding=t > 0, tensor="loop.step", row=t, rows=times))
            order += list(range(a, b))
        order += list(range(b, n))
    return ModelPlan(
        vocab_size=cfg.vocab, hidden_size=cfg.width,
        embedding=PartSpec("token_embedding", "", dict(vocab_size=cfg.vocab, hidden_size=cfg.width, scale=cfg.embedding_scale,
                                                       weight_name="embed")),
        layers=layers, final_norm=norm("final.norm"),
        head=PartSpec("linear_head", "head", dict(vocab_size=cfg.vocab, hidden_size=cfg.width, weight_name="",
                                                  logit_softcap=cfg.logit_softcap)),
        order=order, stream_inputs=inputs)


register_architecture(KapuvikConfig.architecture, KapuvikConfig.model_type, KapuvikConfig, kapuvik_plan)
