"""Fovenex as a plan of parts.

Input: the token's row.  The stream is kept in `streams` copies that every sublayer reads as a weighted sum and writes
back to while they are mixed among themselves (`hyper_connections`; with no `streams` it is the plain pre-norm layer),
every sublayer's output scaled channel by channel and by one multiplier of the model.  Norms are layer norms without
bias.  The mixer is, layer by layer as config.json lists them, one of
  * differential attention: two softmax maps per head over shared values (grouped key/value heads, values of a size of
    their own, q and k RMS-normed per head and map and rotated on their first channels with halves paired, the
    frequencies optionally stretched for long contexts), their difference normed per head and gated per head;
  * latent attention: queries through a normed latent vector of their own; keys and values raised from one normed latent
    vector per position plus a rotated key part that the heads share; a sliding window; a gate element by element.  A
    layer may read the rows that an earlier layer cached instead of making its own.
The feed-forward is down(gelu_tanh(up(h))), or absent.  Output: the layer norm of the sum of the copies, head.
Tensor names: `l<i>.` plus `norm1 | norm2 | ls1 | ls2 | hc{1,2}.{in,out,mix} | mix.{q,k,v,o,g,q.norm,k.norm,lq1,lk1,lq2,lk2}
| mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,g,o} | mlp.{up,down}`, `embed`, `final.norm`, `head`.
"""
from __future__ import annotations

from ..config.model_config import FovenexConfig
from ..config.registry import register_architecture
from ..parts.plan import LayerSpec, ModelPlan, PartSpec

# the feed-forward's activation is the tanh form of gelu: fixed by the design
FEED_FORWARD_ACTIVATION = "gelu_pytorch_tanh"


def _mixer(cfg: FovenexConfig, i: int, p: str) -> PartSpec:
    layer = cfg.layers[i]
    m = layer["mixer"]
    if layer["type"] == "attention":
        rot = m.get("rot")
        position = None
        if rot:
            position = PartSpec("rotary", "", dict(head_dim=m["dim"], theta=float(rot["base"]), rotary_dim=int(rot["dims"]),
                                                   layout="half", scaling=rot.get("scaling")))
        return PartSpec("differential_attention", p, dict(
            hidden_size=cfg.width, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"], v_head_dim=m["vdim"],
            diff=float(m["diff"]), scale=float(m["scale"]), eps=cfg.norm_eps, window=cfg.window_of(m), position=position))
    window = cfg.window_of(m)
    # the rows are kept as long as the longest window among the layer itself and the layers that read its rows
    windows = [window] + [cfg.window_of(cfg.layers[j]["mixer"]) for j in range(len(cfg.layers)) if cfg.rows_source(j) == i]
    return PartSpec("latent_attention", p, dict(
        hidden_size=cfg.width, num_heads=m["heads"], head_dim=m["dim"], rot_dim=m["rot_dim"], v_head_dim=m["vdim"],
        kv_rank=m["kv_rank"], scale=float(m["scale"]), eps=cfg.norm_eps, q_rank=int(m.get("q_rank") or 0), window=window,
        cache_window=0 if min(windows) == 0 else max(windows), output_gate=True, own_rows=m.get("kv_from") is None,
        position=PartSpec("rotary", "", dict(head_dim=m["rot_dim"], theta=float(m["rot"]["base"]), rotary_dim=m["rot_dim"],
                                             layout="half"))))


def fovenex_plan(cfg: FovenexConfig) -> ModelPlan:
    norm = lambda name, streams=1: PartSpec("layer_norm", name, dict(size=cfg.width, eps=cfg.norm_eps, weight_name="", streams=streams))
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = "l%d." % i
        mlp = layer.get("mlp")
        feed_forward = None
        norms = {"mixer": norm(p + "norm1")}
        if mlp is not None:
            feed_forward = PartSpec("dense_mlp", p + "mlp.", dict(hidden_size=cfg.width, intermediate_size=mlp["ff"],
                                                                  activation=FEED_FORWARD_ACTIVATION, names=("up", "down")))
            norms["feed_forward"] = norm(p + "norm2")
        layers.append(LayerSpec(mixer=_mixer(cfg, i, p + "mix."), feed_forward=feed_forward, norms=norms, block="hyper_connections",
                                cache_of=cfg.rows_source(i),
                                block_params=dict(hidden_size=cfg.width, streams=cfg.streams, residual_mult=cfg.residual_mult, prefix=p)))
    return ModelPlan(
        vocab_size=cfg.vocab, hidden_size=cfg.width,
        embedding=PartSpec("token_embedding", "", dict(vocab_size=cfg.vocab, hidden_size=cfg.width, weight_name="embed")),
        layers=layers, final_norm=norm("final.norm", max(cfg.streams, 1)),
        head=PartSpec("linear_head", "head", dict(vocab_size=cfg.vocab, hidden_size=cfg.width, weight_name="")))


register_architecture(FovenexConfig.architecture, FovenexConfig.model_type, FovenexConfig, fovenex_plan)
