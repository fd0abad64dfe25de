"""Typed model configurations, read from an architecture's own config.json keys.

`Qwen3Config` holds exactly the keys that the reference's `Qwen3Config`
deserialises (src/paged/qwen3.rs:30-60): thirteen required keys, three
optional ones about the sliding window, unknown keys ignored.  Nothing here
knows a model size: every number comes from the file or from the caller.
"""
from __future__ import annotations

import dataclasses
import json
import os
from dataclasses import dataclass
from typing import Any, ClassVar, Dict, Optional, Tuple


class ConfigError(ValueError):
    """A config.json that cannot describe a model: lists every fault found."""


def _typed(name: str, value: Any, kind: type, faults: list) -> Any:
    if kind is float and isinstance(value, (int, float)) and not isinstance(value, bool):
        return float(value)
    if kind is int and isinstance(value, int) and not isinstance(value, bool):
        return value
    if kind is bool and isinstance(value, bool):
        return value
    if kind is str and isinstance(value, str):
        return value
    faults.append("key %r: expected %s, got %r" % (name, kind.__name__, value))
    return None


@dataclass(frozen=True)
class ModelConfig:
    """Base of the typed configurations.  A subclass lists its keys as
    dataclass fields; a field without a default is a required key."""

    architecture: ClassVar[str] = ""
    model_type: ClassVar[str] = ""

    # keys that, when present and not null, name something this engine does not do
    unsupported_keys: ClassVar[Dict[str, str]] = {}

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "ModelConfig":
        faults: list = []
        values: Dict[str, Any] = {}
        for key, why in cls.unsupported_keys.items():
            if raw.get(key) is not None:
                faults.append("key %r: %s" % (key, why))
        for f in dataclasses.fields(cls):
            required = f.default is dataclasses.MISSING and f.default_factory is dataclasses.MISSING
            if f.name not in raw or raw[f.name] is None:
                if required:
                    faults.append("missing key %r" % f.name)
                continue
            kind = f.metadata.get("kind", f.type)
            values[f.name] = _typed(f.name, raw[f.name], kind, faults)
        if faults:
            raise ConfigError("config.json for %s: %s" % (cls.__name__, "; ".join(faults)))
        cfg = cls(**values)
        cfg.validate()
        return cfg

    @classmethod
    def from_folder(cls, folder: str) -> "ModelConfig":
        return cls.from_dict(read_config_json(folder))

    def to_dict(self) -> Dict[str, Any]:
        """The config.json that `from_dict` reads back to this configuration."""
        out: Dict[str, Any] = {"architectures": [self.architecture], "model_type": self.model_type}
        out.update(dataclasses.asdict(self))
        return out

    def validate(self) -> None:  # pragma: no cover - overridden
        pass


def read_config_json(folder: str) -> Dict[str, Any]:
    path = os.path.join(folder, "config.json")
    if not os.path.isfile(path):
        raise ConfigError("no config.json in %s" % folder)
    with open(path) as f:
        raw = json.load(f)
    if not isinstance(raw, dict):
        raise ConfigError("%s does not hold a JSON object" % path)
    return raw


def _field(kind: type, **kw):
    return dataclasses.field(metadata={"kind": kind}, **kw)


SUPPORTED_ACTIVATIONS: Tuple[str, ...] = ("silu", "gelu", "gelu_pytorch_tanh", "relu")


@dataclass(frozen=True)
class Qwen3Config(ModelConfig):
    """Qwen3 dense decoder (src/paged/qwen3.rs:30-60).

    `head_dim` is its own key and need not be hidden_size / heads
    (src/paged/qwen3.rs:36, 390).  The window keys are optional and default
    to "no window" (src/paged/qwen3.rs:41-48)."""

    architecture: ClassVar[str] = "Qwen3ForCausalLM"
    model_type: ClassVar[str] = "qwen3"
    # the reference reads 4-bit checkpoints through these (src/paged/qwen3.rs:51-59)
    unsupported_keys: ClassVar[Dict[str, str]] = {
        "quantization": "quantized weights are not supported; the engine holds bfloat16 or float32",
        "quantization_config": "quantized weights are not supported; the engine holds bfloat16 or float32",
    }

    vocab_size: int = _field(int)
    hidden_size: int = _field(int)
    intermediate_size: int = _field(int)
    num_hidden_layers: int = _field(int)
    num_attention_heads: int = _field(int)
    head_dim: int = _field(int)
    attention_bias: bool = _field(bool)
    num_key_value_heads: int = _field(int)
    max_position_embeddings: int = _field(int)
    tie_word_embeddings: bool = _field(bool)
    rope_theta: float = _field(float)
    rms_norm_eps: float = _field(float)
    hidden_act: str = _field(str)
    sliding_window: Optional[int] = _field(int, default=None)
    max_window_layers: int = _field(int, default=0)
    use_sliding_window: bool = _field(bool, default=False)

    def validate(self) -> None:
        faults = []
        for name in (
            "vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
            "num_attention_heads", "head_dim", "num_key_value_heads", "max_position_embeddings",
        ):
            if getattr(self, name) <= 0:
                faults.append("%s must be positive, got %d" % (name, getattr(self, name)))
        if not faults:
            # the reference divides without checking (src/paged/qwen3.rs:385)
            if self.num_attention_heads % self.num_key_value_heads:
                faults.append(
                    "num_attention_heads (%d) is not a multiple of num_key_value_heads (%d)"
                    % (self.num_attention_heads, self.num_key_value_heads)
                )
            if self.head_dim % 2:
                faults.append("head_dim (%d) must be even for the rotation" % self.head_dim)
        if not self.rope_theta > 0:
            faults.append("rope_theta must be positive, got %r" % self.rope_theta)
        if not self.rms_norm_eps > 0:
            faults.append("rms_norm_eps must be positive, got %r" % self.rms_norm_eps)
        if self.hidden_act not in SUPPORTED_ACTIVATIONS:
            faults.append("hidden_act %r is not one of %s" % (self.hidden_act, list(SUPPORTED_ACTIVATIONS)))
        if self.use_sliding_window and not (self.sliding_window and self.sliding_window > 0):
            faults.append("use_sliding_window needs a positive sliding_window")
        if self.max_window_layers < 0:
            faults.append("max_window_layers must not be negative")
        if faults:
            raise ConfigError("Qwen3 configuration: " + "; ".join(faults))

    def window_of_layer(self, layer: int) -> int:
        """Keys a layer's queries see besides themselves, 0 for all.  The
        reference gives `sliding_window` to every layer when
        `use_sliding_window` is set (src/paged/qwen3.rs:373-381) and reads
        `max_window_layers` without using it (default 0, :43-44).  Here the
        first `max_window_layers` layers see everything and the later ones the
        window; at the default of 0 that is the reference's behaviour."""
        if not self.use_sliding_window or not self.sliding_window:
            return 0
        return int(self.sliding_window) if layer >= self.max_window_layers else 0


@dataclass(frozen=True)
class DobepelConfig(ModelConfig):
    """Dobepel: a decoder whose config.json is nested and lists its layers one by one.

        architecture   "Dobepel"
        vocab, width, residual_mult, norm.eps
        embedding.bigram   buckets, mul_prev, mul_cur
        layers[i]      type ("parallel"), mixer.left (heads, kv_heads, dim, vdim, scale, mask.size,
                       mask.keep_first), mixer.right (heads, dim, vdim, decay per head),
                       mlp: null | kind "dense" (ff) | kind "moe" (expert.ff, router.experts,
                       router.top, shared.ff or no shared)

    Every size and constant is read from there; the layers may differ from one another."""

    architecture: ClassVar[str] = "Dobepel"
    model_type: ClassVar[str] = "dobepel"
    LAYER_TYPES: ClassVar[Tuple[str, ...]] = ("parallel",)

    vocab: int = _field(int)
    width: int = _field(int)
    residual_mult: float = _field(float)
    norm_eps: float = _field(float)
    bigram_buckets: int = _field(int)
    bigram_mul_prev: int = _field(int)
    bigram_mul_cur: int = _field(int)
    layers: Tuple[Dict[str, Any], ...] = _field(tuple, default=())

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "DobepelConfig":
        faults: list = []

        def get(d, path, kind, default=dataclasses.MISSING):
            cur = d
            for key in path.split("."):
                if not isinstance(cur, dict) or cur.get(key) is None:
                    if default is dataclasses.MISSING:
                        faults.append("missing key %r" % path)
                    return None if default is dataclasses.MISSING else default
                cur = cur[key]
            return _typed(path, cur, kind, faults)

        values = dict(vocab=get(raw, "vocab", int), width=get(raw, "width", int),
                      residual_mult=get(raw, "residual_mult", float, 1.0), norm_eps=get(raw, "norm.eps", float),
                      bigram_buckets=get(raw, "embedding.bigram.buckets", int),
                      bigram_mul_prev=get(raw, "embedding.bigram.mul_prev", int),
                      bigram_mul_cur=get(raw, "embedding.bigram.mul_cur", int))
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            faults.append("key 'layers': expected a list of layers")
            layers = []
        if faults:
            raise ConfigError("config.json for %s: %s" % (cls.__name__, "; ".join(faults)))
        cfg = cls(layers=tuple(json.loads(json.dumps(layer)) for layer in layers), **values)
        cfg.validate()
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architecture,
                "embedding": {"bigram": {"buckets": self.bigram_buckets, "mul_prev": self.bigram_mul_prev,
                                         "mul_cur": self.bigram_mul_cur}},
                "layers": json.loads(json.dumps(list(self.layers))), "norm": {"eps": self.norm_eps},
                "residual_mult": self.residual_mult, "vocab": self.vocab, "width": self.width}

    def validate(self) -> None:
        faults = []

        def positive(where, d, *keys):
            for k in keys:
                v = d.get(k) if isinstance(d, dict) else None
                if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
                    faults.append("%s.%s must be a positive integer, got %r" % (where, k, v))
                    return False
            return True

        for name in ("vocab", "width", "bigram_buckets"):
            if getattr(self, name) <= 0:
                faults.append("%s must be positive, got %d" % (name, getattr(self, name)))
        if self.bigram_mul_prev < 0 or self.bigram_mul_cur < 0:
            faults.append("the bigram multipliers must not be negative")
        if not self.norm_eps > 0:
            faults.append("norm.eps must be positive, got %r" % self.norm_eps)
        for i, layer in enumerate(self.layers):
            at = "layers[%d]" % i
            if not isinstance(layer, dict) or layer.get("type") not in self.LAYER_TYPES:
                faults.append("%s.type %r is not one of %s" % (at, layer.get("type") if isinstance(layer, dict) else layer,
                                                               list(self.LAYER_TYPES)))
                continue
            mixer = layer.get("mixer") or {}
            left, right = mixer.get("left"), mixer.get("right")
            if positive(at + ".mixer.left", left, "heads", "kv_heads", "dim", "vdim"):
                if left["heads"] % left["kv_heads"]:
                    faults.append("%s.mixer.left: heads (%d) is not a multiple of kv_heads (%d)"
                                  % (at, left["heads"], left["kv_heads"]))
                if not isinstance(left.get("scale"), (int, float)) or isinstance(left.get("scale"), bool):
                    faults.append("%s.mixer.left.scale must be a number, got %r" % (at, left.get("scale")))
                mask = left.get("mask") or {}
                for k in ("size", "keep_first"):
                    v = mask.get(k, 0)
                    if not isinstance(v, int) or isinstance(v, bool) or v < 0:
                        faults.append("%s.mixer.left.mask.%s must be an integer >= 0, got %r" % (at, k, v))
            if positive(at + ".mixer.right", right, "heads", "dim", "vdim"):
                decay = right.get("decay")
                if not isinstance(decay, list) or len(decay) != right["heads"] or \
                        not all(isinstance(d, (int, float)) and not isinstance(d, bool) for d in decay):
                    faults.append("%s.mixer.right.decay must list one number per head" % at)
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
                faults.append("%s.mlp.kind %r is not one of ['dense', 'moe']" % (at, mlp.get("kind") if isinstance(mlp, dict) else mlp))
            elif mlp["kind"] == "dense":
                positive(at + ".mlp", mlp, "ff")
            else:
                positive(at + ".mlp.expert", mlp.get("expert"), "ff")
                if positive(at + ".mlp.router", mlp.get("router"), "experts", "top") and \
                        mlp["router"]["top"] > mlp["router"]["experts"]:
                    faults.append("%s.mlp.router: top (%d) exceeds experts (%d)" % (at, mlp["router"]["top"], mlp["router"]["experts"]))
                if mlp.get("shared") is not None:
                    positive(at + ".mlp.shared", mlp["shared"], "ff")
        if faults:
            raise ConfigError("Dobepel configuration: " + "; ".join(faults))


@dataclass(frozen=True)
class BuvuzenConfig(ModelConfig):
    """Buvuzen: a decoder whose config.json is nested and lists its layers one by one.

        architecture   "Buvuzen"
        vocab, width, norm.eps, embedding.scale, logit_scale
        layers[i]      type ("attention"),
                       mixer (heads, kv_heads, dim, vdim, scale, mask.size),
                       mlp: null | kind "moe" (expert.ff, router.experts, router.identity, router.top, router.scale,
                       router.groups.count, router.groups.keep, shared.ff or no shared),
                       weights_of: j (optional): the layer has no tensors of its own and runs with layer j's

    Every size and constant is read from there; the layers may differ from one another.  Absent optional keys mean
    "not there": no window (mask), multipliers of 1, no identity experts, one group, no shared expert."""

    architecture: ClassVar[str] = "Buvuzen"
    model_type: ClassVar[str] = "buvuzen"
    LAYER_TYPES: ClassVar[Tuple[str, ...]] = ("attention",)

    vocab: int = _field(int)
    width: int = _field(int)
    norm_eps: float = _field(float)
    embedding_scale: float = _field(float, default=1.0)
    logit_scale: float = _field(float, default=1.0)
    layers: Tuple[Dict[str, Any], ...] = _field(tuple, default=())

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "BuvuzenConfig":
        faults: list = []

        def get(d, path, kind, default=dataclasses.MISSING):
            cur = d
            for key in path.split("."):
                if not isinstance(cur, dict) or cur.get(key) is None:
                    if default is dataclasses.MISSING:
                        faults.append("missing key %r" % path)
                    return None if default is dataclasses.MISSING else default
                cur = cur[key]
            return _typed(path, cur, kind, faults)

        values = dict(vocab=get(raw, "vocab", int), width=get(raw, "width", int), norm_eps=get(raw, "norm.eps", float),
                      embedding_scale=get(raw, "embedding.scale", float, 1.0), logit_scale=get(raw, "logit_scale", float, 1.0))
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            faults.append("key 'layers': expected a list of layers")
            layers = []
        if faults:
            raise ConfigError("config.json for %s: %s" % (cls.__name__, "; ".join(faults)))
        cfg = cls(layers=tuple(json.loads(json.dumps(layer)) for layer in layers), **values)
        cfg.validate()
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "embedding": {"scale": self.embedding_scale},
                "layers": json.loads(json.dumps(list(self.layers))), "logit_scale": self.logit_scale,
                "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}

    def weights_layer(self, i: int) -> int:
        """The layer whose tensors layer i runs with: itself, or the end of its `weights_of` chain."""
        seen = set()
        while self.layers[i].get("weights_of") is not None:
            seen.add(i)
            i = int(self.layers[i]["weights_of"])
            if i in seen:
                raise ConfigError("Buvuzen configuration: the layers' weights_of form a circle at layer %d" % i)
        return i

    def validate(self) -> None:
        faults = []

        def positive(where, d, *keys):
            for k in keys:
                v = d.get(k) if isinstance(d, dict) else None
                if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
                    faults.append("%s.%s must be a positive integer, got %r" % (where, k, v))
                    return False
            return True

        def count(where, d, key, default, least=0):
            v = d.get(key, default) if isinstance(d, dict) else default
            if v is None:
                v = default
            if not isinstance(v, int) or isinstance(v, bool) or v < least:
                faults.append("%s.%s must be an integer >= %d, got %r" % (where, key, least, v))
                return default
            return v

        def number(where, d, key):
            v = d.get(key, 1.0) if isinstance(d, dict) else None
            if not isinstance(v, (int, float)) or isinstance(v, bool):
                faults.append("%s.%s must be a number, got %r" % (where, key, v))

        for name in ("vocab", "width"):
            if getattr(self, name) <= 0:
                faults.append("%s must be positive, got %d" % (name, getattr(self, name)))
        if not self.norm_eps > 0:
            faults.append("norm.eps must be positive, got %r" % self.norm_eps)
        n = len(self.layers)
        for i, layer in enumerate(self.layers):
            at = "layers[%d]" % i
            if not isinstance(layer, dict) or layer.get("type") not in self.LAYER_TYPES:
                faults.append("%s.type %r is not one of %s" % (at, layer.get("type") if isinstance(layer, dict) else layer,
                                                               list(self.LAYER_TYPES)))
                continue
            j = layer.get("weights_of")
            if j is not None and (not isinstance(j, int) or isinstance(j, bool) or not 0 <= j < n or j == i):
                faults.append("%s.weights_of must name another layer, got %r" % (at, j))
            mixer = layer.get("mixer")
            if positive(at + ".mixer", mixer, "heads", "kv_heads", "dim", "vdim"):
                if mixer["heads"] % mixer["kv_heads"]:
                    faults.append("%s.mixer: heads (%d) is not a multiple of kv_heads (%d)" % (at, mixer["heads"], mixer["kv_heads"]))
                if "scale" not in mixer:
                    faults.append("%s.mixer.scale is missing" % at)
                number(at + ".mixer", mixer, "scale")
                count(at + ".mixer.mask", mixer.get("mask") or {}, "size", 0)
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if not isinstance(mlp, dict) or mlp.get("kind") != "moe":
                faults.append("%s.mlp.kind %r is not 'moe'" % (at, mlp.get("kind") if isinstance(mlp, dict) else mlp))
                continue
            positive(at + ".mlp.expert", mlp.get("expert"), "ff")
            router = mlp.get("router")
            if positive(at + ".mlp.router", router, "experts", "top"):
                outputs = router["experts"] + count(at + ".mlp.router", router, "identity", 0)
                groups = router.get("groups") or {}
                g, keep = count(at + ".mlp.router.groups", groups, "count", 1, 1), count(at + ".mlp.router.groups", groups, "keep", 1, 1)
                number(at + ".mlp.router", router, "scale")
                if outputs % g or keep > g:
                    faults.append("%s.mlp.router: %d outputs do not form %d equal groups of which %d are kept" % (at, outputs, g, keep))
                elif router["top"] > keep * (outputs // g):
                    faults.append("%s.mlp.router: top (%d) exceeds the outputs of the kept groups (%d)"
                                  % (at, router["top"], keep * (outputs // g)))
            if mlp.get("shared") is not None:
                positive(at + ".mlp.shared", mlp["shared"], "ff")
        if faults:
            raise ConfigError("Buvuzen configuration: " + "; ".join(faults))
        for i in range(n):
            self.weights_layer(i)


@dataclass(frozen=True)
class KapuvikConfig(ModelConfig):
    """Kapuvik: a decoder whose config.json is nested and lists its layers one by one.

        architecture   "Kapuvik"
        vocab, width, norm.eps, embedding.scale, logit_softcap
        loop           start, stop, times: layers start .. stop-1 run `times` times in a row (optional)
        layers[i]      type "parallel":          mixer.left (heads, kv_heads, dim, vdim, scale, softcap, rot.base, rot.dims),
                                                 mixer.right (heads, dim, vdim, decay per head, rot.base, rot.dims),
                                                 mixer.left_scale, mixer.right_scale
                       type "latent_attention":  mixer (heads, dim, rot_dim, vdim, kv_rank, scale, rot.base)
                       type "gla":               mixer (heads, dim, vdim, tau; optional rank: the middle width of the decay's
                                                 projection, otherwise read off the weight file)
                       mlp: null | kind "dense" (ff, limit)

    Every size and constant is read from there; the layers may differ from one another.  Absent optional keys mean
    "not there": no loop, no rotation, no cap, multipliers of 1."""

    architecture: ClassVar[str] = "Kapuvik"
    model_type: ClassVar[str] = "kapuvik"
    LAYER_TYPES: ClassVar[Tuple[str, ...]] = ("parallel", "latent_attention", "gla")

    vocab: int = _field(int)
    width: int = _field(int)
    norm_eps: float = _field(float)
    embedding_scale: float = _field(float, default=1.0)
    logit_softcap: float = _field(float, default=0.0)
    loop_start: int = _field(int, default=0)
    loop_stop: int = _field(int, default=0)
    loop_times: int = _field(int, default=1)
    layers: Tuple[Dict[str, Any], ...] = _field(tuple, default=())

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "KapuvikConfig":
        faults: list = []

        def get(d, path, kind, default=dataclasses.MISSING):
            cur = d
            for key in path.split("."):
                if not isinstance(cur, dict) or cur.get(key) is None:
                    if default is dataclasses.MISSING:
                        faults.append("missing key %r" % path)
                    return None if default is dataclasses.MISSING else default
                cur = cur[key]
            return _typed(path, cur, kind, faults)

        values = dict(vocab=get(raw, "vocab", int), width=get(raw, "width", int), norm_eps=get(raw, "norm.eps", float),
                      embedding_scale=get(raw, "embedding.scale", float, 1.0), logit_softcap=get(raw, "logit_softcap", float, 0.0))
        if raw.get("loop") is not None:
            values.update(loop_start=get(raw, "loop.start", int), loop_stop=get(raw, "loop.stop", int),
                          loop_times=get(raw, "loop.times", int))
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            faults.append("key 'layers': expected a list of layers")
            layers = []
        if faults:
            raise ConfigError("config.json for %s: %s" % (cls.__name__, "; ".join(faults)))
        cfg = cls(layers=tuple(json.loads(json.dumps(layer)) for layer in layers), **values)
        cfg.validate()
        return cfg

    @property
    def looped(self) -> bool:
        return self.loop_stop > self.loop_start

    def to_dict(self) -> Dict[str, Any]:
        out = {"architecture": self.architecture, "embedding": {"scale": self.embedding_scale},
               "layers": json.loads(json.dumps(list(self.layers))), "logit_softcap": self.logit_softcap,
               "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}
        if self.looped:
            out["loop"] = {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}
        return out

    def validate(self) -> None:
        faults = []

        def positive(where, d, *keys):
            ok = True
            for k in keys:
                v = d.get(k) if isinstance(d, dict) else None
                if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
                    faults.append("%s.%s must be a positive integer, got %r" % (where, k, v))
                    ok = False
            return ok

        def number(where, d, key, least=None, required=True):
            v = d.get(key) if isinstance(d, dict) else None
            if v is None and not required:
                return True
            if not isinstance(v, (int, float)) or isinstance(v, bool) or (least is not None and not v > least):
                faults.append("%s.%s must be a number%s, got %r" % (where, key, "" if least is None else " above %g" % least, v))
                return False
            return True

        def rotation(where, d, dim):
            rot = d.get("rot") if isinstance(d, dict) else None
            if rot is None:
                return
            if positive(where + ".rot", rot, "dims") and number(where + ".rot", rot, "base", 0):
                if rot["dims"] % 2 or rot["dims"] > dim:
                    faults.append("%s.rot.dims (%d) must be even and within the head's %d channels" % (where, rot["dims"], dim))

        for name in ("vocab", "width"):
            if getattr(self, name) <= 0:
                faults.append("%s must be positive, got %d" % (name, getattr(self, name)))
        if not self.norm_eps > 0:
            faults.append("norm.eps must be positive, got %r" % self.norm_eps)
        if self.logit_softcap < 0:
            faults.append("logit_softcap must not be negative, got %r" % self.logit_softcap)
        n = len(self.layers)
        if self.loop_stop or self.loop_start or self.loop_times != 1:
            if not (0 <= self.loop_start < self.loop_stop <= n) or self.loop_times < 1:
                faults.append("loop: start %d, stop %d, times %d do not name a run of the %d layers at least once"
                              % (self.loop_start, self.loop_stop, self.loop_times, n))
        for i, layer in enumerate(self.layers):
            at = "layers[%d]" % i
            if not isinstance(layer, dict) or layer.get("type") not in self.LAYER_TYPES:
                faults.append("%s.type %r is not one of %s" % (at, layer.get("type") if isinstance(layer, dict) else layer,
                                                               list(self.LAYER_TYPES)))
                continue
            m, kind = layer.get("mixer"), layer["type"]
            if kind == "parallel":
                left, right = (m or {}).get("left"), (m or {}).get("right")
                if positive(at + ".mixer.left", left, "heads", "kv_heads", "dim", "vdim"):
                    if left["heads"] % left["kv_heads"]:
                        faults.append("%s.mixer.left: heads (%d) is not a multiple of kv_heads (%d)" % (at, left["heads"], left["kv_heads"]))
                    number(at + ".mixer.left", left, "scale")
                    number(at + ".mixer.left", left, "softcap", 0, required=False)
                    rotation(at + ".mixer.left", left, left["dim"])
                if positive(at + ".mixer.right", right, "heads", "dim", "vdim"):
                    decay = right.get("decay")
                    if not isinstance(decay, list) or len(decay) != right["heads"] or \
                            not all(isinstance(d, (int, float)) and not isinstance(d, bool) for d in decay):
                        faults.append("%s.mixer.right.decay must list one number per head" % at)
                    rotation(at + ".mixer.right", right, right["dim"])
                number(at + ".mixer", m, "left_scale", required=False)
                number(at + ".mixer", m, "right_scale", required=False)
            elif kind == "latent_attention":
                if positive(at + ".mixer", m, "heads", "dim", "rot_dim", "vdim", "kv_rank"):
                    number(at + ".mixer", m, "scale")
                    if m["rot_dim"] % 2:
                        faults.append("%s.mixer.rot_dim (%d) must be even" % (at, m["rot_dim"]))
                    if not isinstance(m.get("rot"), dict) or not number(at + ".mixer.rot", m.get("rot"), "base", 0):
                        pass
                    elif m["rot"].get("dims", m["rot_dim"]) != m["rot_dim"]:
                        faults.append("%s.mixer.rot.dims must equal rot_dim" % at)
            else:
                if positive(at + ".mixer", m, "heads", "dim", "vdim"):
                    number(at + ".mixer", m, "tau", 0)
                    if m.get("rank") is not None:
                        positive(at + ".mixer", m, "rank")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                faults.append("%s.mlp.kind %r is not 'dense'" % (at, mlp.get("kind") if isinstance(mlp, dict) else mlp))
            elif positive(at + ".mlp", mlp, "ff"):
                number(at + ".mlp", mlp, "limit", 0)
        if faults:
            raise ConfigError("Kapuvik configuration: " + "; ".join(faults))


@dataclass(frozen=True)
class FovenexConfig(ModelConfig):
    """Fovenex: a decoder whose config.json is nested and lists its layers one by one.

        architecture   "Fovenex"
        vocab, width, norm.eps
        residual_mult  multiplier of every sublayer's output on its way into the stream (absent: 1)
        streams        copies of the stream with learned mixing (absent or 0: one stream, no mixing tensors)
        layers[i]      type "attention":         mixer (heads, kv_heads, dim, vdim, scale, diff, rot.base, rot.dims,
                                                 rot.scaling.{factor, original, fast, slow} (optional), mask.size (optional))
                       type "latent_attention":  mixer (heads, dim, rot_dim, vdim, kv_rank, scale, rot.base,
                                                 q_rank (optional: queries through a latent of their own),
                                                 mask.size (optional window), kv_from (optional: the layer whose cached
                                                 rows it reads instead of making its own))
                       mlp: null | kind "dense" (ff)

    Every size and constant is read from there; the layers may differ from one another."""

    architecture: ClassVar[str] = "Fovenex"
    model_type: ClassVar[str] = "fovenex"
    LAYER_TYPES: ClassVar[Tuple[str, ...]] = ("attention", "latent_attention")

    vocab: int = _field(int)
    width: int = _field(int)
    norm_eps: float = _field(float)
    residual_mult: float = _field(float, default=1.0)
    streams: int = _field(int, default=0)
    layers: Tuple[Dict[str, Any], ...] = _field(tuple, default=())

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "FovenexConfig":
        faults: list = []

        def get(d, path, kind, default=dataclasses.MISSING):
            cur = d
            for key in path.split("."):
                if not isinstance(cur, dict) or cur.get(key) is None:
                    if default is dataclasses.MISSING:
                        faults.append("missing key %r" % path)
                    return None if default is dataclasses.MISSING else default
                cur = cur[key]
            return _typed(path, cur, kind, faults)

        values = dict(vocab=get(raw, "vocab", int), width=get(raw, "width", int), norm_eps=get(raw, "norm.eps", float),
                      residual_mult=get(raw, "residual_mult", float, 1.0), streams=get(raw, "streams", int, 0))
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            faults.append("key 'layers': expected a list of layers")
            layers = []
        if faults:
            raise ConfigError("config.json for %s: %s" % (cls.__name__, "; ".join(faults)))
        cfg = cls(layers=tuple(json.loads(json.dumps(layer)) for layer in layers), **values)
        cfg.validate()
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        out = {"architecture": self.architecture, "layers": json.loads(json.dumps(list(self.layers))),
               "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult, "vocab": self.vocab, "width": self.width}
        if self.streams:
            out["streams"] = self.streams
        return out

    @staticmethod
    def window_of(mixer: Dict[str, Any]) -> int:
        mask = mixer.get("mask")
        return int(mask.get("size") or 0) if isinstance(mask, dict) else 0

    def rows_source(self, i: int) -> Optional[int]:
        """The layer whose cached latent rows layer i reads, or None if it keeps its own (or is no latent layer)."""
        m = self.layers[i].get("mixer") or {}
        return m.get("kv_from") if self.layers[i].get("type") == "latent_attention" else None

    def validate(self) -> None:
        faults = []

        def positive(where, d, *keys):
            ok = True
            for k in keys:
                v = d.get(k) if isinstance(d, dict) else None
                if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
                    faults.append("%s.%s must be a positive integer, got %r" % (where, k, v))
                    ok = False
            return ok

        def number(where, d, key, least=None):
            v = d.get(key) if isinstance(d, dict) else None
            if not isinstance(v, (int, float)) or isinstance(v, bool) or (least is not None and not v > least):
                faults.append("%s.%s must be a number%s, got %r" % (where, key, "" if least is None else " above %g" % least, v))
                return False
            return True

        def window(where, m):
            mask = m.get("mask")
            if mask is not None and (not isinstance(mask, dict) or not positive(where + ".mask", mask, "size")):
                if not isinstance(mask, dict):
                    faults.append("%s.mask must hold a size, got %r" % (where, mask))

        for name in ("vocab", "width"):
            if getattr(self, name) <= 0:
                faults.append("%s must be positive, got %d" % (name, getattr(self, name)))
        if not self.norm_eps > 0:
            faults.append("norm.eps must be positive, got %r" % self.norm_eps)
        if not 0 <= self.streams <= 16:
            faults.append("streams must lie in 0 .. 16, got %r" % self.streams)
        for i, layer in enumerate(self.layers):
            at = "layers[%d]" % i
            if not isinstance(layer, dict) or layer.get("type") not in self.LAYER_TYPES:
                faults.append("%s.type %r is not one of %s" % (at, layer.get("type") if isinstance(layer, dict) else layer,
                                                               list(self.LAYER_TYPES)))
                continue
            m, kind = layer.get("mixer"), layer["type"]
            where = at + ".mixer"
            if kind == "attention":
                if positive(where, m, "heads", "kv_heads", "dim", "vdim"):
                    if m["heads"] % m["kv_heads"]:
                        faults.append("%s: heads (%d) is not a multiple of kv_heads (%d)" % (where, m["heads"], m["kv_heads"]))
                    number(where, m, "scale")
                    if number(where, m, "diff") and not 0 <= m["diff"] < 1:
                        faults.append("%s.diff must lie in [0, 1), got %r" % (where, m["diff"]))
                    rot = m.get("rot")
                    if rot is not None:
                        if not isinstance(rot, dict) or not positive(where + ".rot", rot, "dims") or not number(where + ".rot", rot, "base", 1):
                            pass
                        elif rot["dims"] % 2 or rot["dims"] > m["dim"]:
                            faults.append("%s.rot.dims (%d) must be even and within the head's %d channels" % (where, rot["dims"], m["dim"]))
                        sc = rot.get("scaling") if isinstance(rot, dict) else None
                        if sc is not None:
                            for key in ("factor", "original", "fast", "slow"):
                                number(where + ".rot.scaling", sc, key, 0)
                    window(where, m)
            else:
                if positive(where, m, "heads", "dim", "rot_dim", "vdim", "kv_rank"):
                    number(where, m, "scale")
                    if m["rot_dim"] % 2:
                        faults.append("%s.rot_dim (%d) must be even" % (where, m["rot_dim"]))
                    if not isinstance(m.get("rot"), dict) or not number(where + ".rot", m.get("rot"), "base", 1):
                        pass
                    elif m["rot"].get("dims", m["rot_dim"]) != m["rot_dim"]:
                        faults.append("%s.rot.dims must equal rot_dim" % where)
                    if m.get("q_rank") is not None:
                        positive(where, m, "q_rank")
                    window(where, m)
                    j = m.get("kv_from")
                    if j is not None:
                        src = self.layers[j] if isinstance(j, int) and not isinstance(j, bool) and 0 <= j < i else None
                        sm = src.get("mixer") if isinstance(src, dict) and src.get("type") == "latent_attention" else None
                        if not isinstance(sm, dict) or sm.get("kv_from") is not None:
                            faults.append("%s.kv_from %r must name an earlier latent layer that keeps rows of its own" % (where, j))
                        elif (sm.get("kv_rank"), sm.get("rot_dim"), (sm.get("rot") or {}).get("base")) != \
                                (m["kv_rank"], m["rot_dim"], (m.get("rot") or {}).get("base")):
                            faults.append("%s.kv_from %d: kv_rank, rot_dim and rotation must equal that layer's" % (where, j))
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                faults.append("%s.mlp.kind %r is not 'dense'" % (at, mlp.get("kind") if isinstance(mlp, dict) else mlp))
            else:
                positive(at + ".mlp", mlp, "ff")
        if faults:
            raise ConfigError("Fovenex configuration: " + "; ".join(faults))
