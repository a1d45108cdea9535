"""Typed configuration of the Dezelorn decoder, read from its config.json keys.

A Dezelorn model is a stack of layers that config.json lists one by one: every entry of
``layers`` names its mixer (``type``), gives the mixer's sizes and constants (``mixer``) and
its feed-forward (``mlp``; null for a layer without one).  Layers may differ in every size.
A layer norms both what enters a sublayer and what leaves it, with Dynamic Tanh:

    x <- x + norm1b(mixer(norm1(x)));   x <- x + norm2b(ff(norm2(x)))

The ``attention`` mixer (``parts/conv_attention.py``) has no value projection and no
rotation: queries and keys pass a short causal convolution, the values are the keys, positions
enter through a query temperature, a log-distance bias and a sliding window, the heads'
softmax weights are mixed by a learned matrix and the result is gated.  The feed-forward is
the dense gated one with SiLU.  The embedding is scaled; the head is untied.

Keys read: ``architecture``, ``vocab``, ``width``, ``embedding.scale``, ``norm.eps`` (kept,
though Dynamic Tanh has no use for it), ``layers[i].type``, ``layers[i].mixer.{heads,
kv_heads, dim, vdim, conv, scale, mask.size, q_temp.coef, q_temp.every}``,
``layers[i].mlp.{kind, ff}``.  Anything else is an error: a key that is not read would be a
mechanism that is not computed.

Tensor names: ``embed``, ``head``, ``final.norm`` (+ ``.b``, ``.alpha``), and under ``l<i>.``:
``norm1 norm1b norm2 norm2b`` (each + ``.b``, ``.alpha``), ``mix.{q,k,g,o}``,
``mix.{q,k}.conv``, ``mix.{r1,r2,talk}``, ``mlp.{gate,up,down}``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .qwen2 import ConfigError
from .specs import (BlockSpec, ConvTalkAttentionSpec, DynamicTanhSpec, GatedMLPSpec, LayerRun,
                    ModelSpec)

# positions are not encoded in a table, so nothing in the model bounds them; the engine still
# wants a number to refuse absurd requests with
_MAX_POSITIONS = 1 << 20


def _only(d: Dict[str, Any], allowed, where: str, problems) -> None:
    extra = sorted(k for k in d if k not in allowed)
    if extra:
        problems.append(f"{where}: unknown key(s) " + ", ".join(repr(k) for k in extra))


@dataclass(frozen=True)
class DezelornMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    scale: float
    window: int
    q_temp_coef: float
    q_temp_every: int

    def to_dict(self) -> Dict[str, Any]:
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                "conv": self.conv, "scale": self.scale, "mask": {"size": self.window},
                "q_temp": {"coef": self.q_temp_coef, "every": self.q_temp_every}}


@dataclass(frozen=True)
class DezelornLayer:
    type: str
    mixer: DezelornMixer
    ff: Optional[int]                      # None: the layer has no feed-forward

    def to_dict(self) -> Dict[str, Any]:
        return {"type": self.type, "mixer": self.mixer.to_dict(),
                "mlp": None if self.ff is None else {"kind": "dense", "ff": self.ff}}


@dataclass(frozen=True)
class DezelornConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: Tuple[DezelornLayer, ...]
    eos_token_ids: Tuple[int, ...] = ()

    architecture = "Dezelorn"
    model_type = "dezelorn"

    # ------------------------------------------------------------ parsing
    @classmethod
    def from_dict(cls, cfg: Dict[str, Any]) -> "DezelornConfig":
        p = []
        _only(cfg, ("architecture", "architectures", "model_type", "vocab", "width", "embedding",
                    "norm", "layers", "eos_token_id"), "config", p)
        for key in ("vocab", "width", "embedding", "norm", "layers"):
            if key not in cfg:
                p.append(f"missing key '{key}'")
        if p:
            raise ConfigError("invalid Dezelorn config: " + "; ".join(p))
        _only(cfg["embedding"], ("scale",), "embedding", p)
        _only(cfg["norm"], ("eps",), "norm", p)
        layers = []
        for i, entry in enumerate(cfg["layers"]):
            where = f"layers[{i}]"
            _only(entry, ("type", "mixer", "mlp"), where, p)
            if entry.get("type") != "attention":
                p.append(f"{where}: mixer type {entry.get('type')!r} is not known (attention)")
                continue
            m = entry.get("mixer") or {}
            _only(m, ("heads", "kv_heads", "dim", "vdim", "conv", "scale", "mask", "q_temp"),
                  where + ".mixer", p)
            _only(m.get("mask") or {}, ("size",), where + ".mixer.mask", p)
            _only(m.get("q_temp") or {}, ("coef", "every"), where + ".mixer.q_temp", p)
            try:
                mixer = DezelornMixer(
                    heads=int(m["heads"]), kv_heads=int(m["kv_heads"]), dim=int(m["dim"]),
                    vdim=int(m.get("vdim", m["dim"])), conv=int(m["conv"]), scale=float(m["scale"]),
                    window=int(m["mask"]["size"]), q_temp_coef=float(m["q_temp"]["coef"]),
                    q_temp_every=int(m["q_temp"]["every"]))
            except (KeyError, TypeError) as e:
                p.append(f"{where}.mixer: missing or malformed key {e}")
                continue
            mlp = entry.get("mlp")
            ff = None
            if mlp is not None:
                _only(mlp, ("kind", "ff"), where + ".mlp", p)
                if mlp.get("kind") != "dense":
                    p.append(f"{where}.mlp: kind {mlp.get('kind')!r} is not known (dense)")
                    continue
                ff = int(mlp["ff"])
            layers.append(DezelornLayer("attention", mixer, ff))
        if p:
            raise ConfigError("invalid Dezelorn config: " + "; ".join(p))
        eos = cfg.get("eos_token_id", ())
        eos_ids = tuple(int(e) for e in eos) if isinstance(eos, (list, tuple)) else (int(eos),)
        out = cls(vocab=int(cfg["vocab"]), width=int(cfg["width"]),
                  embedding_scale=float(cfg["embedding"]["scale"]),
                  norm_eps=float(cfg["norm"].get("eps", 0.0)), layers=tuple(layers),
                  eos_token_ids=eos_ids)
        out.validate()
        return out

    def validate(self) -> None:
        p = []
        if self.vocab <= 0 or self.width <= 0:
            p.append("vocab and width must be positive")
        if not self.layers:
            p.append("the model has no layers")
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            where = f"layers[{i}].mixer"
            if min(m.heads, m.kv_heads, m.dim, m.conv, m.window, m.q_temp_every) <= 0:
                p.append(f"{where}: heads, kv_heads, dim, conv, mask.size and q_temp.every "
                         f"must be positive")
                continue
            if m.heads % m.kv_heads:
                p.append(f"{where}: heads ({m.heads}) is not a multiple of kv_heads ({m.kv_heads})")
            if m.vdim != m.dim:
                p.append(f"{where}: the values are the keys, so vdim ({m.vdim}) must equal dim ({m.dim})")
            if layer.ff is not None and layer.ff <= 0:
                p.append(f"layers[{i}].mlp.ff must be positive")
        if p:
            raise ConfigError("invalid Dezelorn config: " + "; ".join(p))

    def to_dict(self) -> Dict[str, Any]:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
             "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
             "layers": [layer.to_dict() for layer in self.layers]}
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    # ----------------------------------------------- the model as plain data
    def to_model_spec(self) -> ModelSpec:
        norm = DynamicTanhSpec(dim=self.width, weight_suffix="", bias_suffix=".b",
                               alpha_suffix=".alpha")
        layers = []
        for layer in self.layers:
            m = layer.mixer
            mixer = ConvTalkAttentionSpec(
                hidden_size=self.width, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim,
                window=m.window, scale=m.scale, conv_taps=m.conv, tied_values=True,
                q_temp_coef=m.q_temp_coef, q_temp_every=m.q_temp_every, distance_bias=True,
                talking_heads=True, output_gate=True)
            ff = None if layer.ff is None else GatedMLPSpec(
                hidden_size=self.width, intermediate_size=layer.ff, activation="silu",
                gate_name="gate", up_name="up", down_name="down", weight_suffix="")
            layers.append(BlockSpec(
                kind="sandwich_norm", mixer=mixer, feed_forward=ff, mixer_norm=norm,
                mixer_post_norm=norm, ff_norm=None if ff is None else norm,
                ff_post_norm=None if ff is None else norm,
                mixer_norm_name="norm1", mixer_post_norm_name="norm1b", mixer_name="mix",
                ff_norm_name="norm2", ff_post_norm_name="norm2b", feed_forward_name="mlp"))
        return ModelSpec(
            architecture=self.architecture, hidden_size=self.width, vocab_size=self.vocab,
            layers=tuple(layers), run_order=tuple(LayerRun(i) for i in range(len(layers))),
            final_norm=norm, tie_word_embeddings=False,
            max_position_embeddings=_MAX_POSITIONS, eos_token_ids=self.eos_token_ids,
            embed_name="embed", lm_head_name="head", final_norm_prefix="final.norm",
            layer_prefix="l{}", embedding_scale=self.embedding_scale,
            # a layer without a feed-forward has no use for the norms around one; a checkpoint that
            # stores them all the same is taken (they are declared, and so required, wherever used)
            ignored_suffixes=(".norm2", ".norm2.b", ".norm2.alpha", ".norm2b", ".norm2b.b", ".norm2b.alpha"))
