"""Typed configuration of the Daferax decoder, read from its config.json keys.

A Daferax model is a stack of layers that config.json lists one by one (``layers[i]``: ``type``
names the mixer, ``mixer`` holds its sizes and constants, ``mlp`` the feed-forward or null).
Layers may differ in every size and in their order.  Only what a sublayer RETURNS is normed (layer
norm with weight and bias); the sublayers read the residual stream itself:

    x <- x + norm1(mixer(x));   x <- x + norm2(ff(x))

Mixers: ``attention`` -- grouped-query attention with RMS-normed query and key heads, rotation of
neighbouring pairs on the first ``rot.dims`` elements, keys of ``dim`` and values of ``vdim``
elements, the values optionally mixed with those of the first value-mixing layer (``v_mix``), one
sigmoid gate a head; ``latent_attention`` -- keys and values of all heads expanded from a normed
latent of ``kv_rank`` elements plus a rotated key part of ``rot_dim`` elements shared by the heads
(YaRN-scaled frequencies from ``rot.scaling``), a sliding window ``mask.size``, a sigmoid gate per
element.  Feed-forward ``moe``: softmax router with group-limited choice of ``top`` experts,
weights = scores x ``router.scale`` (not renormalised), plus a shared expert; ``dense``: one gated
feed-forward of ``ff`` elements.  The output is the final layer norm and the embedding table again.

Optional keys fall back to "the mechanism is absent": no ``mask`` is causal attention over every
earlier key, no ``rot.scaling`` plain frequencies, no ``groups`` one group, no ``shared`` no shared
expert, no ``kv_heads`` one key head per query head.  Any other key is an error: a key that is not
read would be a mechanism that is not computed.

Tensor names: ``embed``, ``final.norm`` (+ ``.b``), and under ``l<i>.``: ``norm1``, ``norm2``
(+ ``.b``); ``mix.{q,k,v,o,g}``, ``mix.{q,k}.norm``, ``mix.vmix``; ``mix.{q,dkv,uk,uv,g,o}``,
``mix.dkv.norm``; ``mlp.router``, ``mlp.e<j>.{gate,up,down}``, ``mlp.shared.{gate,up,down}``;
``mlp.{gate,up,down}``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .qwen2 import ConfigError
from .specs import (BlockSpec, GatedMLPSpec, LatentAttentionSpec, LayerNormSpec, LayerRun, ModelSpec,
                    NoPositionSpec, NormedAttentionSpec, PairRotarySpec, RoutedExpertsSpec)

_MAX_POSITIONS = 1 << 20          # nothing in the model bounds the positions

_MIXER_KEYS = {
    "attention": ("heads", "kv_heads", "dim", "vdim", "rot", "scale", "v_mix", "mask"),
    "latent_attention": ("heads", "dim", "rot_dim", "vdim", "kv_rank", "rot", "scale", "mask"),
}


def _only(d: Dict[str, Any], allowed, where: str, problems) -> None:
    extra = sorted(k for k in d if k not in allowed)
    if extra:
        problems.append(f"{where}: unknown key(s) " + ", ".join(repr(k) for k in extra))


def _rotary(rot: Optional[dict], where: str, p) -> PartSpecLike:
    if not rot:
        return NoPositionSpec()
    _only(rot, ("base", "dims", "scaling"), where, p)
    sc = rot.get("scaling")
    kw = {}
    if sc:
        _only(sc, ("factor", "original", "fast", "slow"), where + ".scaling", p)
        kw = dict(yarn_factor=float(sc["factor"]), yarn_original=float(sc["original"]),
                  yarn_fast=float(sc["fast"]), yarn_slow=float(sc["slow"]))
    return PairRotarySpec(dims=int(rot["dims"]), theta=float(rot["base"]), **kw)


PartSpecLike = object


@dataclass(frozen=True)
class DaferaxConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[dict, ...]               # the entries of config.json's ``layers``, checked
    eos_token_ids: Tuple[int, ...] = ()

    architecture = "Daferax"
    model_type = "daferax"

    # ------------------------------------------------------------ parsing
    @classmethod
    def from_dict(cls, cfg: Dict[str, Any]) -> "DaferaxConfig":
        p = []
        _only(cfg, ("architecture", "architectures", "model_type", "vocab", "width", "norm", "layers",
                    "eos_token_id"), "config", p)
        for key in ("vocab", "width", "norm", "layers"):
            if key not in cfg:
                p.append(f"missing key '{key}'")
        if p:
            raise ConfigError("invalid Daferax config: " + "; ".join(p))
        _only(cfg["norm"], ("eps",), "norm", p)
        eos = cfg.get("eos_token_id", ())
        eos_ids = tuple(int(e) for e in eos) if isinstance(eos, (list, tuple)) else (int(eos),)
        out = cls(vocab=int(cfg["vocab"]), width=int(cfg["width"]), norm_eps=float(cfg["norm"]["eps"]),
                  layers=tuple(_freeze(layer) for layer in cfg["layers"]), eos_token_ids=eos_ids)
        out.to_model_spec()                # every per-layer check happens there
        return out

    def to_dict(self) -> Dict[str, Any]:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
             "norm": {"eps": self.norm_eps}, "layers": [_thaw(layer) for layer in self.layers]}
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    # ----------------------------------------------- the model as plain data
    def _mixer(self, i: int, kind: str, m: dict, first_mix: Optional[int], p):
        where = f"layers[{i}].mixer"
        _only(m, _MIXER_KEYS[kind], where, p)
        mask = m.get("mask") or {}
        _only(mask, ("size",), where + ".mask", p)
        window = int(mask["size"]) if "size" in mask else None
        if window is not None and window < 1:
            p.append(f"{where}.mask.size must be positive")
        rot = _rotary(m.get("rot"), where + ".rot", p)
        if kind == "attention":
            heads, dim = int(m["heads"]), int(m["dim"])
            kv_heads, vdim = int(m.get("kv_heads", heads)), int(m.get("vdim", dim))
            if min(heads, kv_heads, dim, vdim) <= 0 or heads % kv_heads:
                p.append(f"{where}: heads must be a positive multiple of kv_heads; dim, vdim positive")
            if isinstance(rot, PairRotarySpec) and (rot.dims % 2 or not 0 < rot.dims <= dim):
                p.append(f"{where}.rot.dims must be even and at most dim")
            mix = None
            if m.get("v_mix"):
                mix = "source" if first_mix is None or first_mix == i else "mix"
            return NormedAttentionSpec(
                hidden_size=self.width, num_heads=heads, num_kv_heads=kv_heads, head_dim=dim,
                value_dim=vdim, window=window, scale=float(m["scale"]), qk_norm=True,
                qk_norm_eps=self.norm_eps, position=rot, value_mix=mix, head_gate=True)
        heads, dim, rope = int(m["heads"]), int(m["dim"]), int(m["rot_dim"])
        vdim, rank = int(m["vdim"]), int(m["kv_rank"])
        if min(heads, dim, rope, vdim, rank) <= 0 or rope % 2:
            p.append(f"{where}: heads, dim, vdim, kv_rank must be positive, rot_dim positive and even")
        if isinstance(rot, PairRotarySpec) and rot.dims != rope:
            p.append(f"{where}: rot.dims ({rot.dims}) must equal rot_dim ({rope})")
        return LatentAttentionSpec(
            hidden_size=self.width, num_heads=heads, head_dim=dim, rope_dim=rope, value_dim=vdim,
            kv_rank=rank, window=window, scale=float(m["scale"]), latent_norm_eps=self.norm_eps,
            position=rot, element_gate=True)

    def _feed_forward(self, i: int, mlp: dict, p):
        where = f"layers[{i}].mlp"
        kind = mlp.get("kind")
        if kind == "dense":
            _only(mlp, ("kind", "ff"), where, p)
            return GatedMLPSpec(hidden_size=self.width, intermediate_size=int(mlp["ff"]), gate_name="gate",
                                up_name="up", down_name="down", weight_suffix="")
        if kind != "moe":
            p.append(f"{where}: kind {kind!r} is not known (moe, dense)")
            return None
        _only(mlp, ("kind", "expert", "router", "shared"), where, p)
        r = mlp.get("router") or {}
        _only(r, ("experts", "groups", "scale", "top"), where + ".router", p)
        _only(mlp.get("expert") or {}, ("ff",), where + ".expert", p)
        groups = r.get("groups") or {}
        _only(groups, ("count", "keep"), where + ".router.groups", p)
        experts, top = int(r["experts"]), int(r["top"])
        count, keep = int(groups.get("count", 1)), int(groups.get("keep", groups.get("count", 1)))
        if experts <= 0 or count <= 0 or experts % count or not 0 < keep <= count \
                or not 0 < top <= experts // count * keep:
            p.append(f"{where}.router: experts must split into groups.count equal groups, "
                     f"0 < keep <= count, and top experts must fit into the kept groups")
        shared = None
        if mlp.get("shared"):
            _only(mlp["shared"], ("ff",), where + ".shared", p)
            shared = GatedMLPSpec(hidden_size=self.width, intermediate_size=int(mlp["shared"]["ff"]),
                                  gate_name="gate", up_name="up", down_name="down", weight_suffix="")
        return RoutedExpertsSpec(
            hidden_size=self.width, num_experts=experts, top=top, expert_size=int(mlp["expert"]["ff"]),
            num_groups=count, keep_groups=keep, route_scale=float(r.get("scale", 1.0)),
            renormalize=False, shared=shared)

    def to_model_spec(self) -> ModelSpec:
        p = []
        if self.vocab <= 0 or self.width <= 0:
            p.append("vocab and width must be positive")
        if not self.layers:
            p.append("the model has no layers")
        norm = LayerNormSpec(dim=self.width, eps=self.norm_eps, weight_suffix="", bias_suffix=".b")
        entries = [_thaw(layer) for layer in self.layers]
        first_mix = next((i for i, e in enumerate(entries) if e.get("type") == "attention"
                          and (e.get("mixer") or {}).get("v_mix")), None)
        layers = []
        for i, entry in enumerate(entries):
            _only(entry, ("type", "mixer", "mlp"), f"layers[{i}]", p)
            kind = entry.get("type")
            if kind not in _MIXER_KEYS:
                p.append(f"layers[{i}]: mixer type {kind!r} is not known ({', '.join(_MIXER_KEYS)})")
                continue
            try:
                mixer = self._mixer(i, kind, entry.get("mixer") or {}, first_mix, p)
                ff = self._feed_forward(i, entry["mlp"], p) if entry.get("mlp") else None
            except (KeyError, TypeError, ValueError) as e:
                p.append(f"layers[{i}]: missing or malformed key {e}")
                continue
            layers.append(BlockSpec(
                kind="result_norm", mixer=mixer, feed_forward=ff, mixer_post_norm=norm,
                ff_post_norm=None if ff is None else norm, mixer_name="mix", feed_forward_name="mlp",
                mixer_post_norm_name="norm1", ff_post_norm_name="norm2"))
        if p:
            raise ConfigError("invalid Daferax config: " + "; ".join(p))
        mixes = [b.mixer for b in layers if getattr(b.mixer, "value_mix", None)]
        if len({(m.num_kv_heads, m.value_dim) for m in mixes}) > 1:
            raise ConfigError("invalid Daferax config: layers that mix values must agree in "
                              "kv_heads and vdim")
        return ModelSpec(
            architecture=self.architecture, hidden_size=self.width, vocab_size=self.vocab,
            layers=tuple(layers), run_order=tuple(LayerRun(i) for i in range(len(layers))),
            final_norm=norm, tie_word_embeddings=True, max_position_embeddings=_MAX_POSITIONS,
            eos_token_ids=self.eos_token_ids, embed_name="embed", lm_head_name="head",
            final_norm_prefix="final.norm", layer_prefix="l{}",
            # a layer without a feed-forward has no use for the second norm, and the first
            # value-mixing layer none for its mixing factor; a checkpoint may hold them all the same
            ignored_suffixes=(".norm2", ".norm2.b", ".mix.vmix"))


def _freeze(x):
    """Nested dicts and lists as hashable tuples (the config is a frozen dataclass)."""
    if isinstance(x, dict):
        return ("__dict__",) + tuple((k, _freeze(v)) for k, v in x.items())
    if isinstance(x, (list, tuple)):
        return ("__list__",) + tuple(_freeze(v) for v in x)
    return x


def _thaw(x):
    if isinstance(x, tuple) and x and x[0] == "__dict__":
        return {k: _thaw(v) for k, v in x[1:]}
    if isinstance(x, tuple) and x and x[0] == "__list__":
        return [_thaw(v) for v in x[1:]]
    return x
