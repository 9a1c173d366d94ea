"""Pikurax: a decoder whose layers run two mixers side by side, norm before and after every sublayer, and
may pass over some of their layers several times with the embedding fed in again through a projection.

``config.json`` holds ``vocab``, ``width``, ``norm.eps``, ``embedding`` (``scale``; ``bigram`` = {``buckets``,
``mul_prev``, ``mul_cur``}: a second table indexed by a hash of the token and the one before it), an optional ``loop``
(``start``, ``stop``, ``times``), ``logit_scale``, ``logit_softcap`` and a list ``layers``; every entry gives ``type``
(which pair of mixers), ``mixer`` (``left`` and ``right``: their sizes and constants) and ``mlp`` (or null).

- ``parallel``: left, grouped-query softmax attention whose values are its keys as projected (no value matrix),
  with a rotation of the first ``rot.dims`` elements of a head and a mask in chunks of ``mask.size`` positions; right,
  a gated linear recurrent unit per channel behind a short causal convolution (``width`` channels, ``blocks`` parts
  for the gates' matrices, ``conv`` taps).
- ``parallel_2``: left, grouped-query softmax attention over every earlier key with biases on q, k, v, an RMS norm per
  head on q and k, a query temperature, scores capped with tanh (``softcap``), a bias 2^(-8 (h + 1) / heads) x
  distance taken off them, and a sink per head; right, retention: S <- decay_h S + k v^T per head with the fixed
  ``decay`` list, rotated q and k, the read-out divided by its root mean square per head, a silu gate.
Either way the layer adds half the sum of the two results, each RMS-normed over the width with a gain.

The feed-forward is a gated unit with the tanh form of gelu (``kind`` "dense"), or a mixture of silu-gated experts
(``kind`` "moe": ``router.experts``, ``router.top``, the weights a softmax over the chosen logits; ``expert.ff``; an
optional ``shared`` expert times the sigmoid of one more logit).  Norms are layer norms with a gain and no bias.
The head is the embedding table, its logits times ``logit_scale`` and then capped with tanh.  Layer i's tensors
start with ``l<i>.``: ``norm1``, ``norm1b``, ``mix.left.*``, ``mix.right.*``, ``norm2``, ``norm2b``, ``mlp.*``.
"""

from __future__ import annotations

import copy
from typing import Any, Mapping

from .registry import register_architecture
from .spec import ConfigError, LayerRun, LayerSpec, ModelSpec, PartSpec

MIXERS = ("parallel", "parallel_2")
DEFAULT_MAX_POSITIONS = 32768
UNIT_RATE = 8.0            # the factor in the recurrent unit's log a = -rate r softplus(lam)
SLOPE_EXPONENT = 8.0       # the distance bias's slope of head h: 2^(-exponent (h + 1) / heads)


def _positive(where: str, raw, *keys: str) -> None:
    if not isinstance(raw, Mapping):
        raise ConfigError(f"{where} is missing")
    for k in keys:
        if k not in raw:
            raise ConfigError(f"{where} lacks {k!r}")
        if not (isinstance(raw[k], int) and not isinstance(raw[k], bool) and raw[k] > 0):
            raise ConfigError(f"{where}: {k} must be a positive integer, got {raw[k]!r}")


def _number(where: str, raw, *keys: str) -> None:
    if not isinstance(raw, Mapping):
        raise ConfigError(f"{where} is missing")
    for k in keys:
        if not isinstance(raw.get(k), (int, float)) or isinstance(raw.get(k), bool):
            raise ConfigError(f"{where}: {k} must be a number, got {raw.get(k)!r}")


def _rotation(where: str, m: Mapping[str, Any]) -> None:
    rot = m.get("rot")
    _positive(where + ".rot", rot, "dims")
    _number(where + ".rot", rot, "base")
    if rot["dims"] % 2 or rot["dims"] > m["dim"] or not float(rot["base"]) > 0:
        raise ConfigError(f"{where}: rot.dims must be even and at most dim, rot.base positive")


@register_architecture("Pikurax")
class PikuraxConfig:
    def __init__(self, raw: Mapping[str, Any]):
        self.raw = copy.deepcopy(dict(raw))
        self.validate()

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "PikuraxConfig":
        return cls(raw)

    def to_dict(self) -> dict[str, Any]:
        return copy.deepcopy(self.raw)

    # -- reading ------------------------------------------------------------
    @property
    def width(self) -> int:
        return int(self.raw["width"])

    @property
    def vocab(self) -> int:
        return int(self.raw["vocab"])

    @property
    def eps(self) -> float:
        return float(self.raw["norm"]["eps"])

    @property
    def layers(self) -> list[dict]:
        return self.raw["layers"]

    def validate(self) -> None:
        r = self.raw
        _positive("config.json", r, "vocab", "width")
        norm = r.get("norm")
        if not isinstance(norm, Mapping) or "eps" not in norm or not float(norm["eps"]) > 0:
            raise ConfigError("config.json: norm.eps must be a positive number")
        emb = r.get("embedding") or {}
        if "scale" in emb:
            _number("embedding", emb, "scale")
        if emb.get("bigram") is not None:
            _positive("embedding.bigram", emb["bigram"], "buckets", "mul_prev", "mul_cur")
        for key in ("logit_scale", "logit_softcap"):
            if r.get(key) is not None:
                _number("config.json", r, key)
        if not isinstance(r.get("layers"), list) or not r["layers"]:
            raise ConfigError("config.json: layers must be a list with at least one layer")
        loop = r.get("loop")
        if loop is not None:
            _positive("loop", loop, "stop", "times")
            if not (isinstance(loop.get("start"), int) and 0 <= loop["start"] < loop["stop"] <= len(r["layers"])):
                raise ConfigError("loop: 0 <= start < stop <= number of layers must hold")
        for i, layer in enumerate(r["layers"]):
            where = f"layers[{i}]"
            kind = layer.get("type") if isinstance(layer, Mapping) else None
            if kind not in MIXERS:
                raise ConfigError(f"{where}: type {kind!r} is not one of {MIXERS}")
            m = layer.get("mixer")
            if not isinstance(m, Mapping) or not isinstance(m.get("left"), Mapping) or not isinstance(m.get("right"), Mapping):
                raise ConfigError(f"{where}: the mixer needs 'left' and 'right'")
            left, right = m["left"], m["right"]
            _positive(where + ".left", left, "heads", "dim", "vdim")
            if "kv_heads" in left:
                _positive(where + ".left", left, "kv_heads")
            _number(where + ".left", left, "scale")
            if left["heads"] % left.get("kv_heads", left["heads"]):
                raise ConfigError(f"{where}.left: heads must be a multiple of kv_heads")
            if kind == "parallel":
                if left["vdim"] != left["dim"]:
                    raise ConfigError(f"{where}.left: the values are the keys, so vdim must equal dim")
                _rotation(where + ".left", left)
                _positive(where + ".left.mask", left.get("mask"), "size")
                _positive(where + ".right", right, "width", "blocks", "conv")
                if right["width"] % right["blocks"]:
                    raise ConfigError(f"{where}.right: blocks must divide width")
            else:
                temp = left.get("q_temp")
                if temp is not None:
                    _positive(where + ".left.q_temp", temp, "every")
                    _number(where + ".left.q_temp", temp, "coef")
                if left.get("softcap") is not None:
                    _number(where + ".left", left, "softcap")
                _positive(where + ".right", right, "heads", "dim", "vdim")
                _rotation(where + ".right", right)
                decay = right.get("decay")
                if not isinstance(decay, list) or len(decay) != right["heads"] or \
                        not all(isinstance(d, (int, float)) and 0 < d <= 1 for d in decay):
                    raise ConfigError(f"{where}.right: decay must list one number in (0, 1] per head")
            f = layer.get("mlp")
            if f is not None:
                kind_f = f.get("kind", "dense")
                if kind_f == "dense":
                    _positive(where + ".mlp", f, "ff")
                elif kind_f == "moe":
                    _positive(where + ".mlp.router", f.get("router"), "experts", "top")
                    _positive(where + ".mlp.expert", f.get("expert"), "ff")
                    if f["router"]["top"] > f["router"]["experts"]:
                        raise ConfigError(f"{where}.mlp: top must not exceed experts")
                    if f.get("shared") is not None:
                        _positive(where + ".mlp.shared", f["shared"], "ff")
                else:
                    raise ConfigError(f"{where}: feed-forward kind {kind_f!r} is not one of dense, moe")

    # -- the model as data --------------------------------------------------
    def _mixer(self, layer: Mapping[str, Any]) -> PartSpec:
        m, width, eps = layer["mixer"], self.width, self.eps
        left, right = m["left"], m["right"]
        common = {"hidden_size": width, "num_heads": int(left["heads"]),
                  "num_kv_heads": int(left.get("kv_heads", left["heads"])), "head_dim": int(left["dim"]),
                  "value_dim": int(left["vdim"]), "scale": float(left["scale"]), "window": 0}
        names = {"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b",
                 "q_norm": "q.norm", "k_norm": "k.norm", "sink": "sink"}
        if layer["type"] == "parallel":
            rot = left["rot"]
            attention = PartSpec("gqa_attention", {**common, "qk_norm_eps": None, "value_from_key": True,
                                                   "chunk": int(left["mask"]["size"]), "names": names})
            left_position = PartSpec("rotary", {"dim": int(rot["dims"]), "theta": float(rot["base"])})
            other = PartSpec("gated_recurrent_unit", {"hidden_size": width, "width": int(right["width"]),
                                                      "blocks": int(right["blocks"]), "conv_taps": int(right["conv"]),
                                                      "rate": UNIT_RATE})
            right_position = None
        else:
            attention = PartSpec("gqa_attention", {**common, "qk_norm_eps": eps, "qk_norm_scope": "head", "bias": "qkv",
                                                   "q_temp": left.get("q_temp"), "softcap": float(left.get("softcap") or 0.0),
                                                   "sink": True, "names": names})
            left_position = PartSpec("distance_slopes", {"exponent": SLOPE_EXPONENT})
            rot = right["rot"]
            other = PartSpec("retention", {"hidden_size": width, "num_heads": int(right["heads"]), "key_dim": int(right["dim"]),
                                           "value_dim": int(right["vdim"]), "decay": tuple(float(d) for d in right["decay"]),
                                           "norm_eps": eps})
            right_position = PartSpec("rotary", {"dim": int(rot["dims"]), "theta": float(rot["base"])})
        return PartSpec("parallel", {"hidden_size": width, "branch_norm": {"eps": eps, "tensor": "out"}, "branches": (
            {"name": "left", "mixer": attention, "position": left_position, "scale": 0.5},
            {"name": "right", "mixer": other, "position": right_position, "scale": 0.5})})

    def _feed_forward(self, f) -> PartSpec:
        if f is None:
            return PartSpec("none")
        if f.get("kind", "dense") == "dense":
            return PartSpec("gated_unit", {"hidden_size": self.width, "intermediate_size": int(f["ff"]),
                                           "activation": "gelu_tanh"})
        shared = f.get("shared")
        return PartSpec("routed_experts", {
            "hidden_size": self.width, "expert_size": int(f["expert"]["ff"]), "experts": int(f["router"]["experts"]),
            "top": int(f["router"]["top"]), "score": "softmax_chosen", "activation": "swiglu", "scale": "output",
            "shared": {"ff": int(shared["ff"]), "gate": True} if shared else None})

    def schedule(self) -> list[LayerRun]:
        """Every run of a layer has a cache entry of its own; the first layer of every pass of the loop, the first
        pass too, has the embedding's output fed in through the injection part in front of it."""
        n = len(self.layers)
        loop = self.raw.get("loop")
        order = [(i, False) for i in range(n)]
        if loop:
            start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
            order = [(i, False) for i in range(start)]
            for _ in range(times):
                order += [(i, i == start) for i in range(start, stop)]
            order += [(i, False) for i in range(stop, n)]
        return [LayerRun(layer=i, cache=entry, inject=first) for entry, (i, first) in enumerate(order)]

    def model_spec(self) -> ModelSpec:
        width, vocab, r = self.width, self.vocab, self.raw
        norm = PartSpec("layernorm", {"width": width, "eps": self.eps, "tensor": ""})
        layers, optional = [], []
        for i, layer in enumerate(self.layers):
            feed_forward = self._feed_forward(layer.get("mlp"))
            if feed_forward.kind == "none":
                optional += [f"l{i}.norm2", f"l{i}.norm2b"]
            block = PartSpec("sandwich_norm", {"names": {
                "mixer_norm": "norm1", "mixer": "mix", "feed_forward_norm": "norm2", "feed_forward": "mlp",
                "mixer_post_norm": "norm1b", "feed_forward_post_norm": "norm2b"}})
            layers.append(LayerSpec(prefix=f"l{i}", block=block, mixer=self._mixer(layer), feed_forward=feed_forward,
                                    mixer_norm=norm, feed_forward_norm=norm, position=PartSpec("none"),
                                    extra={"mixer_post_norm": norm, "feed_forward_post_norm": norm}))
        emb = r.get("embedding") or {}
        has_loop = bool(r.get("loop"))
        return ModelSpec(
            architecture="Pikurax", hidden_size=width, vocab_size=vocab,
            max_positions=int(r.get("max_positions", DEFAULT_MAX_POSITIONS)),
            embedding=PartSpec("pair_embedding", {"vocab_size": vocab, "width": width, "tensor": "embed",
                                                  "scale": float(emb.get("scale", 1.0)), "pairs": emb.get("bigram"),
                                                  "pairs_tensor": "bigram"}),
            final_norm=norm,
            head=PartSpec("linear_head", {"vocab_size": vocab, "width": width, "tied": True,
                                          "scale": float(r.get("logit_scale") or 1.0),
                                          "softcap": float(r.get("logit_softcap") or 0.0)}),
            layers=tuple(layers), schedule=tuple(self.schedule()),
            names={"embedding": "", "final_norm": "final.norm", "head": "head", "injection": "loop"},
            optional_tensors=tuple(optional),
            injection=PartSpec("concat_projection", {"width": width, "tensor": "in"}) if has_loop else None)
