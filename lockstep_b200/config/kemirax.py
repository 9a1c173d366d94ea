"""Kemirax: a decoder whose layers run their mixer and their feed-forward side by side on one
normed row, with gates on both results.

``config.json`` holds ``vocab``, ``width``, ``norm.eps`` and a list ``layers``; every entry gives
``type`` (which mixer), ``mixer`` (its sizes and constants) and ``mlp`` (its feed-forward, or null
for none).  A layer computes y = norm(x) (an RMS norm whose gain is one number), lets the mixer read
y_t + (y_(t-1) - y_t) * shift and the feed-forward y_t, multiplies each result by a gate
sigmoid(W y + b) of its own and adds the sum to x.  Two mixers:

- ``latent_attention``: per token one normed latent of ``kv_rank`` elements and one rotated key part
  of ``rot_dim`` elements are cached; queries come through a normed latent of ``q_rank`` elements;
  heads of ``dim`` plain + ``rot_dim`` rotated query elements, values of ``vdim``; rotation of halves
  with stretched frequencies (``rot.scaling``); causal softmax over every earlier key.  With
  ``kv_from: j`` the layer has no down-projection and reads what layer j cached.
- ``gla``: gated linear attention, a decayed sum of outer products per head with a decay per key
  channel sigmoid(z)^(1/``tau``), a per-head RMS norm of the read-out and a silu gate.

The feed-forward (``kind`` "moe") routes every token to ``router.top`` of ``router.experts`` +
``router.identity`` experts by softmax scores plus a stored correction; the last ``identity`` experts
return their input; the others are gated units with clamps at ``expert.limit``; ``shared`` is one
more such unit that every token runs, weighted by a sigmoid gate of its own.  Layer i's tensors
start with ``l<i>.``: ``norm1``, ``shift``, ``rg1``, ``rg2``, ``mix.*``, ``mlp.*``; the head is ``head``.
"""

from __future__ import annotations

import copy
from typing import Any, Mapping

from .registry import register_architecture
from .spec import ConfigError, LayerRun, LayerSpec, ModelSpec, PartSpec

MIXERS = ("latent_attention", "gla")
DEFAULT_MAX_POSITIONS = 32768
GLU_ALPHA = 1.702          # the sigmoid's slope in an expert's activation


def _positive(where: str, raw: Mapping[str, Any], *keys: str) -> None:
    for k in keys:
        if not isinstance(raw, Mapping) or k not in raw:
            raise ConfigError(f"{where} lacks {k!r}")
        if not (isinstance(raw[k], int) and not isinstance(raw[k], bool) and raw[k] > 0):
            raise ConfigError(f"{where}: {k} must be a positive integer, got {raw[k]!r}")


def _number(where: str, raw: Mapping[str, Any], *keys: str) -> None:
    for k in keys:
        if not isinstance(raw, Mapping) or not isinstance(raw.get(k), (int, float)) or isinstance(raw.get(k), bool):
            raise ConfigError(f"{where}: {k} must be a number")


@register_architecture("Kemirax")
class KemiraxConfig:
    def __init__(self, raw: Mapping[str, Any]):
        self.raw = copy.deepcopy(dict(raw))
        self.validate()

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "KemiraxConfig":
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
        if not isinstance(r.get("layers"), list) or not r["layers"]:
            raise ConfigError("config.json: layers must be a list with at least one layer")
        for i, layer in enumerate(r["layers"]):
            where = f"layers[{i}]"
            kind = layer.get("type") if isinstance(layer, Mapping) else None
            if kind not in MIXERS:
                raise ConfigError(f"{where}: type {kind!r} is not one of {MIXERS}")
            m = layer.get("mixer")
            if not isinstance(m, Mapping):
                raise ConfigError(f"{where} lacks its mixer's sizes")
            if kind == "gla":
                _positive(where, m, "heads", "dim", "vdim")
                _number(where, m, "tau")
                if not float(m["tau"]) > 0:
                    raise ConfigError(f"{where}: tau must be positive")
            else:
                _positive(where, m, "heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank")
                _number(where, m, "scale")
                rot = m.get("rot")
                _positive(where + ".rot", rot, "dims")
                if rot["dims"] != m["rot_dim"] or rot["dims"] % 2 or not float(rot.get("base", 0)) > 0:
                    raise ConfigError(f"{where}: rot.dims must be even and equal rot_dim, rot.base positive")
                scaling = rot.get("scaling")
                if scaling is not None:
                    _number(where + ".rot.scaling", scaling, "factor", "original", "fast", "slow")
                    if not float(scaling["factor"]) > 0 or not float(scaling["original"]) > 0:
                        raise ConfigError(f"{where}.rot.scaling: factor and original must be positive")
                src = m.get("kv_from")
                if src is not None:
                    if not (isinstance(src, int) and not isinstance(src, bool) and 0 <= src < i) \
                            or r["layers"][src].get("type") != "latent_attention" \
                            or r["layers"][src]["mixer"].get("kv_from") is not None:
                        raise ConfigError(f"{where}: kv_from must name an earlier latent_attention layer with a "
                                          "down-projection of its own")
                    other = r["layers"][src]["mixer"]
                    if any(other[k] != m[k] for k in ("kv_rank", "rot_dim")) or other["rot"] != rot:
                        raise ConfigError(f"{where}: kv_rank, rot_dim and rot must equal those of layer {src}, whose "
                                          "cache it reads")
            f = layer.get("mlp")
            if f is not None:
                if not isinstance(f, Mapping) or f.get("kind", "moe") != "moe":
                    raise ConfigError(f"{where}: feed-forward kind {f.get('kind')!r} is not supported (moe)")
                _positive(where + ".mlp.expert", f.get("expert"), "ff")
                _number(where + ".mlp.expert", f["expert"], "limit")
                router = f.get("router")
                _positive(where + ".mlp.router", router, "experts", "top")
                identity = router.get("identity", 0)
                if not (isinstance(identity, int) and not isinstance(identity, bool) and identity >= 0):
                    raise ConfigError(f"{where}.mlp.router: identity must be a count, got {identity!r}")
                if router["top"] > router["experts"] + identity:
                    raise ConfigError(f"{where}: top exceeds the number of experts")
                shared = f.get("shared")
                if shared is not None:
                    _positive(where + ".mlp.shared", shared, "ff")
                    _number(where + ".mlp.shared", shared, "limit")

    # -- the model as data --------------------------------------------------
    def _mixer(self, layer: Mapping[str, Any]) -> tuple[PartSpec, PartSpec]:
        m, width, eps = layer["mixer"], self.width, self.eps
        if layer["type"] == "gla":
            return PartSpec("gated_linear", {
                "hidden_size": width, "num_heads": int(m["heads"]), "key_dim": int(m["dim"]),
                "value_dim": int(m["vdim"]), "tau": float(m["tau"]), "norm_eps": eps,
                # the rank of the decay's low-rank map is the stored tensors' own; a configuration
                # may name it (random weights need it)
                "decay_rank": m.get("decay_rank")}), PartSpec("none")
        rot = m["rot"]
        position = PartSpec("scaled_rotary", {"dim": int(rot["dims"]), "theta": float(rot["base"]),
                                              "scaling": rot.get("scaling"), "interleaved": False})
        mixer = PartSpec("latent_attention", {
            "hidden_size": width, "num_heads": int(m["heads"]), "head_dim": int(m["dim"]), "rot_dim": int(m["rot_dim"]),
            "value_dim": int(m["vdim"]), "kv_rank": int(m["kv_rank"]), "q_rank": int(m["q_rank"]),
            "scale": float(m["scale"]), "window": 0, "norm_eps": eps, "sink": False,
            "borrows_kv": m.get("kv_from") is not None})
        return mixer, position

    def _feed_forward(self, f: Mapping[str, Any] | None) -> PartSpec:
        if f is None:
            return PartSpec("none")
        router, shared = f["router"], f.get("shared")
        return PartSpec("routed_experts", {
            "hidden_size": self.width, "expert_size": int(f["expert"]["ff"]), "experts": int(router["experts"]),
            "identity": int(router.get("identity", 0)), "top": int(router["top"]), "score": "softmax",
            "correction": True, "scale": "output", "activation": "clamped_glu", "limit": float(f["expert"]["limit"]),
            "alpha": GLU_ALPHA,
            "shared": None if shared is None else {"ff": int(shared["ff"]), "limit": float(shared["limit"]), "gate": True}})

    def model_spec(self) -> ModelSpec:
        width, vocab = self.width, self.vocab
        norm = PartSpec("rmsnorm", {"width": width, "eps": self.eps, "tensor": "", "scalar": True})
        block = PartSpec("shared_norm", {"hidden_size": width, "shift": True, "gates": True, "names": {
            "norm": "norm1", "mixer": "mix", "feed_forward": "mlp", "shift": "shift", "mixer_gate": "rg1",
            "mixer_gate_bias": "rg1.b", "feed_forward_gate": "rg2", "feed_forward_gate_bias": "rg2.b"}})
        layers, schedule, optional = [], [], []
        for i, layer in enumerate(self.layers):
            mixer, position = self._mixer(layer)
            feed_forward = self._feed_forward(layer.get("mlp"))
            if feed_forward.kind == "none":
                optional += [f"l{i}.rg2", f"l{i}.rg2.b"]
            layers.append(LayerSpec(prefix=f"l{i}", block=block, mixer=mixer, feed_forward=feed_forward,
                                    mixer_norm=norm, feed_forward_norm=norm, position=position))
            # part 0 of a layer's cache is its mixer's, part 1 the row its shift carries: a layer that
            # reads another's latents borrows part 0 and keeps a part 1 of its own
            src = layer["mixer"].get("kv_from") if layer["type"] == "latent_attention" else None
            schedule.append(LayerRun(layer=i, cache=i, borrows=() if src is None else ((0, int(src)),)))
        return ModelSpec(
            architecture="Kemirax", hidden_size=width, vocab_size=vocab,
            max_positions=int(self.raw.get("max_positions", DEFAULT_MAX_POSITIONS)),
            embedding=PartSpec("token_embedding", {"vocab_size": vocab, "width": width, "tensor": ""}),
            final_norm=norm,
            head=PartSpec("linear_head", {"vocab_size": vocab, "width": width, "tied": False, "tensor": ""}),
            layers=tuple(layers), schedule=tuple(schedule),
            names={"embedding": "embed", "final_norm": "final.norm", "head": "head"},
            optional_tensors=tuple(optional))
