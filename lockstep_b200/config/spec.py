"""What a model is made of, as plain data.

An architecture's configuration class turns its ``config.json`` keys into a
``ModelSpec``: one ``LayerSpec`` per layer (which mixer, feed-forward, norm and
position encoding, each with its sizes and constants as parameters) and a
``schedule`` that says in which order layers run and whose cache each run uses.
Nothing below the configuration class knows which architecture it serves.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from types import MappingProxyType
from typing import Any, Mapping


def _freeze(params: Mapping[str, Any] | None) -> Mapping[str, Any]:
    return MappingProxyType(dict(params or {}))


@dataclass(frozen=True)
class PartSpec:
    """A part by the name it is registered under, and its parameters."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def __post_init__(self):
        object.__setattr__(self, "params", _freeze(self.params))

    def __getitem__(self, key: str) -> Any:
        return self.params[key]

    def get(self, key: str, default=None) -> Any:
        return self.params.get(key, default)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a block arrangement over a mixer and a feed-forward.

    ``prefix`` is the tensor-name prefix of the layer's weights
    (``model.layers.3``); each part adds its own suffixes.  ``extra`` holds whatever further
    parts the layer's block arrangement asks for, by the name it asks under (norms after the
    mixer or the feed-forward, a second feed-forward branch, ...): the block receives the whole
    ``LayerSpec`` and builds them, nothing else reads them.
    """

    prefix: str
    block: PartSpec            # arrangement, e.g. pre_norm
    mixer: PartSpec            # e.g. gqa_attention
    feed_forward: PartSpec     # e.g. swiglu
    mixer_norm: PartSpec       # norm in front of the mixer
    feed_forward_norm: PartSpec
    position: PartSpec         # position encoding the mixer applies
    extra: Mapping[str, PartSpec] = field(default_factory=dict)

    def __post_init__(self):
        object.__setattr__(self, "extra", _freeze(self.extra))


@dataclass(frozen=True)
class LayerRun:
    """One entry of the schedule: run layer ``layer`` on cache entry ``cache``.

    A layer may be run more than once (give each run its own ``cache``), and a
    run may read a cache entry that an earlier run wrote (``writes_cache``
    False): it then adds nothing to the cache.  ``add_embedding``: the embedding's output for
    the step's tokens is added to the residual stream right before this run (a model that
    passes over some of its layers several times and feeds the embedding in again each time).
    ``borrows``: pairs (part, entry) for a layer whose cache need has several parts: part
    ``part`` of this run's cache is not its own but the same part of cache entry ``entry``, which
    an earlier run wrote, and is only read (a layer that attends over another layer's keys and
    values but carries a state of its own besides).
    ``inject``: the model's injection part (``ModelSpec.injection``) runs on the residual stream right before this
    run (a model that feeds the embedding's output in again through a projection at the start of every pass).
    """

    layer: int
    cache: int
    writes_cache: bool = True
    add_embedding: bool = False
    borrows: tuple = ()
    inject: bool = False


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    final_norm: PartSpec
    head: PartSpec
    layers: tuple[LayerSpec, ...]
    schedule: tuple[LayerRun, ...]
    # tensor-name prefixes of the parts that are not layers
    names: Mapping[str, str] = field(default_factory=lambda: {
        "embedding": "model.embed_tokens", "final_norm": "model.norm", "head": "lm_head"})
    # tensors a model folder may hold although this model reads none of them (say, the norm in
    # front of a feed-forward that the layer does not have)
    optional_tensors: tuple[str, ...] = ()
    # a part that mixes the embedding's output into the residual stream where the schedule says so
    # (``LayerRun.inject``); its tensors lie under ``names["injection"]``
    injection: PartSpec | None = None

    def __post_init__(self):
        object.__setattr__(self, "names", _freeze(self.names))
        object.__setattr__(self, "layers", tuple(self.layers))
        object.__setattr__(self, "schedule", tuple(self.schedule))
        object.__setattr__(self, "optional_tensors", tuple(self.optional_tensors))
        writers: dict[int, int] = {}
        for run in self.schedule:
            if run.inject and self.injection is None:
                raise ValueError("the schedule injects the embedding's output, but the model has no injection part")
            if not 0 <= run.layer < len(self.layers):
                raise ValueError(f"schedule names layer {run.layer}, the model has {len(self.layers)}")
            for part, entry in run.borrows:
                if entry not in writers or entry == run.cache:
                    raise ValueError(f"a run borrows part {part} of cache entry {entry} before any run wrote it")
            if run.writes_cache:
                if run.cache in writers:
                    raise ValueError(f"cache entry {run.cache} is written by two runs of the schedule")
                writers[run.cache] = run.layer
            elif run.cache not in writers:
                raise ValueError(f"a run reads cache entry {run.cache} before any run wrote it")

    @property
    def cache_entries(self) -> int:
        return 1 + max((run.cache for run in self.schedule), default=-1)


def tensor_name(prefix: str, local: str) -> str:
    """The full name of a part's tensor: a part may name a tensor "" to own its prefix itself
    (an embedding stored as ``embed`` rather than ``embed.weight``)."""
    if not prefix:
        return local        # a part without a prefix names its tensors itself
    return f"{prefix}.{local}" if local else prefix


def own_tensors(prefix: str, tensors: Mapping[str, Any]) -> dict[str, Any]:
    """The entries of ``tensors`` that lie under ``prefix``, by their local names (all of them for a part without
    a prefix)."""
    if not prefix:
        return dict(tensors)
    out = {k[len(prefix) + 1:]: v for k, v in tensors.items() if k.startswith(prefix + ".")}
    if prefix in tensors:
        out[""] = tensors[prefix]
    return out


class ConfigError(ValueError):
    """config.json is missing a key, has a wrong value, or asks for what the engine lacks."""
