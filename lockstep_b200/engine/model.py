"""The model: parts assembled from a ``ModelSpec``, and nothing else.

``Model`` builds the embedding, one block per ``LayerSpec``, the final norm and
the head through the part registries, gathers the tensors they need under their
full names, and hands loaded tensors back to them.  The order in which layers
run is ``spec.schedule``.
"""

from __future__ import annotations

from dataclasses import replace

import torch

from ..config.spec import ModelSpec, own_tensors, tensor_name
from ..parts import Runtime, WeightSpec, build_part


class Model:
    def __init__(self, spec: ModelSpec, runtime: Runtime):
        self.spec, self.rt = spec, runtime
        self.embedding = build_part("embedding", spec.embedding, runtime)
        self.blocks = [build_part("block", layer.block, runtime, layer_spec=layer) for layer in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, runtime)
        self.head = build_part("head", spec.head, runtime)
        self.tied_head = bool(getattr(self.head, "tied", False))
        self.injection = build_part("injection", spec.injection, runtime) if spec.injection is not None else None
        # an embedding that keeps something per request (the token before a portion) has a cache entry of its own,
        # after the schedule's
        need = getattr(self.embedding, "cache_need", lambda: None)()
        self.embedding_entry = spec.cache_entries if need is not None else None

    # -- weights ------------------------------------------------------------
    def _named_parts(self):
        n = self.spec.names
        yield n["embedding"], self.embedding
        for layer, block in zip(self.spec.layers, self.blocks):
            yield layer.prefix, block
        yield n["final_norm"], self.final_norm
        yield n["head"], self.head
        if self.injection is not None:
            yield n["injection"], self.injection

    def weight_specs(self) -> dict[str, WeightSpec]:
        out: dict[str, WeightSpec] = {}
        for prefix, part in self._named_parts():
            for local, spec in part.weight_specs().items():
                out[tensor_name(prefix, local)] = spec
        return out

    def aliases(self) -> dict[str, str]:
        """Names the file may store although the model takes them from another tensor."""
        n = self.spec.names
        if not self.tied_head:
            return {}
        table = tensor_name(n["embedding"], next(iter(self.embedding.weight_specs())))
        return {f"{n['head']}.weight": table}

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        for prefix, part in self._named_parts():
            own = own_tensors(prefix, tensors)
            if part is self.head and self.tied_head:
                own = {"weight": self.embedding.table}
            if own or part.weight_specs():
                part.bind(own)

    # -- cache --------------------------------------------------------------
    def cache_needs(self):
        """For each cache entry of the schedule, the need of the layer that writes it, widened
        to what the layers that only read it ask for (a reader with a longer window, or none,
        keeps the writer's pages alive that long)."""
        needs = [None] * self.spec.cache_entries
        for run in self.spec.schedule:
            if run.writes_cache:
                need = self.blocks[run.layer].cache_need()
                if run.borrows:
                    # the borrowed parts are another entry's: this one holds nothing in their place
                    if need is None or need.kind != "several":
                        raise ValueError(f"layer {run.layer} borrows a part of a cache need that has no parts")
                    taken = {part for part, _ in run.borrows}
                    need = replace(need, parts=tuple(None if i in taken else sub for i, sub in enumerate(need.parts)))
                needs[run.cache] = need
        for run in self.spec.schedule:
            if not run.writes_cache and needs[run.cache] is not None:
                needs[run.cache] = needs[run.cache].widened(self.blocks[run.layer].cache_need())
            for part, entry in run.borrows:
                reader, lender = self.blocks[run.layer].cache_need().parts[part], needs[entry]
                if lender is None or lender.kind != "several" or lender.parts[part] is None:
                    raise ValueError(f"layer {run.layer} borrows part {part} of cache entry {entry}, which has none")
                parts = list(lender.parts)
                parts[part] = parts[part].widened(reader)
                needs[entry] = replace(lender, parts=tuple(parts))
        if self.embedding_entry is not None:
            needs.append(self.embedding.cache_need())
        return needs


def expected_weights(spec: ModelSpec) -> dict[str, WeightSpec]:
    """Names, shapes and roles of the tensors a model of ``spec`` reads, without a device."""
    rt = Runtime(device=torch.device("cpu"), dtype=torch.float32, page_size=16,
                 max_positions=2, err=torch.zeros(2, dtype=torch.int32))
    return Model(spec, rt).weight_specs()
