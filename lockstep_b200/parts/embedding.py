"""Token embedding (a gather into the float32 residual stream; LockStep:
engine/model/qwen3.py:319) and the output head (logits = y @ W^T, float32 out;
engine/model/qwen3.py:373), whose weight may be the embedding table itself.

"pair_embedding": the token's row times ``scale``, plus, with ``pairs`` = {"buckets", "mul_prev", "mul_cur"}, row
(previous token x mul_prev + token x mul_cur) mod buckets of a second table of buckets + 1 rows, whose last row
serves a request's first token.  The previous token of a portion's first token is what the request keeps between
steps: the part has a cache need of its own (one int32 per request: the last token it was fed, plus one).

The head takes ``scale`` (a factor on the logits) and ``softcap`` (logits <- cap tanh(logits / cap), after the factor)."""

from __future__ import annotations

import torch

from .. import kernels as K
from .base import CacheNeed, Part, Runtime, WeightSpec, register_part


class TokenEmbedding(Part):
    graph_safe = True

    def __init__(self, vocab_size: int, width: int, runtime: Runtime, tensor: str = "weight"):
        self.vocab, self.width, self.rt = int(vocab_size), int(width), runtime
        self.tensor = str(tensor)     # local name of the table ("" where the part's prefix names it)
        self.table = None

    def weight_specs(self):
        return {self.tensor: WeightSpec((self.vocab, self.width), "table")}

    def bind(self, tensors):
        self.table = tensors[self.tensor]

    def forward(self, ctx) -> torch.Tensor:
        """The float32 residual stream [tokens, width] of the step's tokens.  An
        embedding that encodes absolute positions would add them here (``ctx.positions``)."""
        ids = ctx.token_ids
        h = self.rt.rows(ids.numel(), self.width, dtype=torch.float32)
        K.embed_gather(ids, self.table, h, self.rt.err)
        return h

    def accumulate(self, h: torch.Tensor, ctx) -> None:
        """h += what ``forward`` returned for this step: for a schedule that feeds the embedding
        in again before a later run of a layer.  The table is read again; nothing is kept."""
        K.embed_gather(ctx.token_ids, self.table, h, self.rt.err, accumulate=True)


class PairEmbedding(TokenEmbedding):
    def __init__(self, vocab_size: int, width: int, runtime: Runtime, tensor: str = "weight", scale: float = 1.0,
                 pairs=None, pairs_tensor: str = "pairs"):
        super().__init__(vocab_size, width, runtime, tensor)
        self.scale, self.pairs_tensor = float(scale), str(pairs_tensor)
        self.pairs = None
        if pairs:
            self.pairs = (int(pairs["buckets"]), int(pairs["mul_prev"]), int(pairs["mul_cur"]))
            if self.pairs[0] <= 0 or self.pairs[1] < 0 or self.pairs[2] < 0:
                raise ValueError("pair_embedding: buckets must be positive, the multipliers not negative")
        self.pair_table = None

    def cache_need(self):
        return CacheNeed("state", state_shape=(1,), state_dtype=torch.int32) if self.pairs else None

    def weight_specs(self):
        specs = super().weight_specs()
        if self.pairs:
            specs[self.pairs_tensor] = WeightSpec((self.pairs[0] + 1, self.width), "table")
        return specs

    def bind(self, tensors):
        super().bind(tensors)
        if self.pairs:
            self.pair_table = tensors[self.pairs_tensor]

    def forward(self, ctx, cache=None) -> torch.Tensor:
        ids = ctx.token_ids
        h = self.rt.rows(ids.numel(), self.width, dtype=torch.float32)
        if self.pairs:
            K.pair_embed(ids, ctx.token_slot, cache.state, self.table, self.pair_table, h, self.scale, self.pairs[1],
                         self.pairs[2], self.rt.err)
        else:
            K.pair_embed(ids, None, None, self.table, None, h, self.scale, 0, 0, self.rt.err)
        return h

    def accumulate(self, h, ctx) -> None:
        raise NotImplementedError("pair_embedding feeds a later pass through the model's injection part, not by adding")


class LinearHead(Part):
    graph_safe = True

    def __init__(self, vocab_size: int, width: int, tied: bool, runtime: Runtime, tensor: str = "weight",
                 scale: float = 1.0, softcap: float = 0.0):
        self.vocab, self.width, self.tied, self.rt = int(vocab_size), int(width), bool(tied), runtime
        self.scale, self.softcap = float(scale), float(softcap or 0.0)
        self.tensor = str(tensor)     # local name of an untied head's matrix ("" where the part's prefix names it)
        self.weight = None

    def weight_specs(self):
        return {} if self.tied else {self.tensor: WeightSpec((self.vocab, self.width))}

    def bind(self, tensors):
        self.weight = tensors["weight" if self.tied else self.tensor]

    def forward(self, y: torch.Tensor) -> torch.Tensor:
        logits = self.rt.rows(y.shape[0], self.vocab, dtype=torch.float32)
        K.gemm_nt(y, self.weight, logits, err=self.rt.err)
        if self.scale != 1.0 or self.softcap > 0.0:
            K.scale_cap(logits, self.scale, self.softcap)
        return logits


@register_part("embedding", "token_embedding")
def _build_embedding(spec, runtime, **_):
    return TokenEmbedding(spec["vocab_size"], spec["width"], runtime, spec.get("tensor", "weight"))


@register_part("embedding", "pair_embedding")
def _build_pair_embedding(spec, runtime, **_):
    return PairEmbedding(spec["vocab_size"], spec["width"], runtime, spec.get("tensor", "weight"), spec.get("scale", 1.0),
                         spec.get("pairs"), spec.get("pairs_tensor", "pairs"))


@register_part("head", "linear_head")
def _build_head(spec, runtime, **_):
    return LinearHead(spec["vocab_size"], spec["width"], spec.get("tied", False), runtime, spec.get("tensor", "weight"),
                      spec.get("scale", 1.0), spec.get("softcap", 0.0))
