"""Grouped-query attention over the paged cache.

q, k, v projections without bias as one product over the row-concatenated
weights (a row of the product is the same dot product as in three separate
ones), optional per-head RMSNorm of q and k before the rotation, rotation by
the position encoding, write of k and v into the cache pages, causal softmax
attention with an optional window, output projection added into the residual
stream (LockStep: engine/model/qwen3.py:246-277, engine/kernels/attention.py).

Further parameters, for designs that differ from that one:
- ``value_dim``: the size of a value head where it is not the size of a key head.  The cache
  and the attention kernels then work on heads of one padded size D (the larger of the two,
  rounded up to 16): queries and keys are padded with zeros (no score changes), values too
  (the padded outputs are zero and meet zero columns of the output projection).
- ``qk_norm_scope`` "projection": one RMSNorm over the whole query projection and one over
  the whole key projection, with gains of those sizes, before the heads are split ("head":
  one norm per head with a gain of the head's size).
- ``borrows_kv``: the layer has no key or value tensors; the schedule gives it the cache
  entry of another layer, which it reads with its own queries, window and scale.
- ``names``: the local names of its tensors.
- ``bias``: the four projections have biases (``q_bias`` ... ``o_bias`` in ``names``); those of q, k
  and v are added by the kernel that finishes the heads, the output's goes into the residual stream.
- ``q_temp`` = {"coef": c, "every": n}: the query at position p is multiplied by
  1 + c ln(floor((p + 1) / n) + 1).
- ``score_bias`` "log_distance": r1[head] ln(1 + r2[head] (i - j)) is taken off the score of query i
  with key j; r1 and r2 are tensors of the layer, one number per query head (``names``: ``r1``, ``r2``).
- ``bias`` "qkv": biases on q, k and v only (none on the output projection).
- ``value_from_key``: there is no value projection; the values are the keys as projected, before any norm or
  rotation (the key matrix serves twice in the one product; value heads have the size of key heads).
- ``chunk``: a query sees the earlier keys of its own chunk of ``chunk`` positions only, chunks counted from
  position 0 of the sequence (the kernels take it as a negative window; every page is kept).
- ``softcap``: the scaled score becomes softcap tanh(score / softcap) before any bias is taken off (CUDA-core kernels).
- ``sink``: a learned number per query head (``names``: ``sink``) whose exponential is one more term
  of the softmax's denominator; it has no key and no value.
"""

from __future__ import annotations

import torch

from .. import kernels as K
from .base import CacheNeed, Mixer, PositionEncoding, Runtime, WeightSpec, register_part
from .norm import NormedRows


_DEFAULT_NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight",
                  "q_norm": "q_norm.weight", "k_norm": "k_norm.weight",
                  "q_bias": "q_proj.bias", "k_bias": "k_proj.bias", "v_bias": "v_proj.bias", "o_bias": "o_proj.bias",
                  "r1": "r1", "r2": "r2", "sink": "sink"}


def _f32(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.float32).contiguous()


class ScoreExtras:
    """What the attention kernels add to plain scaled scores: a bias that grows with the distance
    of key and query (``slopes`` alone: linear; with ``log_rates``: logarithmic) and sinks.  The
    tensor-core kernel of prompt portions knows all of them; that of decoded tokens the logarithmic bias (a linear
    bias or a cap keeps decoded tokens on the CUDA-core kernels)."""

    def __init__(self, slopes=None, log_rates=None, sinks=None, softcap: float = 0.0):
        self.slopes, self.log_rates, self.sinks, self.softcap = slopes, log_rates, sinks, float(softcap or 0.0)

    def tensor_cores(self) -> bool:
        """Whether the tensor-core kernel of decoded tokens knows these extras (that of prompt portions knows all)."""
        return (self.slopes is None or self.log_rates is not None) and not self.softcap


def attend(rt: Runtime, q, ctx, cache, nq: int, nkv: int, d: int, window: int, scale: float, exact: bool,
           extras: ScoreExtras) -> torch.Tensor:
    """Causal attention of the step's queries ``q`` [tokens, nq d] over a layer's pages (heads of one
    size ``d``): prompt portions by tiles, single tokens by splits and a fold.  Returns [tokens, nq d]
    in the engine's type.  ``exact``: every row takes the tile kernel, so that a row's bits do not
    depend on whether it was decoded or part of a prompt.  ``window`` < 0: chunks of -window positions."""
    t = q.shape[0]
    tensor_core_attention = not exact and extras.tensor_cores()
    attn = rt.rows(t, nq * d)
    plan, done = None, False
    if not exact and d in (64, 128):
        plan = ctx.attention_plan(window, K.attention_prefill_tc_tile_tokens())
        done = not plan.n_tile or K.attention_prefill_tc(
            q, cache.pages, attn, plan.tile_work, plan.n_tile, cache.block_table, nq, nkv, d,
            window, scale, rt.err, extras.slopes, extras.log_rates, extras.sinks, softcap=extras.softcap)
    if not done:
        plan = ctx.attention_plan(window)
        if plan.n_tile:
            K.attention_tile(q, cache.pages, attn, None, None, plan.tile_work, plan.n_tile,
                             cache.block_table, nq, nkv, d, window, scale, rt.err, extras.slopes,
                             extras.log_rates, extras.sinks, softcap=extras.softcap)
    if plan.n_split:
        part_acc = rt.rows(plan.n_slots, nq, d, dtype=torch.float32)
        part_ml = rt.rows(plan.n_slots, nq, 2, dtype=torch.float32)
        done = False
        if tensor_core_attention:
            done = K.attention_decode_mma(q, cache.pages, part_acc, part_ml, plan.split_work,
                                          plan.n_split, cache.block_table, nq, nkv, d, window,
                                          scale, rt.err, extras.slopes, extras.log_rates)
        if not done and not exact:
            done = K.attention_decode(q, cache.pages, part_acc, part_ml, plan.split_work,
                                      plan.n_split, cache.block_table, nq, nkv, d, window,
                                      scale, rt.err, extras.slopes, extras.log_rates, softcap=extras.softcap)
        if not done:
            K.attention_tile(q, cache.pages, None, part_acc, part_ml, plan.split_work,
                             plan.n_split, cache.block_table, nq, nkv, d, window,
                             scale, rt.err, extras.slopes, extras.log_rates, softcap=extras.softcap)
        K.attention_combine(part_acc, part_ml, attn, plan.combine_items, plan.n_combine, nq, d, extras.sinks)
    return attn


class GQAttention(Mixer):
    graph_safe = True
    accepts_normed_rows = True
    can_overwrite = True

    def __init__(self, hidden_size, num_heads, num_kv_heads, head_dim, scale, window, qk_norm_eps,
                 position: PositionEncoding, runtime: Runtime, value_dim=None, qk_norm_scope="head",
                 borrows_kv=False, names=None, bias=False, q_temp=None, score_bias=None, sink=False,
                 value_from_key=False, chunk=0, softcap=0.0):
        if num_heads % num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if qk_norm_scope not in ("head", "projection"):
            raise ValueError(f"qk_norm_scope must be head or projection, got {qk_norm_scope!r}")
        self.h, self.nq, self.nkv, self.d = int(hidden_size), int(num_heads), int(num_kv_heads), int(head_dim)
        self.dv = int(value_dim or head_dim)
        self.scope, self.borrows = qk_norm_scope, bool(borrows_kv)
        if score_bias not in (None, "log_distance"):
            raise ValueError(f"score_bias must be log_distance or absent, got {score_bias!r}")
        self.bias, self.score_bias, self.sink = bool(bias), score_bias, bool(sink)
        self.output_biased = bool(bias) and bias != "qkv"
        self.value_from_key, self.chunk, self.softcap = bool(value_from_key), int(chunk or 0), float(softcap or 0.0)
        if self.value_from_key and (self.dv != self.d or self.borrows or self.bias):
            raise ValueError("value_from_key: value heads have the size of key heads, and the layer projects its own keys without biases")
        if self.chunk < 0 or (self.chunk and window):
            raise ValueError("chunk must be positive, and a layer has a window or chunks, not both")
        self.q_temp = (float(q_temp["coef"]), int(q_temp["every"])) if q_temp else None
        if self.q_temp is not None and self.q_temp[1] <= 0:
            raise ValueError("q_temp.every must be positive")
        # the general finishing kernel (norm over the projection, heads padded to one size, biases,
        # a query temperature) where the design asks for any of this; else the per-head kernels
        # and the fused products
        self.wide = self.scope == "projection" or self.dv != self.d or self.borrows or self.d % 16 != 0 \
            or self.bias or self.q_temp is not None
        self.pad = -(-max(self.d, self.dv) // 16) * 16 if self.wide else self.d
        if self.pad % 16 or not 16 <= self.pad <= 256:
            raise ValueError(
                f"head size {self.pad} is not supported: the attention kernels take multiples of 16 up to 256")
        self.names = dict(_DEFAULT_NAMES)
        self.names.update(names or {})
        self.scale, self.window = float(scale), int(window or 0)
        self.mask = -self.chunk if self.chunk else self.window     # what the attention kernels and plans are given
        self.qk_norm_eps = qk_norm_eps
        self.position, self.rt = position, runtime
        self.w_qkv = self.w_o = self.q_gain = self.k_gain = self.qkv_bias = self.o_bias = None
        self.extras = ScoreExtras()
        # in float32 every row takes the tile kernel, so that a row's bits do not
        # depend on whether it was decoded or part of a prompt
        self.exact = runtime.dtype == torch.float32

    def cache_need(self):
        return CacheNeed("paged_kv", kv_heads=self.nkv, head_dim=self.pad, window=self.window)

    def attention_windows(self):
        return {self.mask}

    def weight_specs(self):
        n = self.names
        whole = self.scope == "projection"
        specs = {n["q"]: WeightSpec((self.nq * self.d, self.h)),
                 n["o"]: WeightSpec((self.h, self.nq * self.dv))}
        if not self.borrows:
            specs[n["k"]] = WeightSpec((self.nkv * self.d, self.h))
            if not self.value_from_key:
                specs[n["v"]] = WeightSpec((self.nkv * self.dv, self.h))
        if self.qk_norm_eps is not None:
            specs[n["q_norm"]] = WeightSpec((self.nq * self.d if whole else self.d,), "gain")
            if not self.borrows:
                specs[n["k_norm"]] = WeightSpec((self.nkv * self.d if whole else self.d,), "gain")
        small = ("normal", 0.0, 0.02)
        if self.bias:
            specs[n["q_bias"]] = WeightSpec((self.nq * self.d,), "gain", small)
            if self.output_biased:
                specs[n["o_bias"]] = WeightSpec((self.h,), "gain", small)
            if not self.borrows:
                specs[n["k_bias"]] = WeightSpec((self.nkv * self.d,), "gain", small)
                specs[n["v_bias"]] = WeightSpec((self.nkv * self.dv,), "gain", small)
        if self.score_bias == "log_distance":
            specs[n["r1"]] = WeightSpec((self.nq,), "gain", ("uniform", 0.1, 1.0))
            specs[n["r2"]] = WeightSpec((self.nq,), "gain", ("uniform", 0.05, 1.0))
        if self.sink:
            specs[n["sink"]] = WeightSpec((self.nq,), "gain", ("normal", 0.0, 1.0))
        return specs

    def bind(self, tensors):
        n = self.names
        parts = [tensors[n["q"]]] if self.borrows else \
            [tensors[n["q"]], tensors[n["k"]], tensors[n["k" if self.value_from_key else "v"]]]
        self.w_qkv = torch.cat(parts, dim=0).contiguous()
        self.w_o = tensors[n["o"]]
        if self.pad != self.dv:
            # the attention's output has heads of the padded size: zero columns meet the padding
            w = torch.zeros((self.h, self.nq, self.pad), dtype=self.w_o.dtype, device=self.w_o.device)
            w[:, :, :self.dv] = self.w_o.view(self.h, self.nq, self.dv)
            self.w_o = w.view(self.h, self.nq * self.pad).contiguous()
        # asked once: a step allocates nothing for it
        self.extras = ScoreExtras(slopes=self.position.score_slopes(self.nq))
        if self.score_bias == "log_distance":
            if self.extras.slopes is not None:
                raise ValueError("a position encoding with score slopes and a log_distance bias exclude each other")
            self.extras = ScoreExtras(slopes=_f32(tensors[n["r1"]]), log_rates=_f32(tensors[n["r2"]]))
        if self.sink:
            self.extras.sinks = _f32(tensors[n["sink"]])
        self.extras.softcap = self.softcap
        if self.bias:
            parts = [tensors[n["q_bias"]]] if self.borrows else [tensors[n[k]] for k in ("q_bias", "k_bias", "v_bias")]
            self.qkv_bias = _f32(torch.cat([p.reshape(-1) for p in parts]))
            self.o_bias = _f32(tensors[n["o_bias"]]) if self.output_biased else None
        if self.qk_norm_eps is not None:
            self.q_gain = tensors[n["q_norm"]]
            self.k_gain = None if self.borrows else tensors[n["k_norm"]]

    def _project_wide(self, x, ctx, cache, t, cos, sin, rot_dim):
        """q (and k, v) through memory, then the finishing kernel that takes any head sizes."""
        qkv = self.rt.rows(t, self.w_qkv.shape[0])
        if isinstance(x, NormedRows):
            x.linear(self.w_qkv, qkv, K.EPILOGUE_STORE, self.rt.err)
        else:
            K.gemm_nt(x, self.w_qkv, qkv, err=self.rt.err)
        q = self.rt.rows(t, self.nq * self.pad)
        K.qkv_finish(qkv, q, cache.pages, self.q_gain, self.k_gain, cos, sin, ctx.positions, ctx.token_slot,
                     cache.block_table, self.nq, self.nkv, self.d, self.dv, self.pad, rot_dim,
                     self.qk_norm_eps or 0.0, self.scope == "projection", not self.borrows,
                     bool(cache.writes) and not self.borrows, self.rt.err, bias=self.qkv_bias, q_temp=self.q_temp)
        return q

    def output_bias(self):
        return self.o_bias

    def forward(self, x, ctx, cache, residual, overwrite=False):
        nq, nkv, d = self.nq, self.nkv, self.pad
        t = residual.shape[0]
        rot = self.position.rotary()
        cos, sin, rot_dim = rot if rot is not None else (None, None, 0)
        if self.wide:
            if rot_dim and self.position.rotary_interleaved:
                raise ValueError("rotation of neighbouring pairs is not available with padded heads")
            q = self._project_wide(x, ctx, cache, t, cos, sin, rot_dim)
            return self._attend(q, ctx, cache, residual, t, overwrite)
        q = self.rt.rows(t, nq * d)
        heads = (q, cache.pages, self.q_gain, self.k_gain, cos, sin, ctx.positions, ctx.token_slot,
                 cache.block_table, nq, nkv, d, rot_dim, self.qk_norm_eps or 0.0, cache.writes, self.rt.err)
        interleaved = bool(rot_dim and self.position.rotary_interleaved)
        # few tokens: the product finishes its heads itself (norm, rotation, cache write); else
        # the projection goes through memory and a second kernel does that
        fused = False
        if t <= K.FEW_TOKENS and not self.exact and not interleaved:
            # (the product that finishes its heads knows the norm over the whole row only)
            pending = isinstance(x, NormedRows) and x.pending() and x.groups == 1
            fused = K.gemm_nt_tc_qkv_heads(None if pending else (x.materialize() if isinstance(x, NormedRows) else x),
                                           self.w_qkv, *heads,
                                           normed=(x.h, x.gain, x.eps, x.row_index) if pending else None)
        if not fused:
            qkv = self.rt.rows(t, (nq + 2 * nkv) * d)
            if isinstance(x, NormedRows):
                x.linear(self.w_qkv, qkv, K.EPILOGUE_STORE, self.rt.err)
            else:
                K.gemm_nt(x, self.w_qkv, qkv, err=self.rt.err)
            K.qk_norm_rope_store(qkv, *heads, interleaved=interleaved)
        self._attend(q, ctx, cache, residual, t, overwrite)

    def _attend(self, q, ctx, cache, residual, t, overwrite=False):
        attn = attend(self.rt, q, ctx, cache, self.nq, self.nkv, self.pad, self.mask, self.scale, self.exact,
                      self.extras)
        if overwrite:
            K.gemm_nt(attn, self.w_o, residual, K.EPILOGUE_STORE, err=self.rt.err)
            return
        K.gemm_nt(attn, self.w_o, residual, K.EPILOGUE_RESIDUAL, err=self.rt.err)
        if self.o_bias is not None:
            K.row_bias(residual, self.o_bias, add=True)


@register_part("mixer", "gqa_attention")
def _build(spec, runtime, position=None, **_):
    return GQAttention(spec["hidden_size"], spec["num_heads"], spec["num_kv_heads"], spec["head_dim"],
                       spec["scale"], spec.get("window", 0), spec.get("qk_norm_eps"), position, runtime,
                       value_dim=spec.get("value_dim"), qk_norm_scope=spec.get("qk_norm_scope", "head"),
                       borrows_kv=spec.get("borrows_kv", False), names=spec.get("names"),
                       bias=spec.get("bias", False), q_temp=spec.get("q_temp"), score_bias=spec.get("score_bias"),
                       sink=spec.get("sink", False), value_from_key=spec.get("value_from_key", False),
                       chunk=spec.get("chunk", 0), softcap=spec.get("softcap", 0.0))
