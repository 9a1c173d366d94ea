"""Attention over a cached latent.

Per token the layer caches one small vector c (``kv_rank`` elements, RMS-normed with a gain of its
own) and one rotated key part (``rot_dim`` elements) that all heads share, instead of keys and
values per head.  With q_h = [q_plain,h (``head_dim``) ; q_rot,h (``rot_dim``)] per query head:

    key of head h = [W_uk,h c ; k_rot],   value of head h = W_uv,h c,
    score = (q_plain,h . W_uk,h c + q_rot,h . k_rot) * scale.

Since q_plain,h . (W_uk,h c) = (W_uk,h^T q_plain,h) . c, the attention kernels are given one key head
[c ; k_rot] (padded to a multiple of 16) that every query head reads, queries
[W_uk,h^T q_plain,h ; q_rot,h], and values [c ; 0]; the head's output, a weighted sum of latents, then
goes through W_uv,h.  A prompt's tokens and a decoded token take the same path, so a row does not
depend on how its request was cut.  Rotation is the position encoding's (its tables; neighbouring
pairs or halves), a window and a sink per head are optional.

``q_rank``: the queries go through a latent of their own, q = W_uq norm(W_dq x) with an RMSNorm (a gain
per element) between the two maps (``names``: ``q_down``, ``q_norm``, ``q_up``), instead of one matrix ``q``.
``borrows_kv``: the layer has no down-projection of its own; the schedule gives it the cached latents and
rotated key parts of another layer, which it reads with its own W_uk, W_uv, queries and scale.

Kernels: one product for the queries' and the latent's projections, ``latent_finish`` (norm,
rotation, cache write), ``heads_product`` (the two per-head products), the engine's attention
kernels over the paged cache, the output product (csrc/latent.cu, csrc/attention_simt.cu).
"""

from __future__ import annotations

import torch

from .. import kernels as K
from .attention import ScoreExtras, attend
from .base import CacheNeed, Mixer, PositionEncoding, Runtime, WeightSpec, register_part
from .norm import NormedRows

_DEFAULT_NAMES = {"q": "q", "down": "dkv", "down_norm": "dkv.norm", "up_k": "uk", "up_v": "uv", "o": "o",
                  "sink": "sink", "q_down": "dq", "q_norm": "dq.norm", "q_up": "uq"}


class LatentAttention(Mixer):
    graph_safe = True
    accepts_normed_rows = True
    can_overwrite = True

    def __init__(self, hidden_size, num_heads, head_dim, rot_dim, value_dim, kv_rank, scale, window, norm_eps,
                 position: PositionEncoding, runtime: Runtime, sink=False, names=None, q_rank=None, borrows_kv=False):
        self.w, self.H, self.d, self.dr = int(hidden_size), int(num_heads), int(head_dim), int(rot_dim)
        self.dv, self.rank = int(value_dim), int(kv_rank)
        self.q_rank, self.borrows = int(q_rank or 0), bool(borrows_kv)
        self.scale, self.window, self.eps = float(scale), int(window or 0), float(norm_eps)
        self.sink, self.position, self.rt = bool(sink), position, runtime
        self.pad = -(-(self.rank + self.dr) // 16) * 16          # the one head size the attention kernels see
        if not 16 <= self.pad <= 256:
            raise ValueError(f"kv_rank + rot_dim = {self.rank + self.dr} is not supported: the attention kernels "
                             "take heads of up to 256 elements")
        rot = position.rotary() if position is not None else None
        if self.dr and (rot is None or rot[2] != self.dr):
            raise ValueError("the position encoding must rotate exactly the rot_dim part of a head")
        self.names = dict(_DEFAULT_NAMES)
        self.names.update(names or {})
        self.exact = runtime.dtype == torch.float32
        self.extras = ScoreExtras()

    def cache_need(self):
        return CacheNeed("paged_kv", kv_heads=1, head_dim=self.pad, window=self.window)

    def attention_windows(self):
        return {self.window}

    def weight_specs(self):
        n, H = self.names, self.H
        specs = {n["up_k"]: WeightSpec((H * self.d, self.rank)),
                 n["up_v"]: WeightSpec((H * self.dv, self.rank)),
                 n["o"]: WeightSpec((self.w, H * self.dv))}
        if self.q_rank:
            specs.update({n["q_down"]: WeightSpec((self.q_rank, self.w)), n["q_norm"]: WeightSpec((self.q_rank,), "gain"),
                          n["q_up"]: WeightSpec((H * (self.d + self.dr), self.q_rank))})
        else:
            specs[n["q"]] = WeightSpec((H * (self.d + self.dr), self.w))
        if not self.borrows:
            specs.update({n["down"]: WeightSpec((self.rank + self.dr, self.w)),
                          n["down_norm"]: WeightSpec((self.rank,), "gain")})
        if self.sink:
            specs[n["sink"]] = WeightSpec((H,), "gain", ("normal", 0.0, 1.0))
        return specs

    def bind(self, t):
        n, H = self.names, self.H
        # one product for what reads the mixer's input: the queries and, where the layer makes them itself, the
        # latent and the shared key part.  Queries through a latent of their own: that latent is a product of
        # its own with a float32 result, which its norm reads as it is.
        self.w_in = None
        if self.q_rank:
            self.w_q_down, self.q_gain, self.w_q_up = t[n["q_down"]].contiguous(), t[n["q_norm"]], t[n["q_up"]].contiguous()
            if not self.borrows:
                self.w_in = t[n["down"]].contiguous()
        else:
            self.w_in = t[n["q"]].contiguous() if self.borrows else torch.cat([t[n["q"]], t[n["down"]]], dim=0).contiguous()
        self.gain = None if self.borrows else t[n["down_norm"]]
        # W_uk per head, transposed: [H, rank, d], so that the fold is a product with rows of weights
        self.w_fold = t[n["up_k"]].view(H, self.d, self.rank).transpose(1, 2).contiguous()
        self.w_up_v = t[n["up_v"]].view(H, self.dv, self.rank).contiguous()
        self.w_o = t[n["o"]]
        if self.sink:
            self.extras = ScoreExtras(sinks=t[n["sink"]].to(torch.float32).contiguous())

    def forward(self, x, ctx, cache, residual, overwrite=False):
        rt, t, H = self.rt, residual.shape[0], self.H
        if self.borrows == bool(cache.writes):
            raise ValueError("a latent layer writes the cache entry it is given exactly when it has a "
                             "down-projection of its own")
        proj = None
        if self.w_in is not None:
            proj = rt.rows(t, self.w_in.shape[0])
            if isinstance(x, NormedRows) and not self.q_rank:
                x.linear(self.w_in, proj, K.EPILOGUE_STORE, rt.err)
            else:
                x = x.materialize() if isinstance(x, NormedRows) else x
                K.gemm_nt(x, self.w_in, proj, err=rt.err)
        if self.q_rank:
            x = x.materialize() if isinstance(x, NormedRows) else x
            raw = rt.rows(t, self.q_rank, dtype=torch.float32)
            K.gemm_nt(x, self.w_q_down, raw, err=rt.err)
            queries = rt.rows(t, H * (self.d + self.dr))
            # (few tokens: the second map's product norms its rows itself, with the bits of the separate kernel)
            if not K.gemm_nt_tc_rmsnorm(raw, self.q_gain, self.eps, self.w_q_up, queries, K.EPILOGUE_STORE, rt.err):
                cq = rt.rows(t, self.q_rank)
                K.rmsnorm(raw, self.q_gain, cq, self.eps, rt.err)
                K.gemm_nt(cq, self.w_q_up, queries, err=rt.err)
            kv = proj
        else:
            queries, kv = proj, None if self.borrows else proj[:, H * (self.d + self.dr):]
        rot = self.position.rotary() if self.dr else None
        cos, sin, _ = rot if rot is not None else (None, None, 0)
        q = rt.rows(t, H * self.pad)
        # few tokens: the finishing kernel folds W_uk into the queries itself (the same bits, a launch fewer)
        few = t <= K.FEW_TOKENS and H * self.d * 4 <= 40 * 1024
        K.latent_finish(queries, q, cache.pages, self.gain, cos, sin, ctx.positions, ctx.token_slot, cache.block_table,
                        H, self.d, self.dr, self.rank, self.pad, self.eps,
                        bool(self.dr and self.position.rotary_interleaved), bool(cache.writes), rt.err,
                        w_fold=self.w_fold if few else None, kv=kv)
        if not few:
            K.heads_product(queries, self.d + self.dr, self.w_fold, q, self.pad)
        attn = attend(rt, q, ctx, cache, H, 1, self.pad, self.window, self.scale, self.exact, self.extras)
        y = rt.rows(t, H * self.dv)
        K.heads_product(attn, self.pad, self.w_up_v, y, self.dv)
        K.gemm_nt(y, self.w_o, residual, K.EPILOGUE_STORE if overwrite else K.EPILOGUE_RESIDUAL, err=rt.err)


@register_part("mixer", "latent_attention")
def _build(spec, runtime, position=None, **_):
    return LatentAttention(spec["hidden_size"], spec["num_heads"], spec["head_dim"], spec["rot_dim"],
                           spec["value_dim"], spec["kv_rank"], spec["scale"], spec.get("window", 0), spec["norm_eps"],
                           position, runtime, sink=spec.get("sink", False), names=spec.get("names"),
                           q_rank=spec.get("q_rank"), borrows_kv=spec.get("borrows_kv", False))
