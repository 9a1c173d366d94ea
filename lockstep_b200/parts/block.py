"""Arrangement of a layer's parts.  "pre_norm":
h += mixer(norm_a(h)); h += feed_forward(norm_b(h))  (LockStep: engine/model/qwen3.py:242-287).
The names under which the layer's tensors are stored are parameters of the
arrangement, so the same arrangement serves architectures that name them otherwise.
A layer whose feed-forward is of kind "none" is its mixer alone.

"sandwich_norm": a norm after each sublayer as well as before it,
h += norm_c(mixer(norm_a(h))); h += norm_d(feed_forward(norm_b(h))).  The norms after the sublayers are the
``LayerSpec.extra`` parts "mixer_post_norm" and "feed_forward_post_norm" (norms with ``accumulate``); a sublayer
stores its result in a float32 buffer and the norm's kernel adds the normed rows to the stream, or, where the
mixer closes with a kernel of its own that can take the norm along (``Mixer.accepts_post_norm``), that kernel does.

"shared_norm": one norm feeds the mixer and the feed-forward side by side,
h += mixer(y) + feed_forward(y) with y = norm(h).  Two options, each with tensors of the layer:
- ``shift``: the mixer reads y_t + (y_(t-1) - y_t) * mix instead of y_t (``mix`` one number per
  coordinate; zeros stand for the row before a sequence's first).  The last y of a request is part
  of what it keeps between steps: the layer's cache need is its mixer's and a state of one row.
- ``gates``: each sublayer's result is multiplied, coordinate by coordinate, by
  sigmoid(W y + b) with a matrix and a bias of its own (both gates are one product of y).
The feed-forward always reads y itself."""

from __future__ import annotations

import torch

from .. import kernels as K
from ..config.spec import own_tensors, tensor_name
from .base import Block, CacheNeed, Runtime, WeightSpec, build_part, register_part, side_stream
from .norm import RMSNorm

_DEFAULT_NAMES = {
    "mixer_norm": "input_layernorm",
    "mixer": "self_attn",
    "feed_forward_norm": "post_attention_layernorm",
    "feed_forward": "mlp",
}


class PreNormBlock(Block):
    def __init__(self, layer_spec, runtime: Runtime):
        names = dict(_DEFAULT_NAMES)
        names.update(layer_spec.block.get("names", {}) or {})
        self.names = names
        self.position = build_part("position", layer_spec.position, runtime)
        self.mixer_norm = build_part("norm", layer_spec.mixer_norm, runtime)
        self.mixer = build_part("mixer", layer_spec.mixer, runtime, position=self.position)
        self.feed_forward_norm = self.feed_forward = None
        if layer_spec.feed_forward.kind != "none":
            self.feed_forward_norm = build_part("norm", layer_spec.feed_forward_norm, runtime)
            self.feed_forward = build_part("feed_forward", layer_spec.feed_forward, runtime)

    def _children(self):
        return [(self.names[k], getattr(self, k)) for k in _DEFAULT_NAMES if getattr(self, k) is not None]

    def cache_need(self):
        return self.mixer.cache_need()

    @property
    def graph_safe(self):
        return all(part.graph_safe for _, part in self._children()) and self.position.graph_safe

    def attention_windows(self):
        return set().union(*(part.attention_windows() for _, part in self._children()))

    def weight_specs(self):
        out = {}
        for name, part in self._children():
            for local, spec in part.weight_specs().items():
                out[tensor_name(name, local)] = spec
        return out

    def bind(self, tensors):
        for name, part in self._children():
            own = own_tensors(name, tensors)
            if own or part.weight_specs():
                part.bind(own)

    @staticmethod
    def _normed(norm, consumer, h):
        """Rows for ``consumer``: still to be normalised where it can fuse the norm, else the tensor."""
        if consumer.accepts_normed_rows and hasattr(norm, "lazy"):
            return norm.lazy(h)
        return norm.forward(h)

    def _mix(self, h, ctx, cache):
        self.mixer.forward(self._normed(self.mixer_norm, self.mixer, h), ctx, cache, h)

    def _feed_forward(self, h, ctx, cache):
        self.feed_forward.forward(self._normed(self.feed_forward_norm, self.feed_forward, h), ctx, h)

    def steps(self):
        out = [(bool(self.mixer_norm.graph_safe and self.mixer.graph_safe and self.position.graph_safe), self._mix)]
        if self.feed_forward is not None:
            out.append((bool(self.feed_forward_norm.graph_safe and self.feed_forward.graph_safe), self._feed_forward))
        return out

    def forward(self, h, ctx, cache):
        self._mix(h, ctx, cache)
        if self.feed_forward is not None:
            self._feed_forward(h, ctx, cache)


@register_part("block", "pre_norm")
def _build(spec, runtime, layer_spec=None, **_):
    return PreNormBlock(layer_spec, runtime)


class SandwichNormBlock(PreNormBlock):
    def __init__(self, layer_spec, runtime: Runtime):
        super().__init__(layer_spec, runtime)
        self.rt = runtime
        self.names.setdefault("mixer_post_norm", "post_attention_norm")
        self.names.setdefault("feed_forward_post_norm", "post_mlp_norm")
        self.mixer_post_norm = build_part("norm", layer_spec.extra["mixer_post_norm"], runtime)
        self.feed_forward_post_norm = None
        if self.feed_forward is not None:
            self.feed_forward_post_norm = build_part("norm", layer_spec.extra["feed_forward_post_norm"], runtime)
        for post in (self.mixer_post_norm, self.feed_forward_post_norm):
            if post is not None and not hasattr(post, "accumulate"):
                raise ValueError("sandwich_norm: the norm after a sublayer must be able to add its result to the stream")

    def _children(self):
        keys = list(_DEFAULT_NAMES) + ["mixer_post_norm", "feed_forward_post_norm"]
        return [(self.names[k], getattr(self, k)) for k in keys if getattr(self, k) is not None]

    def _sublayer(self, part, post, x, h, ctx, cache=None):
        args = (x, ctx, cache) if cache is not None else (x, ctx)
        if getattr(part, "accepts_post_norm", False):
            part.forward(*args, h, post_norm=post)
            return
        out = self.rt.rows(h.shape[0], h.shape[1], dtype=torch.float32)
        if part.can_overwrite:
            part.forward(*args, out, overwrite=True)
        else:
            K.row_bias(out, None)
            part.forward(*args, out)
        post.accumulate(h, out)

    def _mix(self, h, ctx, cache):
        self._sublayer(self.mixer, self.mixer_post_norm, self._normed(self.mixer_norm, self.mixer, h), h, ctx, cache)

    def _feed_forward(self, h, ctx, cache):
        self._sublayer(self.feed_forward, self.feed_forward_post_norm,
                       self._normed(self.feed_forward_norm, self.feed_forward, h), h, ctx)


@register_part("block", "sandwich_norm")
def _build_sandwich(spec, runtime, layer_spec=None, **_):
    return SandwichNormBlock(layer_spec, runtime)


_SHARED_NAMES = {"norm": "norm", "mixer": "mixer", "feed_forward": "mlp", "shift": "shift",
                 "mixer_gate": "mixer_gate", "mixer_gate_bias": "mixer_gate.bias",
                 "feed_forward_gate": "mlp_gate", "feed_forward_gate_bias": "mlp_gate.bias"}


class SharedNormBlock(Block):
    def __init__(self, layer_spec, runtime: Runtime):
        b = layer_spec.block
        self.names = dict(_SHARED_NAMES)
        self.names.update(b.get("names", {}) or {})
        self.rt, self.width = runtime, int(b["hidden_size"])
        self.shift, self.gates = bool(b.get("shift", False)), bool(b.get("gates", False))
        self.position = build_part("position", layer_spec.position, runtime)
        self.norm = build_part("norm", layer_spec.mixer_norm, runtime)
        self.mixer = build_part("mixer", layer_spec.mixer, runtime, position=self.position)
        self.feed_forward = None
        if layer_spec.feed_forward.kind != "none":
            self.feed_forward = build_part("feed_forward", layer_spec.feed_forward, runtime)
        self.mix = self.w_gates = self.b_gates = None
        self._side = None          # streams of the feed-forward and of the gates' product in steps of few tokens

    def _children(self):
        out = [(self.names["norm"], self.norm), (self.names["mixer"], self.mixer)]
        if self.feed_forward is not None:
            out.append((self.names["feed_forward"], self.feed_forward))
        return out

    def _sublayers(self):
        return ["mixer"] + (["feed_forward"] if self.feed_forward is not None else [])

    def cache_need(self):
        need = self.mixer.cache_need()
        if not self.shift:
            return need
        return CacheNeed("several", parts=(need, CacheNeed("state", state_shape=(self.width,),
                                                           state_dtype=torch.float32)))

    @property
    def graph_safe(self):
        return all(part.graph_safe for _, part in self._children()) and self.position.graph_safe

    def attention_windows(self):
        return set().union(*(part.attention_windows() for _, part in self._children()))

    def weight_specs(self):
        out, n, w = {}, self.names, self.width
        for name, part in self._children():
            for local, spec in part.weight_specs().items():
                out[tensor_name(name, local)] = spec
        if self.shift:
            out[n["shift"]] = WeightSpec((w,), "gain", ("uniform", 0.0, 1.0))
        if self.gates:
            for sub in self._sublayers():
                out[n[sub + "_gate"]] = WeightSpec((w, w))
                out[n[sub + "_gate_bias"]] = WeightSpec((w,), "gain", ("normal", 0.0, 0.5))
        return out

    def bind(self, tensors):
        n = self.names
        for name, part in self._children():
            own = own_tensors(name, tensors)
            if own or part.weight_specs():
                part.bind(own)
        if self.shift:
            self.mix = tensors[n["shift"]].to(torch.float32).reshape(1, self.width).contiguous()
        if self.gates:
            subs = self._sublayers()
            self.w_gates = torch.cat([tensors[n[s + "_gate"]] for s in subs], dim=0).contiguous()
            self.b_gates = torch.cat([tensors[n[s + "_gate_bias"]] for s in subs]).to(torch.float32).contiguous()

    def forward(self, h, ctx, cache):
        rt, t, w = self.rt, h.shape[0], self.width
        mixer_cache, carried = (cache.parts[0], cache.parts[1].state) if self.shift else (cache, None)
        if self.shift and isinstance(self.norm, RMSNorm) and self.norm.groups == 1:
            # the norm and the shift in one pass over the rows (the bits of the two kernels in turn)
            y, x = rt.rows(t, w), rt.rows(t, w)
            K.rmsnorm_shift(h, self.norm.gain, self.norm.eps, self.mix, carried, ctx.token_slot, y, x)
        else:
            x = y = self.norm.forward(h)
            if self.shift:
                x = rt.rows(t, w)
                K.shift_mix(y, self.mix, carried, 0, ctx.token_slot, x.view(1, t, w))
        subs = self._sublayers()
        out = rt.rows(len(subs) * t, w, dtype=torch.float32).view(len(subs), t, w)
        stores = self.mixer.can_overwrite and (self.feed_forward is None or self.feed_forward.can_overwrite)
        if not stores:
            K.row_bias(out.view(len(subs) * t, w), None)
        z = rt.rows(t, len(subs) * w, dtype=torch.float32) if self.gates else None
        beside = stores and t <= K.FEW_TOKENS and rt.options.get("branch_streams", True) \
            and (self.feed_forward is not None or self.gates)
        if beside:
            # a step of few tokens is a chain of launches of a handful of blocks each: the feed-forward and the
            # gates' product run on streams of their own beside the mixer (in a recorded step: branches of the
            # graph) and meet it again before the closing kernel
            main = torch.cuda.current_stream()
            if self._side is None:
                self._side = [side_stream(rt.device, 0), side_stream(rt.device, 1)]
            work = []
            if self.feed_forward is not None:
                work.append(lambda: self.feed_forward.forward(y, ctx, out[1], overwrite=True))
            if self.gates:
                work.append(lambda: K.gemm_nt(y, self.w_gates, z, err=rt.err))
            for side, fn in zip(self._side, work):
                side.wait_stream(main)                 # y and what came before it
                with torch.cuda.stream(side):
                    fn()
            self.mixer.forward(x, ctx, mixer_cache, out[0], overwrite=True)
            for side, _ in zip(self._side, work):
                main.wait_stream(side)
        else:
            if stores:
                self.mixer.forward(x, ctx, mixer_cache, out[0], overwrite=True)
                if self.feed_forward is not None:
                    self.feed_forward.forward(y, ctx, out[1], overwrite=True)
            else:
                self.mixer.forward(x, ctx, mixer_cache, out[0])
                if self.feed_forward is not None:
                    self.feed_forward.forward(y, ctx, out[1])
            if self.gates:
                K.gemm_nt(y, self.w_gates, z, err=rt.err)
        # the closing kernel: the (gated) sum into the residual stream, and the last row of every
        # request's portion into its slot for the next step's shift
        K.gated_sum(h, out, z, self.b_gates, carry=(y, carried, ctx.token_slot) if self.shift else None)


@register_part("block", "shared_norm")
def _build_shared_norm(spec, runtime, layer_spec=None, **_):
    return SharedNormBlock(layer_spec, runtime)
