"""Mixers side by side: several mixers read the same normed rows, and the layer adds
sum_b scale_b * mixer_b(x) to the residual stream.

``branches``: a list of {"name": tensor-name prefix under the mixer's own, "mixer": PartSpec,
"position": PartSpec or None, "scale": number}.  Each branch keeps a cache of its own (pages or
a state slot): the part's need is the branches' needs side by side.  A branch adds its result
into a zeroed float32 buffer of its own as it would into the residual stream (so any registered
mixer can be a branch); one kernel then adds the weighted buffers to the residual stream.  Where
every branch can store its result instead (``Mixer.can_overwrite``) nothing is zeroed, and the
branches' output biases, weighted and summed once when the weights arrive, ride on that kernel.
``branch_norm`` = {"eps", "tensor"}: every branch's result is first divided by its root mean square over the
model width and multiplied by a gain of its own (stored as ``<branch name>.<tensor>``), then weighted and
summed; the closing kernel can also put that sum through the layer's norm after the mixer (``post_norm``, a layer
norm handed in by the block arrangement) before it adds it to the residual stream.
In a step of few tokens, where every kernel is a handful of blocks and the step is a chain of
launches, the branches after the first run on streams of their own beside it (in a recorded
step: branches of the graph) and meet again before the weighted sum.
"""

from __future__ import annotations

import torch

from .. import kernels as K
from ..config.spec import PartSpec, own_tensors, tensor_name
from .base import CacheNeed, Mixer, Runtime, build_part, register_part


class ParallelMixers(Mixer):
    def __init__(self, hidden_size, branches, runtime: Runtime, branch_norm=None):
        self.branch_norm = dict(branch_norm) if branch_norm else None
        self.branch_gain = None
        if not 1 <= len(branches) <= 4:
            raise ValueError("one to four mixers can run side by side")
        self.w, self.rt = int(hidden_size), runtime
        self.names, self.scales, self.mixers = [], [], []
        self._side = None          # streams of the branches after the first, made at first use
        for b in branches:
            position = build_part("position", b.get("position") or PartSpec("none"), runtime)
            self.names.append(str(b["name"]))
            self.scales.append(float(b.get("scale", 1.0)))
            self.mixers.append(build_part("mixer", b["mixer"], runtime, position=position))

    @property
    def graph_safe(self):
        return all(m.graph_safe for m in self.mixers)

    def cache_need(self):
        return CacheNeed("several", parts=tuple(m.cache_need() for m in self.mixers))

    def attention_windows(self):
        return set().union(*(m.attention_windows() for m in self.mixers))

    @property
    def accepts_post_norm(self):
        return self.branch_norm is not None

    def weight_specs(self):
        specs = {tensor_name(name, local): spec for name, m in zip(self.names, self.mixers)
                 for local, spec in m.weight_specs().items()}
        if self.branch_norm:
            from .base import WeightSpec
            for name in self.names:
                specs[tensor_name(name, self.branch_norm.get("tensor", "out"))] = WeightSpec((self.w,), "gain")
        return specs

    def bind(self, tensors):
        if self.branch_norm:
            local = self.branch_norm.get("tensor", "out")
            tensors = dict(tensors)
            gains = [tensors.pop(tensor_name(name, local)) for name in self.names]
            self.branch_gain = torch.stack([g.to(torch.float32) for g in gains]).contiguous()
            if len(set(self.scales)) != 1:
                raise ValueError("parallel: normed branches share one weight")
        for name, m in zip(self.names, self.mixers):
            m.bind(own_tensors(name, tensors))
        self.overwrite = all(m.can_overwrite for m in self.mixers)
        self.bias = None
        if self.overwrite:
            for scale, m in zip(self.scales, self.mixers):
                b = m.output_bias()
                if b is not None:
                    term = scale * b.to(torch.float32)
                    self.bias = term if self.bias is None else self.bias + term
            if self.bias is not None:
                self.bias = self.bias.contiguous()

    def _close(self, residual, out, post_norm):
        """The weighted (and, where asked, normed) sum of the branches into the residual stream."""
        if self.branch_norm is None:
            K.weighted_sum(residual, out, self.scales, self.bias if self.overwrite else None)
            return
        post = (post_norm.gain, post_norm.eps) if post_norm is not None else (None, 0.0)
        K.norm_merge_add(residual, out, self.branch_gain, self.scales[0], post[0], float(self.branch_norm["eps"]), post[1])

    def forward(self, x, ctx, cache, residual, post_norm=None):
        n, t = len(self.mixers), residual.shape[0]
        out = self.rt.rows(n * t, self.w, dtype=torch.float32).view(n, t, self.w)
        if self.overwrite:
            if n > 1 and t <= K.FEW_TOKENS and self.rt.options.get("branch_streams", True):
                main = torch.cuda.current_stream()
                if self._side is None:
                    self._side = [torch.cuda.Stream(device=self.rt.device) for _ in self.mixers[1:]]
                for i, side in enumerate(self._side, start=1):
                    side.wait_stream(main)             # x and what came before it
                    with torch.cuda.stream(side):
                        self.mixers[i].forward(x, ctx, cache.parts[i], out[i], overwrite=True)
                self.mixers[0].forward(x, ctx, cache.parts[0], out[0], overwrite=True)
                for side in self._side:
                    main.wait_stream(side)
            else:
                for i, m in enumerate(self.mixers):
                    m.forward(x, ctx, cache.parts[i], out[i], overwrite=True)
            self._close(residual, out, post_norm)
            return
        K.row_bias(out.view(n * t, self.w), None)
        for i, m in enumerate(self.mixers):
            m.forward(x, ctx, cache.parts[i], out[i])
        self._close(residual, out, post_norm)


@register_part("mixer", "parallel")
def _build(spec, runtime, **_):
    return ParallelMixers(spec["hidden_size"], spec["branches"], runtime, branch_norm=spec.get("branch_norm"))
