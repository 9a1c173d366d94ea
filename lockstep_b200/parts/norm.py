"""RMSNorm: y = x * rsqrt(mean(x^2) + eps) * gain, all in float32
(LockStep: engine/kernels/rmsnorm.py:30-38).  ``offset``: the stored tensor is the gain minus
this number (a tensor that holds the gain minus one: offset 1); the sum is made once, in float32, when the
weights arrive.  ``tensor``: the local name of the stored tensor ("weight"; "" where the norm's
own prefix names it).  ``groups`` > 1: the row is cut into that many equal consecutive parts and
each is divided by its own root mean square (the gain still runs over the whole row).  ``scalar``:
the stored gain is one number for all coordinates (a tensor without dimensions).

"layernorm": y = (x - mean) * rsqrt(var + eps) * gain with var the mean of the squared deviations and no bias,
all in float32.  ``accumulate(residual, x)`` adds the norm of float32 rows ``x`` to ``residual`` (a norm that
follows a sublayer)."""

from __future__ import annotations

import torch

from .. import kernels as K
from .base import Norm, Runtime, WeightSpec, register_part


class NormedRows:
    """Rows that are still to be normalised: a mixer or feed-forward that can make the
    norm inside its first product takes ``h``, ``gain`` and ``eps`` from here; any other
    calls ``materialize()`` and gets the tensor ``Norm.forward`` would have returned."""

    def __init__(self, norm: "RMSNorm", h: torch.Tensor, row_index=None):
        self.norm, self.h, self.row_index = norm, h, row_index
        self.gain, self.eps, self.groups = norm.gain, norm.eps, norm.groups
        self._out = None

    def pending(self) -> bool:
        """True while nobody has asked for the normalised tensor (a product may still make it)."""
        return self._out is None

    def materialize(self) -> torch.Tensor:
        if self._out is None:
            self._out = self.norm.forward(self.h, self.row_index)
        return self._out

    def linear(self, w: torch.Tensor, out: torch.Tensor, epilogue: int, err: torch.Tensor) -> None:
        """out = epilogue(norm(h) @ w.T): fused where the kernel allows, else norm, then product."""
        if self._out is None and K.gemm_nt_tc_rmsnorm(self.h, self.gain, self.eps, w, out, epilogue, err,
                                                      self.row_index, self.groups):
            return
        K.gemm_nt(self.materialize(), w, out, epilogue, err=err)


class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, width: int, eps: float, runtime: Runtime, offset: float = 0.0, tensor: str = "weight",
                 groups: int = 1, scalar: bool = False):
        self.width, self.eps, self.rt = int(width), float(eps), runtime
        self.offset, self.tensor, self.groups, self.scalar = float(offset), str(tensor), int(groups), bool(scalar)
        if self.groups < 1 or self.width % self.groups:
            raise ValueError(f"a norm over {self.width} elements cannot be cut into {self.groups} equal parts")
        self.gain: torch.Tensor | None = None

    def weight_specs(self):
        return {self.tensor: WeightSpec(() if self.scalar else (self.width,), "gain",
                                        ("normal", 0.0, 0.1) if self.offset else None)}

    def bind(self, tensors):
        self.gain = tensors[self.tensor]
        if self.scalar:
            # the kernels take a gain per coordinate: the one number, written out once
            self.gain = self.gain.reshape(1).expand(self.width).contiguous()
        if self.offset:
            self.gain = (self.gain.to(torch.float32) + self.offset).contiguous()

    def lazy(self, h, row_index=None) -> NormedRows:
        """The rows of ``h`` to be normalised, for a part that sets ``accepts_normed_rows``."""
        return NormedRows(self, h, row_index)

    def forward(self, h, row_index=None):
        rows = h.shape[0] if row_index is None else row_index.numel()
        out = self.rt.rows(rows, self.width)
        K.rmsnorm(h, self.gain, out, self.eps, self.rt.err, row_index, self.groups)
        return out


@register_part("norm", "rmsnorm")
def _build(spec, runtime, **_):
    return RMSNorm(spec["width"], spec["eps"], runtime, spec.get("offset", 0.0), spec.get("tensor", "weight"),
                   spec.get("groups", 1), spec.get("scalar", False))


class LayerNorm(Norm):
    graph_safe = True

    def __init__(self, width: int, eps: float, runtime: Runtime, tensor: str = "weight"):
        self.width, self.eps, self.rt, self.tensor = int(width), float(eps), runtime, str(tensor)
        self.gain: torch.Tensor | None = None

    def weight_specs(self):
        return {self.tensor: WeightSpec((self.width,), "gain")}

    def bind(self, tensors):
        self.gain = tensors[self.tensor].to(torch.float32).contiguous()

    def forward(self, h, row_index=None):
        rows = h.shape[0] if row_index is None else row_index.numel()
        out = self.rt.rows(rows, self.width)
        K.layernorm(h, self.gain, out, self.eps, self.rt.err, row_index)
        return out

    def accumulate(self, residual, x):
        """residual += norm(x); both float32 [rows, width]."""
        K.norm_merge_add(residual, x.view(1, *x.shape), None, 1.0, self.gain, 0.0, self.eps)


@register_part("norm", "layernorm")
def _build_layernorm(spec, runtime, **_):
    return LayerNorm(spec["width"], spec["eps"], runtime, spec.get("tensor", "weight"))
