"""Parts that feed the embedding's output into the residual stream again, where the schedule says so
(``LayerRun.inject``: say, before the first layer of every pass over layers that run several times).

"concat_projection": h <- W [h ; x0], with x0 the embedding's output for the step's tokens and W [width, 2 width]
(the columns that meet h first).  ``keep`` is called once a step, right after the embedding: it keeps x0, in the
engine's type, in the right half of a buffer of concatenated rows; every run writes the stream into the left half
and takes the product, whose float32 result is the new stream.
"""

from __future__ import annotations

import torch

from .. import kernels as K
from .base import Part, Runtime, WeightSpec, register_part


class ConcatProjection(Part):
    graph_safe = True

    def __init__(self, width: int, runtime: Runtime, tensor: str = "in"):
        self.width, self.rt, self.tensor = int(width), runtime, str(tensor)
        self.weight = None

    def weight_specs(self):
        # near [I ; 0] in the random-weights mode would need a matrix-shaped distribution; N(0, 1 / sqrt(2 width))
        # keeps the stream's size
        return {self.tensor: WeightSpec((self.width, 2 * self.width), "matrix", ("normal", 0.0, (2.0 * self.width) ** -0.5))}

    def bind(self, tensors):
        self.weight = tensors[self.tensor]

    def keep(self, ctx, h: torch.Tensor) -> None:
        rows = self.rt.rows(h.shape[0], 2 * self.width)
        K.rows_cast(h, rows[:, self.width:])
        ctx._injection_rows = rows

    def forward(self, h: torch.Tensor, ctx) -> None:
        rows = ctx._injection_rows
        K.rows_cast(h, rows[:, :self.width])
        K.gemm_nt(rows, self.weight, h, err=self.rt.err)


@register_part("injection", "concat_projection")
def _build(spec, runtime, **_):
    return ConcatProjection(spec["width"], runtime, spec.get("tensor", "in"))
