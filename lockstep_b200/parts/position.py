"""Position encodings.

"rotary": the half-rotation of LockStep (engine/kernels/rope.py:38-56) with
tables cos/sin[pos, i] of angle pos * theta^(-2i/dim), built in float64 on the
host and kept in float32 (engine/model/qwen3.py:117-129).  ``dim`` may be
smaller than the head size; the dimensions past it are left as they are.
"scaled_rotary": rotation with frequencies stretched for contexts longer than the ``original`` one
(the YaRN scheme): with f_i = theta^(-2i/dim) and dim(t) = dim ln(original / (2 pi t)) / (2 ln theta),
lo = max(floor(dim(fast)), 0), hi = min(ceil(dim(slow)), dim - 1), ramp_i = clamp((i - lo) / max(hi - lo,
0.001), 0, 1), the frequency is f_i / factor * ramp_i + f_i (1 - ramp_i), and cosines and sines are
multiplied by 0.1 ln(factor) + 1.  Without ``scaling`` it is the plain rotation.  ``interleaved``: a
pair is elements (2i, 2i + 1) instead of (i, i + dim / 2).
"distance_slopes": no rotation; the score of a query with a key loses slope_h x their distance, slope_h =
2^(-``exponent`` (h + 1) / heads) for head h (``exponent`` 8 unless given).  ``dim``, ``theta``: a rotation besides.
"none": no position encoding.
"""

from __future__ import annotations

import math

import torch

from .base import PositionEncoding, Runtime, register_part


class Rotary(PositionEncoding):
    graph_safe = True

    def __init__(self, dim: int, theta: float, runtime: Runtime):
        if dim % 2:
            raise ValueError(f"rotary dimension must be even, got {dim}")
        self.dim, self.theta = int(dim), float(theta)
        half = self.dim // 2
        exponent = torch.arange(0, half, dtype=torch.float64) * 2.0 / self.dim
        inv_freq = 1.0 / (self.theta ** exponent)
        pos = torch.arange(runtime.max_positions, dtype=torch.float64)
        ang = pos[:, None] * inv_freq[None, :]
        self.cos = ang.cos().to(torch.float32).to(runtime.device).contiguous()
        self.sin = ang.sin().to(torch.float32).to(runtime.device).contiguous()

    def rotary(self):
        return self.cos, self.sin, self.dim


class ScaledRotary(PositionEncoding):
    graph_safe = True

    def __init__(self, dim: int, theta: float, runtime: Runtime, scaling=None, interleaved: bool = False):
        if dim % 2 or dim <= 0:
            raise ValueError(f"rotary dimension must be even and positive, got {dim}")
        self.dim, self.theta = int(dim), float(theta)
        self.rotary_interleaved = bool(interleaved)
        i = torch.arange(self.dim // 2, dtype=torch.float64)
        freq = self.theta ** (-2.0 * i / self.dim)
        magnitude = 1.0
        if scaling:
            factor, original = float(scaling["factor"]), float(scaling["original"])

            def dim_of(turns: float) -> float:
                return self.dim * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.theta))

            lo = max(math.floor(dim_of(float(scaling["fast"]))), 0)
            hi = min(math.ceil(dim_of(float(scaling["slow"]))), self.dim - 1)
            ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
            freq = freq / factor * ramp + freq * (1.0 - ramp)
            magnitude = 0.1 * math.log(factor) + 1.0
        pos = torch.arange(runtime.max_positions, dtype=torch.float64)
        ang = pos[:, None] * freq[None, :]
        self.cos = (ang.cos() * magnitude).to(torch.float32).to(runtime.device).contiguous()
        self.sin = (ang.sin() * magnitude).to(torch.float32).to(runtime.device).contiguous()

    def rotary(self):
        return self.cos, self.sin, self.dim


class DistanceSlopes(PositionEncoding):
    graph_safe = True

    def __init__(self, runtime: Runtime, exponent: float = 8.0, dim: int = 0, theta: float = 10000.0):
        self.exponent, self.rt = float(exponent), runtime
        self.inner = Rotary(dim, theta, runtime) if dim else None

    def rotary(self):
        return self.inner.rotary() if self.inner is not None else None

    def score_slopes(self, num_heads: int):
        s = [2.0 ** (-self.exponent * (h + 1) / num_heads) for h in range(num_heads)]
        return torch.tensor(s, dtype=torch.float64).to(torch.float32).to(self.rt.device).contiguous()


class NoPosition(PositionEncoding):
    graph_safe = True


@register_part("position", "rotary")
def _build_rotary(spec, runtime, **_):
    return Rotary(spec["dim"], spec["theta"], runtime)


@register_part("position", "scaled_rotary")
def _build_scaled_rotary(spec, runtime, **_):
    return ScaledRotary(spec["dim"], spec["theta"], runtime, scaling=spec.get("scaling"),
                        interleaved=spec.get("interleaved", False))


@register_part("position", "distance_slopes")
def _build_slopes(spec, runtime, **_):
    return DistanceSlopes(runtime, spec.get("exponent", 8.0), spec.get("dim", 0), spec.get("theta", 10000.0))


@register_part("position", "none")
def _build_none(spec, runtime, **_):
    return NoPosition()
