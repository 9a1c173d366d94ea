"""SwiGLU feed-forward: down(silu(gate(x)) * up(x)), no biases, added into the
residual stream (LockStep: engine/model/qwen3.py:285-287, engine/kernels/swiglu.py:25-29).
gate and up are one product over the row-concatenated weights, with the
activation in that product's epilogue."""

from __future__ import annotations

import torch

from .. import kernels as K
from .base import FeedForward, Runtime, WeightSpec, register_part
from .norm import NormedRows


class SwiGLU(FeedForward):
    graph_safe = True
    accepts_normed_rows = True

    def __init__(self, hidden_size: int, intermediate_size: int, runtime: Runtime):
        self.h, self.i, self.rt = int(hidden_size), int(intermediate_size), runtime
        self.w_gate_up = self.w_down = None

    def weight_specs(self):
        return {
            "gate_proj.weight": WeightSpec((self.i, self.h)),
            "up_proj.weight": WeightSpec((self.i, self.h)),
            "down_proj.weight": WeightSpec((self.h, self.i)),
        }

    def bind(self, tensors):
        self.w_gate_up = torch.cat([tensors["gate_proj.weight"], tensors["up_proj.weight"]], dim=0).contiguous()
        self.w_down = tensors["down_proj.weight"]

    def forward(self, x, ctx, residual):
        act = self.rt.rows(residual.shape[0], self.i)
        if isinstance(x, NormedRows):
            x.linear(self.w_gate_up, act, K.EPILOGUE_SILU_MUL, self.rt.err)
        else:
            K.gemm_nt(x, self.w_gate_up, act, K.EPILOGUE_SILU_MUL, err=self.rt.err)
        K.gemm_nt(act, self.w_down, residual, K.EPILOGUE_RESIDUAL, err=self.rt.err)


class ClampedGLU(FeedForward):
    """down(g sigmoid(alpha g) (u + 1)) with g = min(gate(x), limit), u = clamp(up(x), -limit, limit); all three
    projections may have biases.  gate and up are one product with a float32 result; the activation kernel adds
    their biases, and the down projection's bias into the residual stream, where the product then adds itself."""

    graph_safe = True
    accepts_normed_rows = True

    def __init__(self, hidden_size: int, intermediate_size: int, limit: float, alpha: float, bias: bool,
                 runtime: Runtime, names=None):
        self.h, self.i, self.rt = int(hidden_size), int(intermediate_size), runtime
        self.limit, self.alpha, self.bias = float(limit), float(alpha), bool(bias)
        self.names = {"gate": "gate", "up": "up", "down": "down", "gate_bias": "gate.b", "up_bias": "up.b",
                      "down_bias": "down.b"}
        self.names.update(names or {})
        self.w_gate_up = self.w_down = self.b_gate_up = self.b_down = None

    def weight_specs(self):
        n = self.names
        specs = {n["gate"]: WeightSpec((self.i, self.h)), n["up"]: WeightSpec((self.i, self.h)),
                 n["down"]: WeightSpec((self.h, self.i))}
        if self.bias:
            small = ("normal", 0.0, 0.02)
            specs.update({n["gate_bias"]: WeightSpec((self.i,), "gain", small), n["up_bias"]: WeightSpec((self.i,), "gain", small),
                          n["down_bias"]: WeightSpec((self.h,), "gain", small)})
        return specs

    def bind(self, tensors):
        n = self.names
        self.w_gate_up = torch.cat([tensors[n["gate"]], tensors[n["up"]]], dim=0).contiguous()
        self.w_down = tensors[n["down"]]
        if self.bias:
            self.b_gate_up = torch.cat([tensors[n["gate_bias"]], tensors[n["up_bias"]]]).to(torch.float32).contiguous()
            self.b_down = tensors[n["down_bias"]].to(torch.float32).contiguous()

    def forward(self, x, ctx, residual):
        rows = residual.shape[0]
        gate_up = self.rt.rows(rows, 2 * self.i, dtype=torch.float32)
        if isinstance(x, NormedRows):
            x.linear(self.w_gate_up, gate_up, K.EPILOGUE_STORE, self.rt.err)
        else:
            K.gemm_nt(x, self.w_gate_up, gate_up, K.EPILOGUE_STORE, err=self.rt.err)
        act = self.rt.rows(rows, self.i)
        K.clamped_glu(gate_up, self.b_gate_up, act, self.limit, self.alpha,
                      residual if self.bias else None, self.b_down)
        K.gemm_nt(act, self.w_down, residual, K.EPILOGUE_RESIDUAL, err=self.rt.err)


class GatedUnit(FeedForward):
    """down(act(gate(x)) * up(x)) without biases, ``activation`` "gelu_tanh" (0.5 z (1 + tanh(sqrt(2 / pi) (z +
    0.044715 z^3)))) or "silu".  gate and up are one product with a float32 result, the activation a kernel."""

    graph_safe = True
    accepts_normed_rows = True
    can_overwrite = True

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str, runtime: Runtime, names=None):
        if activation not in ("gelu_tanh", "silu"):
            raise ValueError(f"gated_unit: activation {activation!r} is not known (gelu_tanh, silu)")
        self.h, self.i, self.activation, self.rt = int(hidden_size), int(intermediate_size), activation, runtime
        self.names = {"gate": "gate", "up": "up", "down": "down"}
        self.names.update(names or {})
        self.w_gate_up = self.w_down = None

    def weight_specs(self):
        n = self.names
        return {n["gate"]: WeightSpec((self.i, self.h)), n["up"]: WeightSpec((self.i, self.h)),
                n["down"]: WeightSpec((self.h, self.i))}

    def bind(self, tensors):
        n = self.names
        self.w_gate_up = torch.cat([tensors[n["gate"]], tensors[n["up"]]], dim=0).contiguous()
        self.w_down = tensors[n["down"]]

    def forward(self, x, ctx, residual, overwrite=False):
        rows = residual.shape[0]
        gate_up = self.rt.rows(rows, 2 * self.i, dtype=torch.float32)
        if isinstance(x, NormedRows):
            x.linear(self.w_gate_up, gate_up, K.EPILOGUE_STORE, self.rt.err)
        else:
            K.gemm_nt(x, self.w_gate_up, gate_up, K.EPILOGUE_STORE, err=self.rt.err)
        act = self.rt.rows(rows, self.i)
        K.clamped_glu(gate_up, None, act, float("inf"), 1.0, up_offset=0.0, gelu=self.activation == "gelu_tanh")
        K.gemm_nt(act, self.w_down, residual, K.EPILOGUE_STORE if overwrite else K.EPILOGUE_RESIDUAL, err=self.rt.err)


@register_part("feed_forward", "gated_unit")
def _build_gated_unit(spec, runtime, **_):
    return GatedUnit(spec["hidden_size"], spec["intermediate_size"], spec.get("activation", "gelu_tanh"), runtime,
                     names=spec.get("names"))


@register_part("feed_forward", "clamped_glu")
def _build_clamped_glu(spec, runtime, **_):
    return ClampedGLU(spec["hidden_size"], spec["intermediate_size"], spec["limit"], spec.get("alpha", 1.702),
                      spec.get("bias", True), runtime, names=spec.get("names"))


@register_part("feed_forward", "swiglu")
def _build(spec, runtime, **_):
    return SwiGLU(spec["hidden_size"], spec["intermediate_size"], runtime)
