"""A feed-forward of routed experts.

Router logits z = W_router x in float32; scores from ``score`` of z ("sigmoid", or "softmax" over all
experts, or "softmax_chosen": the logits themselves, and the weights the softmax over the chosen logits alone); the ``top`` largest scores chosen (ties to the lower index), with ``correction`` after
adding a stored number per expert that only the choice sees; the weight of a chosen expert is its
score (not renormalised).  ``scale`` "input": the weight multiplies what goes into the expert;
"output": what comes out of it.  An expert is down(act(up(.))) without biases, with ``activation``
"relu2" (the square of relu) or "clamped_glu" (gate and up maps, g = min(gate, limit), u =
clamp(up, -limit, limit), g sigmoid(alpha g) (u + 1)) or "swiglu" (silu(gate) up, no clamps).  The last ``identity`` of the router's
outputs are experts without tensors that return their input.  ``shared`` = {"ff", "limit", "gate"}:
one more expert of the same form that every token runs, added with the weight sigmoid(w_g . x)
where ``gate`` is set (else one).  The token's chosen experts are summed in order of rank, the
shared expert last, and added into the residual stream.

On the device: the router's product (the shared expert's gate rides on it as one more row, and the
shared expert's first product as more rows behind it), the choice, a sort of the step's (token, choice) pairs by expert (a counting sort made by one block),
the two products over the sorted rows tile by tile (a tile belongs to one expert), and the sum
(csrc/experts.cu).  Nothing goes through the host, so the part can be recorded in a graph; the
work lists are sized for the worst case, every expert holding a partly filled last tile.
"""

from __future__ import annotations

import torch

from .. import kernels as K
from .base import FeedForward, Runtime, WeightSpec, register_part, side_stream

_DEFAULT_NAMES = {"router": "router", "correction": "correction", "expert": "e{}", "up": "up", "gate": "gate",
                  "down": "down", "shared": "shared", "shared_gate": "shared.sg"}


class RoutedExperts(FeedForward):
    graph_safe = True
    can_overwrite = True

    def __init__(self, hidden_size: int, expert_size: int, experts: int, top: int, runtime: Runtime,
                 score: str = "sigmoid", activation: str = "relu2", scale: str = "input", limit: float = 0.0,
                 alpha: float = 1.702, identity: int = 0, correction: bool = False, shared=None, names=None):
        if score not in ("sigmoid", "softmax", "softmax_chosen") or activation not in ("relu2", "clamped_glu", "swiglu") \
                or scale not in ("input", "output"):
            raise ValueError(f"routed_experts: score {score!r}, activation {activation!r} or scale {scale!r} is not known")
        if experts < 1 or identity < 0 or not 1 <= top <= experts + identity or experts + identity > 512:
            raise ValueError(f"top {top} of {experts} + {identity} experts is not supported (up to 512 experts)")
        self.h, self.f, self.E, self.top, self.rt = int(hidden_size), int(expert_size), int(experts), int(top), runtime
        self.score, self.activation, self.scale = score, activation, scale
        self.limit, self.alpha, self.identity, self.correction = float(limit), float(alpha), int(identity), bool(correction)
        self.glu = activation in ("clamped_glu", "swiglu")
        # "swiglu" is the gated unit without clamps, with the sigmoid's slope 1 and nothing added to u
        self.up_offset = 1.0
        if activation == "swiglu":
            self.limit, self.alpha, self.up_offset = 0.0, 1.0, 0.0
        self.score_mode = {"sigmoid": 0, "softmax": 1, "softmax_chosen": 2}[score]
        if shared and not self.glu:
            raise ValueError("routed_experts: a shared expert takes the gated activation (clamped_glu)")
        self.shared = dict(shared) if shared else None
        self.names = dict(_DEFAULT_NAMES)
        self.names.update(names or {})
        self.w_router = self.w_up = self.w_down = self.bias = None

    def _expert_specs(self, prefix: str, f: int) -> dict:
        n = self.names
        specs = {f"{prefix}.{n['up']}": WeightSpec((f, self.h)), f"{prefix}.{n['down']}": WeightSpec((self.h, f))}
        if self.glu:
            specs[f"{prefix}.{n['gate']}"] = WeightSpec((f, self.h))
        return specs

    def weight_specs(self):
        n = self.names
        specs = {n["router"]: WeightSpec((self.E + self.identity, self.h))}
        if self.correction:
            specs[n["correction"]] = WeightSpec((self.E + self.identity,), "gain", ("normal", 0.0, 0.02))
        for e in range(self.E):
            specs.update(self._expert_specs(n["expert"].format(e), self.f))
        if self.shared:
            specs.update(self._expert_specs(n["shared"], int(self.shared["ff"])))
            if self.shared.get("gate"):
                specs[n["shared_gate"]] = WeightSpec((1, self.h))
        return specs

    def _up(self, t, prefix):
        """An expert's first matrix: with a gated activation the gate rows, then the up rows."""
        n = self.names
        return torch.cat([t[f"{prefix}.{n['gate']}"], t[f"{prefix}.{n['up']}"]], dim=0) if self.glu else t[f"{prefix}.{n['up']}"]

    def bind(self, t):
        n = self.names
        router = [t[n["router"]]]
        if self.shared and self.shared.get("gate"):
            router.append(t[n["shared_gate"]].reshape(1, self.h))        # its logit: one more column of the router's product
        self.shared_at = 0
        if self.shared:
            # the shared expert's first product reads the same rows: it rides on the router's product too, from a
            # column that is a multiple of 8 on (its activation then loads 16 bytes at a time)
            rows = sum(r.shape[0] for r in router)
            self.shared_at = -(-rows // 8) * 8
            router.append(torch.zeros((self.shared_at - rows, self.h), dtype=router[0].dtype, device=router[0].device))
            router.append(self._up(t, n["shared"]))
        self.w_router = torch.cat(router, dim=0).contiguous()
        self.bias = t[n["correction"]].to(torch.float32).contiguous() if self.correction else None
        names = [n["expert"].format(e) for e in range(self.E)]
        self.w_up = torch.stack([self._up(t, p) for p in names]).contiguous()                   # [E, f or 2 f, h]
        self.w_down = torch.stack([t[f"{p}.{n['down']}"] for p in names]).contiguous()          # [E, h, f]
        if self.shared:
            self.w_shared_down = t[f"{n['shared']}.{n['down']}"]

    def _activate(self, wide, rows, f):
        act = self.rt.rows(rows, f)
        K.clamped_glu(wide, None, act, self.limit if self.limit > 0 else float("inf"), self.alpha, up_offset=self.up_offset)
        return act

    def _shared(self, first, tokens):
        """The shared expert on every token, from its columns of the router's product: float32 [tokens, hidden]."""
        rt, f = self.rt, int(self.shared["ff"])
        wide = first[:, self.shared_at:self.shared_at + 2 * f]
        act = rt.rows(tokens, f)
        limit = float(self.shared.get("limit", self.limit))
        K.clamped_glu(wide, None, act, limit if limit > 0 else float("inf"), self.alpha, up_offset=self.up_offset)
        out = rt.rows(tokens, self.h, dtype=torch.float32)
        K.gemm_nt(act, self.w_shared_down, out, err=rt.err)
        return out

    def forward(self, x, ctx, residual, overwrite=False):
        rt, tokens = self.rt, residual.shape[0]
        f32, i32 = torch.float32, torch.int32
        pairs = tokens * self.top
        routed = self.E + self.identity
        logits = rt.rows(tokens, self.w_router.shape[0], dtype=f32)
        K.gemm_nt(x, self.w_router, logits, err=rt.err)
        # few tokens: the shared expert runs on a stream of its own beside the routed ones (every kernel here is a
        # handful of blocks) and meets them before the sum
        shared, shared_on = None, None
        if self.shared and tokens <= K.FEW_TOKENS and rt.options.get("branch_streams", True) and x.is_cuda:
            shared_on = side_stream(rt.device, 2)
            shared_on.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(shared_on):
                shared = self._shared(logits, tokens)
        ids = rt.rows(tokens, self.top, dtype=i32)
        weights = rt.rows(tokens, self.top, dtype=f32)
        # bfloat16 products go to the tensor cores where TMA can address the rows (16-byte pitches)
        tensor_cores = (rt.dtype == torch.bfloat16 and K.USE_TENSOR_CORES[0] and self.h % 8 == 0 and self.f % 8 == 0)
        tile = K.experts_tile_rows(tensor_cores)
        max_tiles = min(pairs, pairs // tile + self.E)
        plan = rt.rows(1 + 3 * max_tiles, dtype=i32)
        row_token = rt.rows(pairs, dtype=i32)
        row_weight = rt.rows(pairs, dtype=f32)
        pair_row = rt.rows(pairs, dtype=i32)
        if tokens <= K.FEW_TOKENS:
            # few tokens: the choice and the plan in one launch of one block
            K.experts_route_plan(logits, self.top, ids, weights, routed, self.score_mode, self.bias, self.E, tile,
                                 plan, max_tiles, row_token, row_weight, pair_row, rt.err)
        else:
            K.experts_route(logits, self.top, ids, weights, experts=routed, softmax=self.score_mode,
                            correction=self.bias)
            K.experts_plan(ids, weights, self.E, tile, plan, max_tiles, row_token, row_weight, pair_row, rt.err)
        on_input = self.scale == "input"
        # one expert a token and nothing beside it: the second product adds into the residual stream itself (an
        # element has one writer); else its rows go through memory and are added in order of rank
        alone = self.top == 1 and on_input and not self.identity and not self.shared and not overwrite
        y = residual if alone else rt.rows(pairs, self.h, dtype=f32)
        down = 2 if alone else 1
        wide = rt.rows(pairs, 2 * self.f, dtype=f32) if self.glu else None
        act = None if self.glu else rt.rows(pairs, self.f)
        if tensor_cores:
            sorted_rows = rt.rows(pairs, self.h)
            K.experts_gather(x, row_token, row_weight if on_input else None, sorted_rows)
            ok = K.experts_product_tc(1 if self.glu else 0, plan, max_tiles, sorted_rows, self.w_up, wide if self.glu else act,
                                      rt.err)
            if self.glu:
                act = self._activate(wide, pairs, self.f)
            if not (ok and K.experts_product_tc(down, plan, max_tiles, act, self.w_down, y, rt.err, row_token)):
                raise K.KernelError("routed_experts: the tensor-core product refused shapes it was chosen for")
        else:
            K.experts_product(3 if self.glu else 0, plan, max_tiles, x, row_token, row_weight if on_input else None,
                              self.w_up, wide if self.glu else act)
            if self.glu:
                act = self._activate(wide, pairs, self.f)
            K.experts_product(down, plan, max_tiles, act, row_token, row_weight, self.w_down, y)
        if alone:
            return
        plain = on_input and not self.identity and not self.shared and not overwrite
        if plain:
            K.experts_combine(y, pair_row, residual, self.top)
            return
        if shared_on is not None:
            torch.cuda.current_stream().wait_stream(shared_on)
        elif self.shared:
            shared = self._shared(logits, tokens)
        gate = logits[:, routed:routed + 1] if self.shared and self.shared.get("gate") else None
        K.experts_mix(y, pair_row, ids, None if on_input else weights, self.E, x, residual, shared=shared,
                      shared_gate=gate, store=overwrite)


@register_part("feed_forward", "routed_experts")
def _build(spec, runtime, **_):
    return RoutedExperts(spec["hidden_size"], spec["expert_size"], spec["experts"], spec["top"], runtime,
                         score=spec.get("score", "sigmoid"), activation=spec.get("activation", "relu2"),
                         scale=spec.get("scale", "input"), limit=spec.get("limit", 0.0), alpha=spec.get("alpha", 1.702),
                         identity=spec.get("identity", 0), correction=spec.get("correction", False),
                         shared=spec.get("shared"), names=spec.get("names"))
