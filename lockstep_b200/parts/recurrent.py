"""Mixers that carry a fixed-size state per request instead of keys and values.

Both keep, per head, a float32 matrix S [key channels, value channels] in the request's state
slot, walk a portion token by token, and finish with a per-head RMSNorm and a gate before the
output projection.  The slot also carries what the next portion needs of the tokens before it.

"gated_delta" (per head, with a decay g per key channel):
    S <- diag(g_t) S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;  o_t = S^T q_t
  q, k, v come through short causal convolutions (their last taps - 1 inputs are carried) and
  silu; q and k are unit vectors per head, q scaled by dk^(-1/2); beta = sigmoid(W_b x);
  g = exp(-exp(A_log) softplus(W_a2 W_a1 x + dt_bias)); the read-out is normed per head, times a
  gain shared by the heads, times sigmoid(W_g2 W_g1 x).

"wkv" (per head, with a decay w per key channel and a bonus u for the current token):
    o_t = (S + diag(u) k_t v_t^T)^T r_t;  S <- diag(w_t) S + k_t v_t^T
  r, k, v, the gate and the decay's low-rank map each read their own mix of the token and the
  one before it (carried across portions): x + (x_prev - x) mu;  w = exp(-exp(W_w2 tanh(W_w1 m) +
  w0)); the read-out is normed per head, times a gain over all heads, times silu(W_g m).

"gated_linear" (per head, with a decay a per key channel):
    S <- diag(a_t) S + k_t v_t^T;  o_t = S^T q_t
  q = W_q x * dk^(-1/2), k, v straight from their projections; a = sigmoid(W_a2 W_a1 x + b)^(1/tau),
  made through its logarithm; the read-out is normed per head, times a gain shared by the heads,
  times silu(W_g x).  Nothing but S is carried.

"gated_recurrent_unit" (per channel of ``width`` channels, in ``blocks`` equal parts):
    u = conv(W_x x + b_x);  r = sigmoid(A_b u_b + a_b), i = sigmoid(I_b u_b + i_b) with square matrices per part;
    log a = -``rate`` r softplus(lam);  S <- a S + sqrt(1 - a^2) i u;  out = W_o (S gelu(W_y x + b_y))
  a causal convolution of ``conv_taps`` taps per channel (its last taps - 1 inputs are carried beside S).

"retention" (per head, with one fixed decay per head, ``decay``):
    S <- decay_h S + k_t v_t^T;  o_t = S^T q_t
  q and k rotated by the position encoding (k then times dk^(-1/2)); the read-out is divided by its root mean
  square per head (no gain), times silu(W_g x).  Nothing but S is carried.

The projections run as the engine's products (tensor cores in bfloat16); everything between
them and the recurrence, the recurrence and the state are float32 (csrc/recurrent.cu).
"""

from __future__ import annotations

import torch

from .. import kernels as K
from .base import CacheNeed, Mixer, Runtime, WeightSpec, register_part
from .norm import NormedRows


def portion_list(ctx, state: torch.Tensor, rt: Runtime):
    """(device list, its capacity) of the step's portions, made once per step on the device
    from ``ctx.token_slot`` and kept on the context for the other layers (a recorded step makes
    it in its graph).  There are at most as many portions as state slots."""
    made = getattr(ctx, "_portion_list", None)
    if made is None:
        cap = min(int(ctx.token_slot.numel()), int(state.shape[0]))
        out = torch.empty(1 + 3 * cap, dtype=torch.int32, device=rt.device)
        K.find_portions(ctx.token_slot, out, cap, rt.err)
        made = ctx._portion_list = (out, cap)
    return made


def _f32(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.float32).contiguous()


class GatedDelta(Mixer):
    graph_safe = True
    accepts_normed_rows = True       # its one product of the mixer's input can make the norm itself

    def __init__(self, hidden_size, num_heads, num_kv_heads, key_dim, value_dim, conv_taps, norm_eps, unit_eps,
                 runtime: Runtime, decay_rank=None, gate_rank=None):
        if num_heads % num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if not 1 <= conv_taps <= 8:
            raise ValueError(f"a convolution of {conv_taps} taps is not supported (1 to 8)")
        if key_dim > 256:
            raise ValueError(f"key_dim {key_dim} is not supported (up to 256)")
        self.w, self.H, self.G = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.dk, self.dv, self.taps = int(key_dim), int(value_dim), int(conv_taps)
        self.eps, self.unit_eps, self.rt = float(norm_eps), float(unit_eps), runtime
        self.Kd, self.Vd = self.G * self.dk, self.H * self.dv
        self.C = 2 * self.Kd + self.Vd
        # ranks of the two low-rank maps; -1: whatever the stored tensors have
        self.rank_a, self.rank_g = int(decay_rank or -1), int(gate_rank or -1)

    def cache_need(self):
        return CacheNeed("state", state_shape=(self.H * self.dk * self.dv + (self.taps - 1) * self.C,),
                         state_dtype=torch.float32)

    def weight_specs(self):
        taps = ("normal", 0.0, 0.5)
        return {
            "q": WeightSpec((self.Kd, self.w)), "k": WeightSpec((self.Kd, self.w)), "v": WeightSpec((self.Vd, self.w)),
            "q.conv": WeightSpec((self.Kd, self.taps), "gain", taps), "k.conv": WeightSpec((self.Kd, self.taps), "gain", taps),
            "v.conv": WeightSpec((self.Vd, self.taps), "gain", taps),
            "b": WeightSpec((self.H, self.w)), "A_log": WeightSpec((self.H,), "gain", ("normal", -1.0, 0.5)),
            "norm": WeightSpec((self.dv,), "gain"),
            "a1": WeightSpec((self.rank_a, self.w)), "a2": WeightSpec((self.H * self.dk, self.rank_a)),
            "dt_bias": WeightSpec((self.H * self.dk,), "gain", ("normal", -1.0, 1.0)),
            "g1": WeightSpec((self.rank_g, self.w)), "g2": WeightSpec((self.Vd, self.rank_g)),
            "o": WeightSpec((self.w, self.Vd)),
        }

    def bind(self, t):
        if t["a1"].shape[0] != t["a2"].shape[1] or t["g1"].shape[0] != t["g2"].shape[1]:
            raise ValueError("the two halves of a low-rank map do not have the same rank")
        # one product for everything that reads the mixer's input: q, k, v, beta, then (from a column
        # that is a multiple of 8, so that the next products can take them where they lie) the
        # inputs of the two low-rank maps
        zeros = lambda rows: torch.zeros((rows, self.w), dtype=t["q"].dtype, device=t["q"].device)
        self.low_at = -(-(self.C + self.H) // 8) * 8
        parts = [t["q"], t["k"], t["v"], t["b"], zeros(self.low_at - self.C - self.H), t["a1"], t["g1"]]
        self.ra, self.rg = t["a1"].shape[0], t["g1"].shape[0]
        parts.append(zeros(-(self.low_at + self.ra + self.rg) % 8))
        self.w_in = torch.cat(parts, dim=0).contiguous()
        self.conv_w = _f32(torch.cat([t["q.conv"], t["k.conv"], t["v.conv"]], dim=0))
        self.w_a2, self.w_g2, self.w_o = t["a2"].contiguous(), t["g2"].contiguous(), t["o"]
        self.dt_bias, self.a_log, self.gain = _f32(t["dt_bias"]), _f32(t["A_log"]), _f32(t["norm"])

    def forward(self, x, ctx, cache, residual):
        rt, tokens = self.rt, residual.shape[0]
        f32 = torch.float32
        proj = rt.rows(tokens, self.w_in.shape[0])
        if isinstance(x, NormedRows):
            x.linear(self.w_in, proj, K.EPILOGUE_STORE, rt.err)
        else:
            K.gemm_nt(x, self.w_in, proj, err=rt.err)
        # the low-rank maps' second halves as products with float32 results: the decay's goes
        # through the prep kernel (a token a block, beside the convolutions), the gate's to the
        # read-out kernel, which takes its sigmoid
        decay = rt.rows(tokens, self.H * self.dk, dtype=f32)
        z_gate = rt.rows(tokens, self.Vd, dtype=f32)
        K.gemm_nt(proj[:, self.low_at:self.low_at + self.ra], self.w_a2, decay, err=rt.err)
        K.gemm_nt(proj[:, self.low_at + self.ra:self.low_at + self.ra + self.rg], self.w_g2, z_gate, err=rt.err)
        qkv = rt.rows(tokens, self.C, dtype=f32)
        beta = rt.rows(tokens, self.H, dtype=f32)
        K.delta_prep(proj, self.conv_w, self.dt_bias, self.a_log, cache.state, ctx.token_slot, qkv, decay, beta,
                     self.H, self.G, self.dk, self.dv, self.taps, self.unit_eps)
        portions, cap = portion_list(ctx, cache.state, rt)
        o = rt.rows(tokens, self.Vd, dtype=f32)
        K.state_rule(K.RULE_DELTA, rt.dtype, portions, cap, cache.state, qkv, None, None, decay, beta, None, o,
                     proj, self.C, self.taps - 1, self.H, self.G, self.dk, self.dv)
        y = rt.rows(tokens, self.Vd)
        K.head_rms_gate(o, self.gain, z_gate, None, y, self.H, self.dv, True, self.eps, gate_logit=True)
        K.gemm_nt(y, self.w_o, residual, K.EPILOGUE_RESIDUAL, err=rt.err)


class Wkv(Mixer):
    graph_safe = True
    MIXES = ("r", "k", "v", "g", "w")

    def __init__(self, hidden_size, num_heads, head_dim, norm_eps, runtime: Runtime, decay_rank=None):
        if head_dim > 256:
            raise ValueError(f"head_dim {head_dim} is not supported (up to 256)")
        self.w, self.H, self.d = int(hidden_size), int(num_heads), int(head_dim)
        self.eps, self.rt = float(norm_eps), runtime
        self.A = self.H * self.d
        self.rank = int(decay_rank or -1)      # -1: whatever the stored tensors have

    def cache_need(self):
        return CacheNeed("state", state_shape=(self.H * self.d * self.d + self.w,), state_dtype=torch.float32)

    def weight_specs(self):
        specs = {f"mu.{s}": WeightSpec((self.w,), "gain", ("uniform", 0.0, 1.0)) for s in self.MIXES}
        specs.update({
            "r": WeightSpec((self.A, self.w)), "k": WeightSpec((self.A, self.w)), "v": WeightSpec((self.A, self.w)),
            "g": WeightSpec((self.A, self.w)), "w1": WeightSpec((self.rank, self.w)),
            "w2": WeightSpec((self.A, self.rank)),
            "w0": WeightSpec((self.A,), "gain", ("normal", -2.5, 1.0)),
            "u": WeightSpec((self.H, self.d), "gain", ("normal", 0.0, 0.5)),
            "norm": WeightSpec((self.A,), "gain"), "o": WeightSpec((self.w, self.A)),
        })
        return specs

    def bind(self, t):
        if t["w1"].shape[0] != t["w2"].shape[1]:
            raise ValueError("the two halves of the decay's low-rank map do not have the same rank")
        self.mu = _f32(torch.stack([t[f"mu.{s}"] for s in self.MIXES]))
        self.w_r, self.w_k, self.w_v, self.w_g = t["r"], t["k"], t["v"], t["g"]
        self.w_w1, self.w_w2, self.w_o = t["w1"], t["w2"].contiguous(), t["o"]
        self.w0, self.bonus, self.gain = _f32(t["w0"]), _f32(t["u"].reshape(-1)), _f32(t["norm"])

    def forward(self, x, ctx, cache, residual):
        rt, tokens = self.rt, residual.shape[0]
        f32 = torch.float32
        prev_offset = self.H * self.d * self.d
        mixed = rt.rows(len(self.MIXES) * tokens, self.w).view(len(self.MIXES), tokens, self.w)
        K.shift_mix(x, self.mu, cache.state, prev_offset, ctx.token_slot, mixed)
        r, k, v, g = (rt.rows(tokens, self.A) for _ in range(4))
        low = rt.rows(tokens, self.w_w1.shape[0])
        for i, (w, out) in enumerate(((self.w_r, r), (self.w_k, k), (self.w_v, v), (self.w_g, g), (self.w_w1, low))):
            K.gemm_nt(mixed[i], w, out, err=rt.err)
        K.tanh_rows(low)
        decay = rt.rows(tokens, self.A, dtype=f32)
        K.gemm_nt(low, self.w_w2, decay, err=rt.err)
        K.double_exp_decay(decay, self.w0)
        portions, cap = portion_list(ctx, cache.state, rt)
        o = rt.rows(tokens, self.A, dtype=f32)
        K.state_rule(K.RULE_WKV, rt.dtype, portions, cap, cache.state, r, k, v, decay, None, self.bonus, o,
                     x, self.w, 1, self.H, self.H, self.d, self.d)
        y = rt.rows(tokens, self.A)
        K.head_rms_gate(o, self.gain, None, g, y, self.H, self.d, False, self.eps)
        K.gemm_nt(y, self.w_o, residual, K.EPILOGUE_RESIDUAL, err=rt.err)


class GatedLinear(Mixer):
    graph_safe = True
    accepts_normed_rows = True
    can_overwrite = True

    def __init__(self, hidden_size, num_heads, key_dim, value_dim, tau, norm_eps, runtime: Runtime, decay_rank=None):
        if key_dim > 512:
            raise ValueError(f"key_dim {key_dim} is not supported (up to 512)")
        if not float(tau) > 0:
            raise ValueError("tau must be positive")
        self.w, self.H, self.dk, self.dv = int(hidden_size), int(num_heads), int(key_dim), int(value_dim)
        self.tau, self.eps, self.rt = float(tau), float(norm_eps), runtime
        self.Kd, self.Vd = self.H * self.dk, self.H * self.dv
        self.rank = int(decay_rank or -1)      # -1: whatever the stored tensors have

    def cache_need(self):
        return CacheNeed("state", state_shape=(self.H * self.dk * self.dv,), state_dtype=torch.float32)

    def weight_specs(self):
        return {"q": WeightSpec((self.Kd, self.w)), "k": WeightSpec((self.Kd, self.w)), "v": WeightSpec((self.Vd, self.w)),
                "g": WeightSpec((self.Vd, self.w)), "o": WeightSpec((self.w, self.Vd)),
                "norm": WeightSpec((self.dv,), "gain"),
                "a1": WeightSpec((self.rank, self.w)), "a2": WeightSpec((self.Kd, self.rank)),
                "a2.b": WeightSpec((self.Kd,), "gain", ("normal", 3.0, 1.0))}

    def bind(self, t):
        if t["a1"].shape[0] != t["a2"].shape[1]:
            raise ValueError("the two halves of the decay's low-rank map do not have the same rank")
        # one product for everything that reads the mixer's input; every part starts at a column
        # that is a multiple of 8, so that kernels and products can take it where it lies
        zeros = lambda rows: torch.zeros((rows, self.w), dtype=t["q"].dtype, device=t["q"].device)
        parts, self.at, col = [], {}, 0
        for name in ("q", "k", "v", "g", "a1"):
            self.at[name] = col
            parts += [t[name], zeros(-t[name].shape[0] % 8)]
            col += t[name].shape[0] + (-t[name].shape[0] % 8)
        self.ra = t["a1"].shape[0]
        self.w_in = torch.cat(parts, dim=0).contiguous()
        self.w_a2, self.w_o = t["a2"].contiguous(), t["o"]
        self.a_bias, self.gain = _f32(t["a2.b"]), _f32(t["norm"])

    def forward(self, x, ctx, cache, residual, overwrite=False):
        rt, tokens, at = self.rt, residual.shape[0], self.at
        proj = rt.rows(tokens, self.w_in.shape[0])
        if isinstance(x, NormedRows):
            x.linear(self.w_in, proj, K.EPILOGUE_STORE, rt.err)
        else:
            K.gemm_nt(x, self.w_in, proj, err=rt.err)
        decay = rt.rows(tokens, self.Kd, dtype=torch.float32)
        K.gemm_nt(proj[:, at["a1"]:at["a1"] + self.ra], self.w_a2, decay, err=rt.err)
        K.sigmoid_power_decay(decay, self.a_bias, self.tau)
        portions, cap = portion_list(ctx, cache.state, rt)
        o = rt.rows(tokens, self.Vd, dtype=torch.float32)
        K.state_rule(K.RULE_GLA, rt.dtype, portions, cap, cache.state, proj[:, at["q"]:at["q"] + self.Kd],
                     proj[:, at["k"]:at["k"] + self.Kd], proj[:, at["v"]:at["v"] + self.Vd], decay, None, None, o,
                     None, 0, 0, self.H, self.H, self.dk, self.dv, out_scale=self.dk ** -0.5)
        y = rt.rows(tokens, self.Vd)
        K.head_rms_gate(o, self.gain, None, proj[:, at["g"]:at["g"] + self.Vd], y, self.H, self.dv, True, self.eps)
        K.gemm_nt(y, self.w_o, residual, K.EPILOGUE_STORE if overwrite else K.EPILOGUE_RESIDUAL, err=rt.err)


class GatedRecurrentUnit(Mixer):
    graph_safe = True
    accepts_normed_rows = True
    can_overwrite = True

    def __init__(self, hidden_size, width, blocks, conv_taps, runtime: Runtime, rate: float = 8.0, names=None):
        if width % blocks:
            raise ValueError(f"gated_recurrent_unit: {blocks} parts do not divide {width} channels")
        if not 1 <= conv_taps <= 16:
            raise ValueError(f"a convolution of {conv_taps} taps is not supported (1 to 16)")
        self.w, self.C, self.blocks, self.taps = int(hidden_size), int(width), int(blocks), int(conv_taps)
        self.rate, self.rt = float(rate), runtime
        self.names = {"y": "y", "y_bias": "y.b", "x": "x", "x_bias": "x.b", "conv": "conv", "conv_bias": "conv.b",
                      "r": "ra", "r_bias": "ra.b", "i": "ri", "i_bias": "ri.b", "lam": "lam", "o": "o"}
        self.names.update(names or {})

    def cache_need(self):
        return CacheNeed("state", state_shape=(self.taps * self.C,), state_dtype=torch.float32)

    def weight_specs(self):
        n, C, bw = self.names, self.C, self.C // self.blocks
        small = ("normal", 0.0, 0.02)
        gate = ("normal", 0.0, bw ** -0.5)
        return {n["y"]: WeightSpec((C, self.w)), n["y_bias"]: WeightSpec((C,), "gain", small),
                n["x"]: WeightSpec((C, self.w)), n["x_bias"]: WeightSpec((C,), "gain", small),
                n["conv"]: WeightSpec((C, self.taps), "gain", ("normal", 0.0, 0.5)),
                n["conv_bias"]: WeightSpec((C,), "gain", small),
                n["r"]: WeightSpec((self.blocks, bw, bw), "matrix", gate), n["r_bias"]: WeightSpec((self.blocks, bw), "gain", small),
                n["i"]: WeightSpec((self.blocks, bw, bw), "matrix", gate), n["i_bias"]: WeightSpec((self.blocks, bw), "gain", small),
                n["lam"]: WeightSpec((C,), "gain", ("normal", -2.0, 1.0)), n["o"]: WeightSpec((self.w, C))}

    def bind(self, t):
        n = self.names
        # one product for both branches: y's columns, then x's from a column that is a multiple of 8
        pad = -self.C % 8
        zeros = torch.zeros((pad, self.w), dtype=t[n["y"]].dtype, device=t[n["y"]].device)
        self.x_at = self.C + pad
        self.w_in = torch.cat([t[n["y"]], zeros, t[n["x"]]], dim=0).contiguous()
        self.y_bias, self.x_bias = _f32(t[n["y_bias"]]), _f32(t[n["x_bias"]])
        self.conv_w, self.conv_b = _f32(t[n["conv"]]), _f32(t[n["conv_bias"]])
        # the gates' matrices transposed to [part, in, out]: a thread of the gates' kernel owns an output channel
        self.w_r = t[n["r"]].transpose(1, 2).contiguous()
        self.w_i = t[n["i"]].transpose(1, 2).contiguous()
        self.b_r, self.b_i = _f32(t[n["r_bias"]].reshape(-1)), _f32(t[n["i_bias"]].reshape(-1))
        self.softplus_lam = torch.nn.functional.softplus(_f32(t[n["lam"]])).contiguous()
        self.w_o = t[n["o"]]

    def forward(self, x, ctx, cache, residual, overwrite=False):
        rt, tokens = self.rt, residual.shape[0]
        proj = rt.rows(tokens, self.w_in.shape[0])
        if isinstance(x, NormedRows):
            x.linear(self.w_in, proj, K.EPILOGUE_STORE, rt.err)
        else:
            K.gemm_nt(x, self.w_in, proj, err=rt.err)
        a = rt.rows(tokens, self.C, dtype=torch.float32)
        b = rt.rows(tokens, self.C, dtype=torch.float32)
        K.unit_gates(proj, self.x_at, self.x_bias, self.conv_w, self.conv_b, cache.state, ctx.token_slot, self.w_r, self.w_i,
                     self.b_r, self.b_i, self.softplus_lam, a, b, self.blocks, self.taps, self.rate)
        portions, cap = portion_list(ctx, cache.state, rt)
        y = rt.rows(tokens, self.C)
        K.unit_scan(portions, cap, a, b, proj, 0, self.x_at, self.y_bias, self.x_bias, cache.state, y, self.taps)
        K.gemm_nt(y, self.w_o, residual, K.EPILOGUE_STORE if overwrite else K.EPILOGUE_RESIDUAL, err=rt.err)


class Retention(Mixer):
    graph_safe = True
    accepts_normed_rows = True
    can_overwrite = True

    def __init__(self, hidden_size, num_heads, key_dim, value_dim, decay, norm_eps, position, runtime: Runtime):
        if key_dim > 512:
            raise ValueError(f"key_dim {key_dim} is not supported (up to 512)")
        if len(decay) != num_heads or not all(0.0 < float(d) <= 1.0 for d in decay):
            raise ValueError("retention: one decay in (0, 1] per head")
        self.w, self.H, self.dk, self.dv = int(hidden_size), int(num_heads), int(key_dim), int(value_dim)
        self.decay_values, self.eps, self.position, self.rt = [float(d) for d in decay], float(norm_eps), position, runtime
        self.Kd, self.Vd = self.H * self.dk, self.H * self.dv

    def cache_need(self):
        return CacheNeed("state", state_shape=(self.H * self.dk * self.dv,), state_dtype=torch.float32)

    def weight_specs(self):
        return {"q": WeightSpec((self.Kd, self.w)), "k": WeightSpec((self.Kd, self.w)), "v": WeightSpec((self.Vd, self.w)),
                "g": WeightSpec((self.Vd, self.w)), "o": WeightSpec((self.w, self.Vd))}

    def bind(self, t):
        zeros = lambda rows: torch.zeros((rows, self.w), dtype=t["q"].dtype, device=t["q"].device)
        parts, self.at, col = [], {}, 0
        for name in ("q", "k", "v", "g"):
            self.at[name] = col
            parts += [t[name], zeros(-t[name].shape[0] % 8)]
            col += t[name].shape[0] + (-t[name].shape[0] % 8)
        self.w_in = torch.cat(parts, dim=0).contiguous()
        self.w_o = t["o"]
        dev = t["q"].device
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32).repeat_interleave(self.dk).to(dev).contiguous()
        self.ones = torch.ones(self.dv, dtype=torch.float32, device=dev)

    def forward(self, x, ctx, cache, residual, overwrite=False):
        rt, tokens, at = self.rt, residual.shape[0], self.at
        proj = rt.rows(tokens, self.w_in.shape[0])
        if isinstance(x, NormedRows):
            x.linear(self.w_in, proj, K.EPILOGUE_STORE, rt.err)
        else:
            K.gemm_nt(x, self.w_in, proj, err=rt.err)
        rot = self.position.rotary()
        cos, sin, rot_dim = rot if rot is not None else (None, None, 0)
        if rot_dim and self.position.rotary_interleaved:
            raise ValueError("retention rotates halves of a head")
        qkv = rt.rows(tokens, 2 * self.Kd + self.Vd, dtype=torch.float32)
        K.rotate_rows(proj, at["q"], at["k"], at["v"], cos, sin, ctx.positions, qkv, self.H, self.dk, self.dv, rot_dim,
                      self.dk ** -0.5, rt.err)
        portions, cap = portion_list(ctx, cache.state, rt)
        o = rt.rows(tokens, self.Vd, dtype=torch.float32)
        K.state_rule(K.RULE_GLA, torch.float32, portions, cap, cache.state, qkv[:, :self.Kd], qkv[:, self.Kd:2 * self.Kd],
                     qkv[:, 2 * self.Kd:], self.decay, None, None, o, None, 0, 0, self.H, self.H, self.dk, self.dv,
                     decay_fixed=True)
        y = rt.rows(tokens, self.Vd)
        K.head_rms_gate(o, self.ones, None, proj[:, at["g"]:at["g"] + self.Vd], y, self.H, self.dv, True, self.eps)
        K.gemm_nt(y, self.w_o, residual, K.EPILOGUE_STORE if overwrite else K.EPILOGUE_RESIDUAL, err=rt.err)


@register_part("mixer", "gated_recurrent_unit")
def _build_unit(spec, runtime, **_):
    return GatedRecurrentUnit(spec["hidden_size"], spec["width"], spec["blocks"], spec["conv_taps"], runtime,
                              rate=spec.get("rate", 8.0), names=spec.get("names"))


@register_part("mixer", "retention")
def _build_retention(spec, runtime, position=None, **_):
    return Retention(spec["hidden_size"], spec["num_heads"], spec["key_dim"], spec["value_dim"], spec["decay"],
                     spec["norm_eps"], position, runtime)


@register_part("mixer", "gated_linear")
def _build_gated_linear(spec, runtime, **_):
    return GatedLinear(spec["hidden_size"], spec["num_heads"], spec["key_dim"], spec["value_dim"], spec["tau"],
                       spec["norm_eps"], runtime, decay_rank=spec.get("decay_rank"))


@register_part("mixer", "gated_delta")
def _build_delta(spec, runtime, **_):
    return GatedDelta(spec["hidden_size"], spec["num_heads"], spec["num_kv_heads"], spec["key_dim"],
                      spec["value_dim"], spec["conv_taps"], spec["norm_eps"], spec.get("unit_eps", 1e-6), runtime,
                      decay_rank=spec.get("decay_rank"), gate_rank=spec.get("gate_rank"))


@register_part("mixer", "wkv")
def _build_wkv(spec, runtime, **_):
    return Wkv(spec["hidden_size"], spec["num_heads"], spec["head_dim"], spec["norm_eps"], runtime,
               decay_rank=spec.get("decay_rank"))
