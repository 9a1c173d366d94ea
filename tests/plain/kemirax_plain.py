"""The Kemirax design written out plainly, one function per mechanism, in float64 by default,
whole sequences at a time and without a cache.  It shares no code with the engine: tests compare
the engine's kernels, cache and step function with it.

Notation: ``x`` [n, width] is a sequence of n tokens at positions 0 .. n-1; linear weights are
[out, in] and applied as ``x @ W.T``; ``w`` is the dictionary of the model's tensors by name,
``p`` a tensor-name prefix, ``m`` a mixer's and ``f`` a feed-forward's entry of the configuration.
"""

from __future__ import annotations

import math

import torch


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def scalar_rms_norm(x, gain, eps):
    """Unit root mean square (eps inside the root), times one number for the whole row."""
    return unit_rms(x, eps) * gain.reshape(())


def shifted(h, mix, before=None):
    """Every row moved towards the row before it: h_t + (h_(t-1) - h_t) * mix, the row before the
    first being ``before`` (zeros at the start of a sequence)."""
    first = torch.zeros_like(h[:1]) if before is None else before.reshape(1, -1)
    prev = torch.cat([first, h[:-1]], dim=0)
    return h + (prev - h) * mix


def output_gate(h, w, name):
    """sigmoid(W h + b), one number per coordinate of a sublayer's result."""
    return torch.sigmoid(h @ w[name].T + w[name + ".b"])


# ---------------------------------------------------------------------------
# rotation
# ---------------------------------------------------------------------------

def stretched_frequencies(dims, base, scaling=None, dtype=torch.float64):
    """(f [dims/2], magnitude): f_i = base^(-2i/dims); with ``scaling`` the slow end of the
    spectrum is divided by ``factor`` along a linear ramp and the magnitude is 0.1 ln(factor) + 1."""
    i = torch.arange(dims // 2, dtype=dtype)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def turn_dim(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(turn_dim(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(scaling["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotary_tables(positions, dims, base, scaling=None, dtype=torch.float64):
    f, mag = stretched_frequencies(dims, base, scaling, dtype)
    ang = torch.as_tensor(positions, dtype=dtype)[:, None] * f[None, :]
    return ang.cos() * mag, ang.sin() * mag


def rotate_halves(x, cos, sin):
    """x [n, heads, dims]: element i is paired with element i + dims/2."""
    half = x.shape[-1] // 2
    u, v = x[..., :half], x[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([u * c - v * s, v * c + u * s], dim=-1)


# ---------------------------------------------------------------------------
# attention over a cached latent, with queries through a latent of their own
# ---------------------------------------------------------------------------

def causal_softmax_attention(q, k, v, scale, weights=False):
    """q, k [n, H, d], v [n, H, dv]; query i sees every key j <= i."""
    n = q.shape[0]
    scores = torch.einsum("ihd,jhd->hij", q, k) * scale
    hidden = torch.arange(n)[None, :] > torch.arange(n)[:, None]
    p = torch.softmax(scores.masked_fill(hidden[None], float("-inf")), dim=-1)
    return p if weights else torch.einsum("hij,jhd->ihd", p, v)


def key_latent(x, w, p, m, eps, positions=None):
    """What a latent layer caches per token: the normed latent c [n, kv_rank] and the rotated key
    part [n, rot_dim] that all heads share."""
    n, rank, rot = x.shape[0], m["kv_rank"], m["rot"]
    positions = range(n) if positions is None else positions
    cos, sin = rotary_tables(positions, rot["dims"], rot["base"], rot.get("scaling"), x.dtype)
    down = x @ w[p + ".dkv"].T
    c = unit_rms(down[:, :rank], eps) * w[p + ".dkv.norm"]
    return c, rotate_halves(down[:, None, rank:], cos, sin)[:, 0]


def latent_queries(x, w, p, m, eps, positions=None):
    """[n, H, dim + rot_dim]: queries from a normed latent of their own, the last rot_dim of each
    head rotated."""
    n, H, d, dr, rot = x.shape[0], m["heads"], m["dim"], m["rot_dim"], m["rot"]
    positions = range(n) if positions is None else positions
    cos, sin = rotary_tables(positions, rot["dims"], rot["base"], rot.get("scaling"), x.dtype)
    cq = unit_rms(x @ w[p + ".dq"].T, eps) * w[p + ".dq.norm"]
    q = (cq @ w[p + ".uq"].T).view(n, H, d + dr)
    return torch.cat([q[..., :d], rotate_halves(q[..., d:], cos, sin)], dim=-1)


def latent_attention_mixer(x, w, p, m, eps, cached=None, weights=False):
    """``cached``: (c, rotated key part) of the layer whose cache this one reads, or None for a
    layer that makes its own.  Returns (output, (c, rotated key part))."""
    n, H, d, dv = x.shape[0], m["heads"], m["dim"], m["vdim"]
    c, k_rot = key_latent(x, w, p, m, eps) if cached is None else cached
    q = latent_queries(x, w, p, m, eps)
    k = torch.cat([(c @ w[p + ".uk"].T).view(n, H, d), k_rot[:, None, :].expand(n, H, -1)], dim=-1)
    v = (c @ w[p + ".uv"].T).view(n, H, dv)
    o = causal_softmax_attention(q, k, v, m["scale"], weights)
    if weights:
        return o, (c, k_rot)
    return o.reshape(n, H * dv) @ w[p + ".o"].T, (c, k_rot)


# ---------------------------------------------------------------------------
# gated linear attention
# ---------------------------------------------------------------------------

def channel_decay(x, w, p, tau):
    """sigmoid(z)^(1/tau) with z from a low-rank map with a bias, through its logarithm."""
    z = (x @ w[p + ".a1"].T) @ w[p + ".a2"].T + w[p + ".a2.b"]
    return torch.exp(torch.nn.functional.logsigmoid(z) / tau)


def decayed_outer_product_rule(q, k, v, alpha, state=None):
    """q, k, alpha [n, H, dk], v [n, H, dv].  S [H, dk, dv] from zero (or ``state``):
    S <- diag(alpha_t) S + k_t v_t^T, o_t = S^T q_t.  Returns (o [n, H, dv], S)."""
    n, H, dk = q.shape
    S = torch.zeros(H, dk, v.shape[-1], dtype=q.dtype) if state is None else state.clone()
    out = []
    for t in range(n):
        S = S * alpha[t][:, :, None] + k[t][:, :, None] * v[t][:, None, :]
        out.append(torch.einsum("hkv,hk->hv", S, q[t]))
    return torch.stack(out), S


def gated_linear_mixer(x, w, p, m, eps):
    n, H, d, dv = x.shape[0], m["heads"], m["dim"], m["vdim"]
    q = (x @ w[p + ".q"].T).view(n, H, d) * d ** -0.5
    k = (x @ w[p + ".k"].T).view(n, H, d)
    v = (x @ w[p + ".v"].T).view(n, H, dv)
    o, _ = decayed_outer_product_rule(q, k, v, channel_decay(x, w, p, m["tau"]).view(n, H, d))
    o = unit_rms(o, eps) * w[p + ".norm"]
    return (o.reshape(n, H * dv) * torch.nn.functional.silu(x @ w[p + ".g"].T)) @ w[p + ".o"].T


# ---------------------------------------------------------------------------
# the feed-forward: routed experts, some of them the identity, and a shared expert
# ---------------------------------------------------------------------------

def clamped_expert(x, w, p, limit):
    g = (x @ w[p + ".gate"].T).clamp(max=limit)
    u = (x @ w[p + ".up"].T).clamp(-limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + ".down"].T


def route(x, w, p, router):
    """(chosen [n, top] in order of rank, their weights [n, top]): softmax scores over all
    experts; the choice is by score + correction (ties to the lower index), the weight is the
    score itself."""
    scores = torch.softmax(x @ w[p + ".router"].T, dim=-1)
    choice = scores + w[p + ".correction"]
    order = torch.sort(choice, dim=-1, descending=True, stable=True).indices[:, :router["top"]]
    return order, torch.gather(scores, 1, order)


def expert_mixture(x, w, p, f):
    router = f["router"]
    real = router["experts"]                     # experts real .. real + identity - 1 return their input
    chosen, weight = route(x, w, p, router)
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        for e, s in zip(chosen[t].tolist(), weight[t]):
            y = clamped_expert(x[t:t + 1], w, f"{p}.e{e}", f["expert"]["limit"])[0] if e < real else x[t]
            out[t] = out[t] + s * y
    shared = f.get("shared")
    if shared:
        gate = torch.sigmoid(x @ w[p + ".shared.sg"].T)              # [n, 1]
        out = out + gate * clamped_expert(x, w, p + ".shared", shared["limit"])
    return out


# ---------------------------------------------------------------------------
# layers, model
# ---------------------------------------------------------------------------

def layer_forward(x, w, i, cfg, caches):
    """One layer: a single norm feeds both sublayers, the mixer through the token shift; each
    sublayer's result passes its gate, and their sum is added to the stream."""
    layer, eps, p = cfg["layers"][i], cfg["norm"]["eps"], f"l{i}"
    h = scalar_rms_norm(x, w[p + ".norm1"], eps)
    hm = shifted(h, w[p + ".shift"])
    m = layer["mixer"]
    if layer["type"] == "gla":
        mixed = gated_linear_mixer(hm, w, p + ".mix", m, eps)
    elif layer["type"] == "latent_attention":
        source = m.get("kv_from")
        mixed, made = latent_attention_mixer(hm, w, p + ".mix", m, eps, None if source is None else caches[source])
        caches[i] = made
    else:
        raise ValueError(layer["type"])
    total = mixed * output_gate(h, w, p + ".rg1")
    if layer.get("mlp"):
        total = total + expert_mixture(h, w, p + ".mlp", layer["mlp"]) * output_gate(h, w, p + ".rg2")
    return x + total


def forward(cfg, w, tokens, dtype=torch.float64, trace=None):
    """Logits [n, vocab] of one sequence.  ``trace``: a list that receives the residual stream
    after every layer."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    caches: dict = {}
    for i in range(len(cfg["layers"])):
        x = layer_forward(x, w, i, cfg, caches)
        if trace is not None:
            trace.append(x.clone())
    return scalar_rms_norm(x, w["final.norm"], cfg["norm"]["eps"]) @ w["head"].T


def read_model_folder(folder):
    """(config dictionary, tensors by name in float64) of a model folder."""
    import json
    from pathlib import Path

    from safetensors.torch import load_file

    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    w = {k: (v.double() if v.is_floating_point() else v) for k, v in load_file(str(folder / "model.safetensors")).items()}
    return cfg, w


def model_logits(folder, tokens, dtype=torch.float64):
    cfg, w = read_model_folder(folder)
    return forward(cfg, w, tokens, dtype)
