"""The Pikurax design written out plainly, one function per mechanism, in float64 by default,
whole sequences at a time and without a cache.  It shares no code with the engine: tests compare
the engine's kernels, cache and step function with it.

Notation: ``x`` [n, width] is a sequence of n tokens at positions 0 .. n-1; linear weights are
[out, in] and applied as ``x @ W.T``; a "mixer" maps the normed residual stream to what is added
to it.  ``w`` is the dictionary of the model's tensors by name, ``p`` a tensor-name prefix.
"""

from __future__ import annotations

import math

import torch


# ---------------------------------------------------------------------------
# small pieces
# ---------------------------------------------------------------------------

def layer_norm(x, gain, eps):
    """(x - mean) / sqrt(var + eps) * gain, var the mean of the squared deviations; no bias."""
    mu = x.mean(-1, keepdim=True)
    dev = x - mu
    return dev / torch.sqrt((dev * dev).mean(-1, keepdim=True) + eps) * gain


def rms_unit(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def rotate_halves(x, base, dims, positions=None):
    """x [n, heads, d]: element i < dims/2 is paired with element i + dims/2; the pair (u, v) at position
    p becomes (u cos a - v sin a, v cos a + u sin a), a = p base^(-2i/dims); elements from dims on pass."""
    n = x.shape[0]
    half = dims // 2
    pos = torch.arange(n, dtype=torch.float64) if positions is None else positions.to(torch.float64)
    freq = torch.tensor([float(base) ** (-2.0 * i / dims) for i in range(half)], dtype=torch.float64)
    ang = pos[:, None] * freq[None, :]
    cos, sin = ang.cos().to(x.dtype)[:, None, :], ang.sin().to(x.dtype)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], dim=-1)


# ---------------------------------------------------------------------------
# embedding
# ---------------------------------------------------------------------------

def bigram_rows(tokens, bg):
    """For each token the row of the pair table: (previous * mul_prev + token * mul_cur) mod buckets, and row
    ``buckets`` for a sequence's first token."""
    rows = []
    for t, tok in enumerate(tokens):
        rows.append(bg["buckets"] if t == 0 else (tokens[t - 1] * bg["mul_prev"] + tok * bg["mul_cur"]) % bg["buckets"])
    return rows


def embedding(tokens, w, cfg):
    e = cfg["embedding"]
    ids = torch.tensor(list(tokens), dtype=torch.long)
    x = w["embed"][ids] * float(e.get("scale", 1.0))
    if e.get("bigram"):
        x = x + w["bigram"][torch.tensor(bigram_rows(list(tokens), e["bigram"]), dtype=torch.long)]
    return x


# ---------------------------------------------------------------------------
# softmax attention with a mask, a cap, a distance bias and a sink
# ---------------------------------------------------------------------------

def softmax_attention(q, k, v, scale, chunk=0, softcap=0.0, slopes=None, sinks=None, weights=False):
    """q [n, H, d], k [n, G, d], v [n, G, dv].  score(i, j) = q_i . k_j scale, capped as cap tanh(score / cap),
    minus slopes[h] (i - j); visible are j <= i, and with ``chunk`` only those with i // chunk == j // chunk;
    with ``sinks`` the softmax's denominator holds exp(sinks[h]) as one more term."""
    n, H, _ = q.shape
    rep = H // k.shape[1]
    kk, vv = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, kk) * scale
    if softcap:
        s = softcap * torch.tanh(s / softcap)
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    if slopes is not None:
        s = s - slopes[:, None, None] * (i - j).clamp(min=0).to(q.dtype)[None]
    hidden = j > i
    if chunk:
        hidden = hidden | (torch.div(i, chunk, rounding_mode="floor") != torch.div(j, chunk, rounding_mode="floor"))
    s = s.masked_fill(hidden[None], float("-inf"))
    if sinks is not None:
        m = torch.maximum(s.max(-1, keepdim=True).values, sinks[:, None, None])
        e = torch.exp(s - m)
        pr = e / (e.sum(-1, keepdim=True) + torch.exp(sinks[:, None, None] - m))
    else:
        pr = torch.softmax(s, dim=-1)
    if weights:
        return pr
    return torch.einsum("hij,jhd->ihd", pr, vv)


def chunked_attention_mixer(x, w, p, m, weights=False):
    """Left side of a ``parallel`` layer: values are the keys as projected, rotation of q and k, chunks."""
    n = x.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = (x @ w[p + ".q"].T).view(n, H, d)
    k = (x @ w[p + ".k"].T).view(n, G, d)
    v = k
    rot = m["rot"]
    q, k = rotate_halves(q, rot["base"], rot["dims"]), rotate_halves(k, rot["base"], rot["dims"])
    o = softmax_attention(q, k, v, m["scale"], chunk=m["mask"]["size"], weights=weights)
    if weights:
        return o
    return o.reshape(n, H * d) @ w[p + ".o"].T


def distance_slopes(H, dtype=torch.float64):
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], dtype=dtype)


def query_temperature(n, coef, every, dtype=torch.float64):
    pos = torch.arange(n, dtype=torch.int64)
    return 1.0 + coef * torch.log((torch.div(pos + 1, every, rounding_mode="floor") + 1).to(dtype))


def biased_attention_mixer(x, w, p, m, eps, weights=False):
    """Left side of a ``parallel_2`` layer: biases, per-head norms of q and k, temperature, cap, bias, sink."""
    n = x.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (x @ w[p + ".q"].T + w[p + ".q.b"]).view(n, H, d)
    k = (x @ w[p + ".k"].T + w[p + ".k.b"]).view(n, G, d)
    v = (x @ w[p + ".v"].T + w[p + ".v.b"]).view(n, G, dv)
    q = rms_unit(q, eps) * w[p + ".q.norm"]
    k = rms_unit(k, eps) * w[p + ".k.norm"]
    t = m.get("q_temp")
    if t:
        q = q * query_temperature(n, t["coef"], t["every"], x.dtype)[:, None, None]
    o = softmax_attention(q, k, v, m["scale"], softcap=float(m.get("softcap", 0.0) or 0.0),
                          slopes=distance_slopes(H, x.dtype), sinks=w[p + ".sink"], weights=weights)
    if weights:
        return o
    return o.reshape(n, H * dv) @ w[p + ".o"].T


# ---------------------------------------------------------------------------
# recurrences
# ---------------------------------------------------------------------------

def causal_conv(x, taps_w, bias):
    """x [n, c], taps_w [c, taps] (last column the current token's), zeros before the start."""
    n, c = x.shape
    taps = taps_w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, c, dtype=x.dtype), x], dim=0)
    out = torch.zeros_like(x)
    for j in range(taps):
        out = out + padded[j:j + n] * taps_w[:, j]
    return out + bias


def gated_unit_recurrence(u, r, i, lam, state=None):
    """S_t = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t with a_t = exp(-8 r_t softplus(lam)); returns (S [n, c], last S)."""
    log_a = -8.0 * r * torch.nn.functional.softplus(lam)
    a = torch.exp(log_a)
    b = torch.sqrt(1.0 - a * a) * i * u
    S = torch.zeros(u.shape[1], dtype=u.dtype) if state is None else state.clone()
    out = []
    for t in range(u.shape[0]):
        S = a[t] * S + b[t]
        out.append(S)
    return torch.stack(out), S


def gated_unit_mixer(x, w, p, m):
    """Right side of a ``parallel`` layer."""
    n = x.shape[0]
    width, blocks = m["width"], m["blocks"]
    y = gelu_tanh(x @ w[p + ".y"].T + w[p + ".y.b"])
    u = causal_conv(x @ w[p + ".x"].T + w[p + ".x.b"], w[p + ".conv"], w[p + ".conv.b"])
    ub = u.view(n, blocks, width // blocks)
    r = torch.sigmoid(torch.einsum("boi,nbi->nbo", w[p + ".ra"], ub) + w[p + ".ra.b"]).reshape(n, width)
    i = torch.sigmoid(torch.einsum("boi,nbi->nbo", w[p + ".ri"], ub) + w[p + ".ri.b"]).reshape(n, width)
    S, _ = gated_unit_recurrence(u, r, i, w[p + ".lam"])
    return (S * y) @ w[p + ".o"].T


def retention_rule(q, k, v, decay, state=None):
    """q, k [n, H, dk], v [n, H, dv], decay [H]: S <- decay S + k_t v_t^T, o_t = S^T q_t."""
    n, H, dk = q.shape
    S = torch.zeros(H, dk, v.shape[-1], dtype=q.dtype) if state is None else state.clone()
    out = []
    for t in range(n):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out.append(torch.einsum("hkv,hk->hv", S, q[t]))
    return torch.stack(out), S


def retention_mixer(x, w, p, m, eps):
    """Right side of a ``parallel_2`` layer."""
    n = x.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = (x @ w[p + ".q"].T).view(n, H, dk)
    k = (x @ w[p + ".k"].T).view(n, H, dk)
    v = (x @ w[p + ".v"].T).view(n, H, dv)
    rot = m["rot"]
    q = rotate_halves(q, rot["base"], rot["dims"])
    k = rotate_halves(k, rot["base"], rot["dims"]) * dk ** -0.5
    o, _ = retention_rule(q, k, v, torch.tensor(m["decay"], dtype=x.dtype))
    o = rms_unit(o, eps).reshape(n, H * dv) * silu(x @ w[p + ".g"].T)
    return o @ w[p + ".o"].T


def mixer(x, w, p, layer, eps):
    m = layer["mixer"]
    if layer["type"] == "parallel":
        left = chunked_attention_mixer(x, w, p + ".left", m["left"])
        right = gated_unit_mixer(x, w, p + ".right", m["right"])
    elif layer["type"] == "parallel_2":
        left = biased_attention_mixer(x, w, p + ".left", m["left"], eps)
        right = retention_mixer(x, w, p + ".right", m["right"], eps)
    else:
        raise ValueError(layer["type"])
    return 0.5 * (rms_unit(left, eps) * w[p + ".left.out"] + rms_unit(right, eps) * w[p + ".right.out"])


# ---------------------------------------------------------------------------
# feed-forward
# ---------------------------------------------------------------------------

def gated_unit(x, w, p, act):
    return (act(x @ w[p + ".gate"].T) * (x @ w[p + ".up"].T)) @ w[p + ".down"].T


# a list here collects, per routed layer run, the smallest gap between the last chosen and the first rejected logit
ROUTING_GAPS = None


def route(x, w, p, top):
    """Chosen experts [n, top] (largest logits first, ties to the lower index) and their weights: the softmax over
    the chosen logits alone."""
    z = x @ w[p + ".router"].T
    order = torch.sort(z, dim=-1, descending=True, stable=True).indices[:, :top]
    if ROUTING_GAPS is not None and z.shape[1] > top:
        ranked = torch.sort(z, dim=-1, descending=True).values
        ROUTING_GAPS.append(float((ranked[:, top - 1] - ranked[:, top]).min()))
    return order, torch.softmax(torch.gather(z, 1, order), dim=-1), z


def feed_forward(x, w, p, f):
    if f["kind"] == "dense":
        return gated_unit(x, w, p, gelu_tanh)
    experts, top = f["router"]["experts"], f["router"]["top"]
    ids, weights, _ = route(x, w, p, top)
    out = torch.zeros_like(x)
    for e in range(experts):
        y = gated_unit(x, w, f"{p}.e{e}", silu)
        out = out + y * (weights * (ids == e)).sum(-1, keepdim=True)
    if f.get("shared"):
        out = out + gated_unit(x, w, p + ".shared", silu) * torch.sigmoid(x @ w[p + ".shared.sg"].T)
    return out


# ---------------------------------------------------------------------------
# the model
# ---------------------------------------------------------------------------

def layer_runs(cfg):
    """[(layer, first of a pass)] in the order the layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    runs = [(i, False) for i in range(start)]
    for _ in range(times):
        runs += [(i, i == start) for i in range(start, stop)]
    return runs + [(i, False) for i in range(stop, n)]


def forward(tokens, w, cfg, dtype=torch.float64, streams=False):
    """Logits [n, vocab] of the whole sequence (and, with ``streams``, the residual stream after every layer run)."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    eps = float(cfg["norm"]["eps"])
    x0 = embedding(tokens, w, cfg)
    x, kept = x0, []
    for i, first in layer_runs(cfg):
        layer, p = cfg["layers"][i], f"l{i}"
        if first:
            x = torch.cat([x, x0], dim=-1) @ w["loop.in"].T
        x = x + layer_norm(mixer(layer_norm(x, w[p + ".norm1"], eps), w, p + ".mix", layer, eps), w[p + ".norm1b"], eps)
        if layer.get("mlp"):
            x = x + layer_norm(feed_forward(layer_norm(x, w[p + ".norm2"], eps), w, p + ".mlp", layer["mlp"]),
                               w[p + ".norm2b"], eps)
        kept.append(x)
    y = layer_norm(x, w["final.norm"], eps)
    logits = y @ w["embed"].T * float(cfg.get("logit_scale", 1.0))
    cap = float(cfg.get("logit_softcap", 0.0) or 0.0)
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return (logits, torch.stack(kept)) if streams else logits


def model_logits(folder, tokens, dtype=torch.float64, edit=None):
    """Logits of the model stored in ``folder`` (config.json, model.safetensors) for the whole sequence.
    ``edit(config)`` may change the configuration first (a test that asks what a mechanism is worth)."""
    import json
    from pathlib import Path

    from safetensors.torch import load_file

    cfg = json.loads((Path(folder) / "config.json").read_text())
    if edit is not None:
        edit(cfg)
    return forward(tokens, load_file(str(Path(folder) / "model.safetensors")), cfg, dtype)
