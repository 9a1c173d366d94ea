"""Small Pikurax configurations for the tests, and what the tests share.

The configurations differ from each other in every size and option: heads, key heads (one, some, as many as
heads), head sizes (multiples of 16 and not), rotated parts (whole heads, parts of them), chunks, values smaller
and larger than keys, temperatures and caps (also none), recurrent units of one and several parts with one to
five taps, retention heads, dense and routed feed-forwards (one expert, all experts chosen, with and without a
shared expert), layers without a feed-forward, loops from the first layer, over the middle, of one pass, and
none, embeddings with and without the pair table, eps, vocabulary, width (also no multiple of 8), page size.
"""

from __future__ import annotations

import json
from pathlib import Path

import torch


def chunked(heads, kv_heads, dim, rot_dims, chunk, width, blocks, conv, base=10000.0, scale=None):
    return {"type": "parallel", "mixer": {
        "left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": float(scale or dim ** -0.5),
                 "rot": {"dims": rot_dims, "base": float(base)}, "mask": {"size": chunk}},
        "right": {"width": width, "blocks": blocks, "conv": conv}}}


def biased(heads, kv_heads, dim, vdim, r_heads, r_dim, r_rot, r_vdim, decay, q_temp=(0.3, 16), softcap=8.0, base=10000.0,
           scale=None):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": float(scale or dim ** -0.5)}
    if q_temp is not None:
        left["q_temp"] = {"coef": float(q_temp[0]), "every": int(q_temp[1])}
    if softcap is not None:
        left["softcap"] = float(softcap)
    return {"type": "parallel_2", "mixer": {
        "left": left,
        "right": {"heads": r_heads, "dim": r_dim, "vdim": r_vdim, "rot": {"dims": r_rot, "base": float(base)},
                  "decay": [float(d) for d in decay]}}}


def dense(layer, ff):
    return {**layer, "mlp": {"kind": "dense", "ff": ff}}


def moe(layer, experts, top, ff, shared=None):
    f = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared is not None:
        f["shared"] = {"ff": shared}
    return {**layer, "mlp": f}


def bare(layer):
    return {**layer, "mlp": None}


def model(width, vocab, eps, layers, loop=None, pairs=(61, 7, 3), scale=4.0, logit_scale=1.5, logit_softcap=20.0):
    cfg = {"architecture": "Pikurax", "width": width, "vocab": vocab, "norm": {"eps": eps}, "layers": list(layers),
           "embedding": {"scale": float(scale)}, "logit_scale": float(logit_scale)}
    if pairs is not None:
        cfg["embedding"]["bigram"] = {"buckets": pairs[0], "mul_prev": pairs[1], "mul_cur": pairs[2]}
    if logit_softcap is not None:
        cfg["logit_softcap"] = float(logit_softcap)
    if loop is not None:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


# S: both kinds of layer, every kind of feed-forward, a loop over the middle
MODEL_S = model(72, 193, 1e-5, [
    dense(chunked(3, 3, 16, 8, 24, 40, 5, 4), 56),
    moe(biased(4, 2, 24, 16, 3, 8, 4, 24, (0.9, 0.97, 0.995)), 5, 2, 24, shared=40),
    moe(chunked(4, 1, 32, 32, 40, 48, 2, 2, base=500.0), 3, 1, 16),
    bare(biased(2, 2, 16, 40, 2, 16, 16, 8, (0.99, 0.5), q_temp=None, softcap=None)),
], loop=(1, 3, 3))
PAGE_S = 16

# T: heads the tensor-core attention takes (64 and 128), sizes the tensor-core products take, forty experts,
# a loop from the first layer, a large pair table
MODEL_T = model(128, 211, 3e-6, [
    moe(chunked(6, 3, 64, 32, 80, 160, 8, 3, base=250000.0), 40, 4, 72, shared=104),
    dense(biased(2, 1, 128, 128, 4, 32, 32, 64, (0.97, 0.98, 0.99, 0.999), q_temp=(0.5, 48), softcap=30.0), 256),
    moe(chunked(2, 2, 128, 64, 200, 128, 1, 5), 6, 6, 40),
], loop=(0, 2, 2), pairs=(1009, 31, 7), scale=11.0)
PAGE_T = 8

# U: odd sizes everywhere: a width and a vocabulary that are no multiples of 8, heads of 10 and 12 elements,
# one expert, no loop, no pair table, no cap on the logits, one tap
MODEL_U = model(52, 101, 2e-6, [
    moe(chunked(3, 1, 10, 6, 7, 26, 2, 1, base=77.0), 1, 1, 27, shared=13),
    dense(biased(3, 3, 12, 6, 1, 6, 2, 10, (0.9,), q_temp=(1.0, 5), softcap=2.0), 30),
    moe(biased(2, 1, 10, 14, 3, 10, 10, 6, (1.0, 0.8, 0.95), q_temp=None, softcap=50.0), 7, 7, 10),
    bare(chunked(1, 1, 20, 20, 300, 13, 13, 3)),
], pairs=None, scale=1.0, logit_scale=1.0, logit_softcap=None)
PAGE_U = 32

MODELS = {"S": (MODEL_S, PAGE_S), "T": (MODEL_T, PAGE_T), "U": (MODEL_U, PAGE_U)}


def layers_model(layers, width=48, vocab=97, eps=1e-5, **kw):
    return model(width, vocab, eps, list(layers), **kw)


def random_config(seed: int) -> dict:
    """A configuration drawn from a seed: widths of 128 to 512, three to seven layers of either kind in any order, heads
    of 32 to 128 elements on one to four key heads, chunks of 48 to 384, units of one to eight parts and two to five
    taps, retention heads of 16 to 64 key elements, any feed-forward, loops anywhere or none."""
    import random

    r = random.Random(seed)
    width, vocab = r.choice([128, 192, 256, 320, 384, 512]), r.choice([257, 384, 500, 512, 1000])
    layers = []
    for _ in range(r.choice([3, 4, 5, 6, 7])):
        kv = r.choice([1, 2, 4])
        heads = kv * r.choice([1, 2, 4])
        if r.random() < 0.6:
            dim = r.choice([32, 48, 64, 96, 128])
            parts = r.choice([1, 2, 4, 8])
            layer = chunked(heads, kv, dim, r.choice([dim, dim // 2, 16]), r.choice([48, 64, 100, 128, 384]),
                            parts * r.choice([16, 40, 64]), parts, r.choice([2, 3, 4, 5]), base=r.choice([1e4, 1e6, 2e5]),
                            scale=r.choice([dim ** -0.5, 0.1, 0.2]))
        else:
            dim, vdim = r.choice([32, 64, 96, 128]), r.choice([32, 64, 96])
            r_heads, r_dim = r.choice([2, 3, 4, 6]), r.choice([16, 32, 64])
            layer = biased(heads, kv, dim, vdim, r_heads, r_dim, r.choice([r_dim, r_dim // 2]), r.choice([32, 64]),
                           [1.0 - 2.0 ** -r.randint(3, 10) for _ in range(r_heads)],
                           q_temp=r.choice([None, (0.3, 64), (0.1, 16)]), softcap=r.choice([None, 20.0, 50.0]),
                           base=r.choice([1e4, 1e6]), scale=r.choice([dim ** -0.5, 0.1]))
        kind = r.random()
        if kind < 0.15:
            layers.append(bare(layer))
        elif kind < 0.45:
            layers.append(dense(layer, r.choice([128, 256, 384])))
        else:
            experts = r.choice([4, 8, 12])
            layers.append(moe(layer, experts, r.choice([1, 2, 3]), r.choice([32, 64, 96]),
                              shared=r.choice([None, 64, 96, 128])))
    loop = None
    if r.random() < 0.75:
        start = r.randrange(len(layers))
        stop = r.randint(start + 1, len(layers))
        loop = (start, stop, r.choice([1, 2, 3]))
    return model(width, vocab, r.choice([1e-6, 1e-5]), layers, loop=loop,
                 pairs=r.choice([None, (509, 31, 7), (4093, 257, 5)]), scale=r.choice([1.0, 8.0, 12.0]),
                 logit_scale=r.choice([1.0, 2.5]), logit_softcap=r.choice([None, 25.0]))


INIT_STD = 0.15


def make_folder(tmp_path, config, seed: int, dtype: str, init_std: float = INIT_STD, edit=None) -> Path:
    """A model folder of random weights; ``edit(tensors)`` may change them before they are written (a test that
    needs weights which make a fault show)."""
    from safetensors.torch import save_file

    from lockstep_b200.config import config_from_dict
    from lockstep_b200.engine.model import expected_weights
    from lockstep_b200.weights.random_init import random_tensors

    folder = Path(tmp_path) / f"pikurax-{seed}-{dtype}"
    folder.mkdir(parents=True, exist_ok=True)
    cfg = config_from_dict(config)
    tensors = random_tensors(expected_weights(cfg.model_spec()), seed, dtype, init_std, 0.1)
    for name in tensors:
        # a pair table as large as the token table's rows, routers whose logits lie well apart
        if name == "bigram" or name.endswith(".router"):
            tensors[name] = (tensors[name].float() * 4.0).to(tensors[name].dtype)
    if edit is not None:
        edit(tensors)
    (folder / "config.json").write_text(json.dumps(cfg.to_dict(), indent=1))
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(folder / "model.safetensors"))
    return folder


def plain_logits(folder, tokens, edit=None) -> torch.Tensor:
    from plain import pikurax_plain as plain

    return plain.model_logits(folder, tokens, torch.float64, edit=edit)


def plain_logits_and_gap(folder, tokens):
    """The plain logits, and the smallest gap between a chosen and a rejected router logit anywhere in the run (inf
    where nothing is routed): where it is tiny, float32 rounding decides a choice, and every later row of the request
    carries the other expert through the recurrent states."""
    from plain import pikurax_plain as plain

    plain.ROUTING_GAPS = []
    try:
        logits = plain.model_logits(folder, tokens, torch.float64)
        return logits, min(plain.ROUTING_GAPS, default=float("inf"))
    finally:
        plain.ROUTING_GAPS = None


# Error bounds relative to 1 + the request's largest plain logit (see kemirax_models: float32 the rounding of
# sums and carried states; bfloat16 the rounding of every product's output).
TOLERANCE = {"float32": 4e-5, "bfloat16": 8e-2}
# In bfloat16 a router's input carries the rounding of everything before it; where two logits lie closer than that
# the engine and the plain run choose differently, and the row differs by an expert's output, rightly.  Behind a
# routed layer the recurrent states carry the difference to every later row of the request, so a model that routes in
# front of them, several passes long, may have most rows of its long requests off in bfloat16 (PERSISTENT): its
# float32 run, on requests without a close call, is what holds every row.
CLOSE_CALLS = {"float32": 0.0, "bfloat16": 0.10}
PERSISTENT = 0.7


def assert_close(rows, plain_by_uid, dtype, what, close_calls=None, slack=1.0):
    worst, bad = 0.0, []
    for (uid, pos), got in sorted(rows.items()):
        want = plain_by_uid[uid][pos].float()
        err = float((got - want).abs().max()) / (1.0 + float(plain_by_uid[uid].abs().max()))
        worst = max(worst, err)
        if not err <= slack * TOLERANCE[dtype]:
            bad.append((uid, pos, err))
    allowed = int((CLOSE_CALLS[dtype] if close_calls is None else close_calls) * len(rows))
    assert len(bad) <= allowed, (
        f"{what}: {len(bad)} of {len(rows)} rows are off ({allowed} allowed); the first is request {bad[0][0]} "
        f"position {bad[0][1]}: relative error {bad[0][2]:.3e} > {slack * TOLERANCE[dtype]:.1e}")
    return worst
