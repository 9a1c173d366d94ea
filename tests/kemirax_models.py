"""Small Kemirax configurations for the tests, and what the tests share.

The configurations differ from each other in every size and option: heads, plain, rotated and
value sizes of the latent layers (all unequal), latents of keys and of queries of different ranks,
layers that read another layer's cached latents (one, two readers of one layer; the first layer
of either kind), frequency stretching (also none), heads and sizes of the linear layers, experts
(one, several, more than a warp has lanes), identity experts (none, more than real ones), top (one,
all), limits of experts and of the shared expert (unequal), layers without a shared expert and
without a feed-forward, eps, vocabulary, width (also no multiple of 8), page size.
"""

from __future__ import annotations

import json
from pathlib import Path

import torch


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, kv_from=None, base=10000.0, scaling=None, scale=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
         "scale": float(scale if scale is not None else (dim + rot_dim) ** -0.5),
         "rot": {"dims": rot_dim, "base": float(base)}}
    if scaling is not None:
        m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), map(float, scaling)))
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m}


def gla(heads, dim, vdim, tau=8.0, decay_rank=5):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": float(tau), "decay_rank": decay_rank}}


def with_moe(layer, experts=None, identity=0, top=1, ff=16, limit=1.5, shared=None):
    """``shared``: (ff, limit) of the shared expert, or None."""
    layer = dict(layer)
    if experts is None:
        layer["mlp"] = None
        return layer
    layer["mlp"] = {"kind": "moe", "expert": {"ff": ff, "limit": float(limit)},
                    "router": {"experts": experts, "identity": identity, "top": top}}
    if shared is not None:
        layer["mlp"]["shared"] = {"ff": shared[0], "limit": float(shared[1])}
    return layer


def model(width, vocab, eps, layers):
    return {"architecture": "Kemirax", "width": width, "vocab": vocab, "norm": {"eps": eps}, "layers": layers}


# S: both mixers, two readers of the first latent layer's cache, every option of the feed-forward once
MODEL_S = model(72, 193, 1e-5, [
    with_moe(latent(3, 16, 8, 24, 40, 20, scaling=(4.0, 64, 8.0, 1.0)), experts=5, identity=2, top=2, ff=24, limit=1.2, shared=(40, 0.7)),
    with_moe(gla(2, 24, 40, tau=4.0), experts=3, identity=0, top=3, ff=16),
    with_moe(latent(2, 24, 8, 16, 40, 36, kv_from=0, scaling=(4.0, 64, 8.0, 1.0)), experts=1, identity=3, top=2, ff=32, limit=0.6),
    with_moe(gla(3, 8, 16, decay_rank=2)),
    with_moe(latent(4, 8, 8, 8, 40, 12, kv_from=0, scaling=(4.0, 64, 8.0, 1.0)), experts=4, identity=1, top=1, ff=8, shared=(8, 2.5)),
    with_moe(latent(1, 40, 16, 48, 24, 56, base=500.0), experts=2, identity=0, top=1, ff=48, limit=3.0),
])
PAGE_S = 16

# T: starts with a linear layer; a cached row (latent + rotated part) of 128 and one of 64 elements,
# which the tensor-core attention takes in bfloat16; sizes the tensor-core products take (multiples
# of 8); forty experts (more than a warp's lanes)
MODEL_T = model(128, 211, 3e-6, [
    with_moe(gla(2, 64, 32, tau=16.0, decay_rank=8), experts=40, identity=8, top=4, ff=64, limit=2.0, shared=(96, 1.0)),
    with_moe(latent(4, 32, 16, 48, 112, 64, scaling=(2.0, 32, 4.0, 0.5)), experts=6, identity=6, top=3, ff=128, limit=1.0),
    with_moe(latent(2, 64, 16, 16, 112, 80, kv_from=1, scaling=(2.0, 32, 4.0, 0.5)), experts=2, identity=1, top=2, ff=40, shared=(24, 0.5)),
    with_moe(latent(8, 16, 8, 24, 56, 32, base=1000.0), experts=3, identity=0, top=2, ff=72, limit=0.9),
])
PAGE_T = 8

# U: odd sizes everywhere: a width and a vocabulary that are no multiples of 8 (no row pitch of 16
# bytes: the CUDA-core products also in bfloat16), heads of 10, 6 and 12, latents of 21 and 5, ranks of 1,
# an expert of 27, only identity experts beside one real one, all experts chosen
MODEL_U = model(52, 101, 2e-6, [
    with_moe(latent(3, 10, 6, 14, 21, 5, base=77.0, scaling=(1.5, 40, 6.0, 0.7)), experts=1, identity=2, top=3, ff=27, limit=0.9, shared=(13, 1.1)),
    with_moe(gla(3, 6, 10, tau=3.0, decay_rank=1), experts=7, identity=0, top=7, ff=10),
    with_moe(latent(1, 12, 6, 22, 21, 1, kv_from=0, base=77.0, scaling=(1.5, 40, 6.0, 0.7))),
    with_moe(gla(1, 40, 6, tau=1.0, decay_rank=3), experts=2, identity=5, top=2, ff=14, shared=(30, 0.4)),
])
PAGE_U = 32

MODELS = {"S": (MODEL_S, PAGE_S), "T": (MODEL_T, PAGE_T), "U": (MODEL_U, PAGE_U)}


def layers_model(layers, width=48, vocab=97, eps=1e-5):
    return model(width, vocab, eps, list(layers))


def random_config(seed: int) -> dict:
    """A configuration drawn from a seed: widths of 192 to 512, six to twelve layers in any order of the two
    mixers, readers of any earlier lender, cached rows of 80 to 256 elements, experts with and without identity and
    shared experts, layers without a feed-forward."""
    import random

    r = random.Random(seed)
    width, vocab = r.choice([256, 320, 384, 448, 512, 192]), r.choice([384, 500, 512, 640, 1000])
    rot_dim = r.choice([16, 32, 64])
    kv_rank = r.choice([64, 96, 128, 160, 192 - (rot_dim if rot_dim == 64 else 0)])
    scaling = None
    if r.random() < 0.8:
        scaling = (r.choice([2.0, 4.0, 8.0, 16.0]), r.choice([256, 512, 1024, 2048]), r.choice([32.0, 16.0, 8.0]),
                   r.choice([1.0, 2.0, 0.5]))
    base = r.choice([10000.0, 500000.0, 1000.0])
    layers, lenders = [], []
    for i in range(r.choice([6, 8, 10, 12])):
        if r.random() < 0.3:
            layer = gla(r.choice([2, 4, 6]), r.choice([32, 48, 64, 128]), r.choice([32, 64, 96]), tau=r.choice([4.0, 16.0, 8.0]),
                        decay_rank=r.choice([8, 16, 24]))
        else:
            source = r.choice(lenders) if lenders and r.random() < 0.5 else None
            if source is None:
                lenders.append(i)
            dim = r.choice([16, 32, 48, 64])
            layer = latent(r.choice([2, 4, 6, 8]), dim, rot_dim, r.choice([16, 32, 64]), kv_rank, r.choice([48, 96, 128, 192]),
                           kv_from=source, base=base, scaling=scaling, scale=r.choice([0.125, (dim + rot_dim) ** -0.5, 0.2]))
        if r.random() < 0.1:
            layers.append(with_moe(layer))
        else:
            shared = None if r.random() < 0.15 else (r.choice([64, 96, 128, 192]), r.choice([1.0, 2.0, 5.0]))
            layers.append(with_moe(layer, experts=r.choice([4, 8, 12, 16]), identity=r.choice([0, 2, 4, 6]), top=r.choice([1, 2, 3, 4]),
                                   ff=r.choice([32, 64, 96, 128]), limit=r.choice([1.0, 2.0, 4.0, 7.0]), shared=shared))
    return model(width, vocab, r.choice([1e-6, 1e-5]), layers)


# standard deviation of the random matrices: rows are of unit size behind the norm, and larger weights
# make every softmax a choice of one key (the tests that want that ask for it)
INIT_STD = 0.15


def make_folder(tmp_path, config, seed: int, dtype: str, init_std: float = INIT_STD, edit=None) -> Path:
    """A model folder of random weights; ``edit(tensors)`` may change them before they are
    written (a test that needs weights which make a fault show)."""
    from safetensors.torch import save_file

    from lockstep_b200.config import config_from_dict
    from lockstep_b200.engine.model import expected_weights
    from lockstep_b200.weights.random_init import random_tensors

    folder = Path(tmp_path) / f"kemirax-{seed}-{dtype}"
    folder.mkdir(parents=True, exist_ok=True)
    cfg = config_from_dict(config)
    tensors = random_tensors(expected_weights(cfg.model_spec()), seed, dtype, init_std, 0.1)
    for name in tensors:
        # corrections as large as the gaps between scores, so that they change choices; gates' matrices
        # large enough for gates away from one half
        if name.endswith(".correction"):
            tensors[name] = (tensors[name].float() * 10.0).to(tensors[name].dtype)
        if name.endswith((".rg1", ".rg2")):
            tensors[name] = (tensors[name].float() * 3.0).to(tensors[name].dtype)
    if edit is not None:
        edit(tensors)
    (folder / "config.json").write_text(json.dumps(cfg.to_dict(), indent=1))
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(folder / "model.safetensors"))
    return folder


def plain_logits(folder, tokens) -> torch.Tensor:
    from plain import kemirax_plain as plain

    return plain.model_logits(folder, tokens, torch.float64)


# Error bounds relative to 1 + the request's largest plain logit: in float32 the rounding of sums
# a few hundred terms long and of a state carried over a few hundred tokens (a product or a state
# that lost mantissa bits would be a hundred times above it); in bfloat16 the rounding of every
# product's output to 8 bits of mantissa.
TOLERANCE = {"float32": 4e-5, "bfloat16": 6e-2}
# In bfloat16 a router's input carries the rounding of everything before it, and where two experts'
# choice scores lie closer than that, the engine and the plain run choose differently: the row then
# differs by an expert's output times its weight, rightly.  So a few rows of a bfloat16 run may be
# off; float32 has no such rows, and it is the float32 run that holds every row to its bound.
CLOSE_CALLS = {"float32": 0.0, "bfloat16": 0.10}


def assert_close(rows, plain_by_uid, dtype, what, close_calls=None, slack=1.0):
    """``slack``: a factor on the bound, for weights that amplify rounding on purpose."""
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
