"""Kemirax on the device against the plain implementation: the kernels of every mechanism alone
(the norm with one number, the token shift and the row it carries, the gated sum, queries through
a latent, a layer that reads another's cached latents, softmax routing with a correction, identity
and shared experts), one-layer models, and whole models cut in four ways (whole prompts; a prompt
and then token by token; portions down to two tokens; up to three live requests, portions of some
beside single tokens of others, on so few pages and slots that they are used again), in float32
and bfloat16; weights made so that a far key, a lost shift row, a lost state or a wrong expert
shows; greedy generation through the entry point and the scheduler; the command line; the trace
runner."""

from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import helpers as H
import kemirax_models as M
from plain import kemirax_plain as plain

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
DEV = "cuda:0"
F32, BF16 = torch.float32, torch.bfloat16


def make_runner(folder, dtype, page, steps=None, max_live=3, num_pages=None, **kw):
    from lockstep_b200.engine import ModelRunner

    if num_pages is None:
        num_pages = H.max_live_tokens(steps, round_to=page) // page
    return ModelRunner(folder, dtype=dtype, num_pages=num_pages, page_size=page, max_live=max_live,
                       max_seq_len=1024, **kw)


PLANS = {
    "whole": H.plan_whole,
    "then_single": lambda r: H.plan_bulk_then_single(r, tail=70),
    "portions": lambda r: H.plan_portions(r, sizes=(7, 2, 17, 3, 33, 2, 5, 64, 1, 2, 150)),
    "mixed": lambda r: H.plan_mixed(r, max_live=3),
}


# ---------------------------------------------------------------------------
# kernels alone
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("width", [72, 52, 320, 7])
def test_norm_with_one_number(dtype, width):
    from lockstep_b200 import kernels as K
    from lockstep_b200.config.spec import PartSpec
    from lockstep_b200.parts import Runtime
    from lockstep_b200.parts.base import build_part

    g = torch.Generator().manual_seed(width)
    rt = Runtime(device=torch.device(DEV), dtype=dtype, page_size=16, max_positions=8, err=K.new_error_word(DEV))
    norm = build_part("norm", PartSpec("rmsnorm", {"width": width, "eps": 1e-3, "tensor": "", "scalar": True}), rt)
    assert norm.weight_specs()[""].shape == ()
    gain = torch.tensor(1.7).to(dtype)
    norm.bind({"": gain.to(DEV)})
    x = torch.randn(9, width, generator=g) * torch.linspace(0.01, 20.0, 9)[:, None]     # rows well below and above eps
    got = norm.forward(x.to(DEV))
    want = plain.scalar_rms_norm(x.double(), gain.double(), 1e-3)
    K.raise_on_fault(rt.err)
    assert float((got.cpu().double() - want).abs().max()) < (3e-6 if dtype == F32 else 2e-2)
    # eps sits inside the root: the smallest row is far from unit size
    assert float(want[0].pow(2).mean().sqrt()) < 0.9 * 1.7 < float(want[-1].pow(2).mean().sqrt()) / 0.999


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("width", [40, 52, 256])
def test_token_shift_carries_a_row_and_the_gated_sum_keeps_it(dtype, width):
    """Three requests in portions over several calls: every row moves towards the row before it,
    also across calls (the row a slot carries), a request's first row towards zeros; the closing
    kernel adds the gated branches and keeps each portion's last row."""
    from lockstep_b200 import kernels as K

    g = torch.Generator().manual_seed(width)
    lengths = {2: 13, 0: 5, 1: 8}
    rows = {s: torch.randn(n, width, generator=g).to(dtype) for s, n in lengths.items()}
    mix = torch.rand(1, width, generator=g)
    want = {s: plain.shifted(r.double(), mix.double()[0]) for s, r in rows.items()}
    state = torch.zeros(4, width + 3, device=DEV)
    state[3] = 5.0                                        # a slot nobody uses stays as it is
    bias = torch.randn(2 * width, generator=g)
    got, at_row = {}, {}

    def call(pieces):
        y = torch.cat([rows[s][a:a + c] for s, a, c in pieces]).to(DEV)
        n = y.shape[0]
        slot = torch.tensor(sum(([s] * c for s, a, c in pieces), []), dtype=torch.int32, device=DEV)
        out = torch.empty(1, n, width, dtype=dtype, device=DEV)
        K.shift_mix(y, mix.to(DEV), state, 0, slot, out)
        at = 0
        for s, a, c in pieces:
            got[(s, a)] = out[0, at:at + c].cpu().double()
            at += c
        # the closing kernel: a gated sum of two branches into the stream, and the carried rows
        h = torch.randn(n, width, generator=g)
        branches = torch.randn(2, n, width, generator=g)
        z = torch.randn(n, 2 * width, generator=g) * 2
        stream = h.to(DEV)
        K.gated_sum(stream, branches.to(DEV), z.to(DEV), bias.to(DEV), carry=(y, state, slot))
        gates = torch.sigmoid(z.double() + bias.double())
        ref = h.double() + gates[:, :width] * branches[0].double() + gates[:, width:] * branches[1].double()
        assert float((stream.cpu().double() - ref).abs().max()) < 1e-5
        plain_sum = h.to(DEV)
        K.gated_sum(plain_sum, branches.to(DEV), None, None)
        assert float((plain_sum.cpu().double() - h.double() - branches.double().sum(0)).abs().max()) < 1e-5
        for s, a, c in pieces:
            at_row[s] = a + c - 1

    call([(2, 0, 6), (0, 0, 5), (1, 0, 1)])
    for s in (2, 0, 1):
        assert torch.equal(state[s, :width].cpu(), rows[s][at_row[s]].float())
    call([(1, 1, 2), (2, 6, 1)])
    call([(2, 7, 1)])
    call([(2, 8, 5), (1, 3, 5)])
    tol = 1e-6 if dtype == F32 else 2e-2
    for (s, a), r in got.items():
        assert float((r - want[s][a:a + r.shape[0]]).abs().max()) < tol, (s, a)
    assert float(state[3].min()) == 5.0 and float(state[3].max()) == 5.0
    assert float(state[:3, width:].abs().sum()) == 0.0     # only the row's own columns are written
    # the shift matters: unshifted rows are something else, and so is a first row that forgot the row before it
    assert float((want[2] - rows[2].double()).abs().max()) > 0.1


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("width", [40, 52, 7, 1024])
def test_norm_and_shift_in_one_pass_give_the_bits_of_the_two_in_turn(dtype, width):
    from lockstep_b200 import kernels as K

    g = torch.Generator().manual_seed(width)
    slots = [2] * 5 + [0] * 1 + [1] * 3 + [3] * 1100          # (more than a thousand rows: four rows a block)
    tokens = len(slots)
    h = (torch.randn(tokens, width, generator=g) * torch.linspace(0.05, 9.0, tokens)[:, None]).to(DEV)
    gain = torch.full((width,), 1.3).to(dtype).to(DEV)
    mu = torch.rand(1, width, generator=g).to(DEV)
    state = torch.randn(5, width + 4, generator=g).to(DEV)
    slot = torch.tensor(slots, dtype=torch.int32, device=DEV)
    err = K.new_error_word(DEV)
    y0 = torch.empty(tokens, width, dtype=dtype, device=DEV)
    K.rmsnorm(h, gain, y0, 1e-4, err)
    x0 = torch.empty(1, tokens, width, dtype=dtype, device=DEV)
    K.shift_mix(y0, mu, state, 0, slot, x0)
    y1, x1 = torch.empty_like(y0), torch.empty_like(y0)
    K.rmsnorm_shift(h, gain, 1e-4, mu, state, slot, y1, x1)
    K.raise_on_fault(err)
    assert torch.equal(y0, y1) and torch.equal(x0[0], x1)
    want = plain.scalar_rms_norm(h.double().cpu(), torch.tensor(1.3).to(dtype).double(), 1e-4)
    assert float((y1.double().cpu() - want).abs().max()) < (5e-6 if dtype == F32 else 3e-2)
    # every portion's first row leans on its slot's carried row, the others on the row before
    first = plain.shifted(want[:5], mu.double().cpu()[0], before=state[2, :width].double().cpu())
    assert float((x1[:5].double().cpu() - first).abs().max()) < (1e-5 if dtype == F32 else 6e-2)


@pytest.mark.parametrize("experts, top", [(12, 3), (5, 5), (40, 4), (1, 1), (300, 7)])
def test_softmax_routing_chooses_by_corrected_scores_and_weighs_by_plain_ones(experts, top):
    from lockstep_b200 import kernels as K

    g = torch.Generator().manual_seed(experts)
    tokens = 33
    logits = torch.randn(tokens, experts + 2, generator=g) * 2          # two more columns that are not experts
    logits[:, experts:] = 50.0                                          # (they would win every choice and take all the weight)
    correction = torch.randn(experts, generator=g) * 0.2
    ids = torch.empty(tokens, top, dtype=torch.int32, device=DEV)
    weights = torch.empty(tokens, top, device=DEV)
    K.experts_route(logits.to(DEV), top, ids, weights, experts=experts, softmax=True, correction=correction.to(DEV))
    w = {"r.router": torch.eye(experts, dtype=torch.float64), "r.correction": correction.double()}
    want_ids, want_w = plain.route(logits[:, :experts].double(), w, "r", {"top": top})
    scores = torch.softmax(logits[:, :experts].double(), -1)
    choice = scores + correction.double()
    # a token whose choice hangs on float32 rounding is left out (there are few)
    ranked = choice.sort(-1, descending=True).values
    gaps = (ranked[:, :-1] - ranked[:, 1:])[:, :top].min(-1).values if experts > 1 else torch.ones(tokens)
    sure = gaps > 1e-6
    assert int(sure.sum()) >= tokens - 3
    assert torch.equal(ids.cpu().long()[sure], want_ids[sure])
    assert float((weights.cpu().double()[sure] - want_w[sure]).abs().max()) < 1e-6
    if 1 < top < experts:
        # the correction changes choices, and the weights are not renormalised
        assert not torch.equal(want_ids, torch.sort(scores, dim=-1, descending=True, stable=True).indices[:, :top])
        assert float(want_w.sum(-1).max()) < 0.999


@pytest.mark.parametrize("tokens, real, identity, top", [(1, 5, 2, 3), (8, 32, 4, 4), (32, 40, 0, 7), (19, 1, 6, 2)])
def test_choice_and_plan_in_one_launch_are_those_of_the_two_in_turn(tokens, real, identity, top):
    from lockstep_b200 import kernels as K

    g = torch.Generator().manual_seed(tokens)
    experts, pairs, tile = real + identity, tokens * top, 64
    logits = (torch.randn(tokens, experts + 3, generator=g) * 2).to(DEV)
    correction = (torch.randn(experts, generator=g) * 0.2).to(DEV)
    max_tiles = min(pairs, pairs // tile + real)
    err = K.new_error_word(DEV)

    def buffers():
        i32, f32 = torch.int32, torch.float32
        return dict(ids=torch.full((tokens, top), -7, dtype=i32, device=DEV), weights=torch.zeros(tokens, top, device=DEV),
                    plan=torch.full((1 + 3 * max_tiles,), -7, dtype=i32, device=DEV),
                    row_token=torch.full((pairs,), -7, dtype=i32, device=DEV), row_weight=torch.full((pairs,), -7.0, device=DEV),
                    pair_row=torch.full((pairs,), -7, dtype=i32, device=DEV))

    a, b = buffers(), buffers()
    K.experts_route(logits, top, a["ids"], a["weights"], experts=experts, softmax=True, correction=correction)
    K.experts_plan(a["ids"], a["weights"], real, tile, a["plan"], max_tiles, a["row_token"], a["row_weight"], a["pair_row"], err)
    K.experts_route_plan(logits, top, b["ids"], b["weights"], experts, True, correction, real, tile, b["plan"], max_tiles,
                         b["row_token"], b["row_weight"], b["pair_row"], err)
    K.raise_on_fault(err)
    assert torch.equal(a["ids"], b["ids"]) and torch.equal(a["weights"], b["weights"])
    tiles = int(a["plan"][0])
    assert tiles == int(b["plan"][0]) and torch.equal(a["plan"][:1 + 3 * tiles], b["plan"][:1 + 3 * tiles])
    # rows of one expert may come in either order (they are handed out by atomic counters): the sets agree
    real_pair = (a["ids"].flatten() < real).cpu()
    assert torch.equal(a["pair_row"].cpu()[real_pair].sort().values, b["pair_row"].cpu()[real_pair].sort().values)
    for name in ("a", "b"):
        d = a if name == "a" else b
        rows = d["pair_row"].cpu()[real_pair].long()
        assert torch.equal(d["row_token"].cpu()[rows].long(), (torch.arange(pairs) // top)[real_pair])
        assert torch.equal(d["row_weight"].cpu()[rows], d["weights"].flatten().cpu()[real_pair])


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("store", [False, True])
def test_mixing_real_identity_and_shared_experts(dtype, store):
    from lockstep_b200 import kernels as K

    g = torch.Generator().manual_seed(3)
    tokens, top, width, real, identity = 19, 3, 44, 4, 3
    ids = torch.stack([torch.randperm(real + identity, generator=g)[:top] for _ in range(tokens)]).to(torch.int32)
    ids[0] = torch.tensor([4, 5, 6])                 # a token of identity experts alone
    ids[1] = torch.tensor([0, 1, 2])                 # and one of real experts alone
    weights = torch.rand(tokens, top, generator=g)
    y = torch.randn(tokens * top, width, generator=g)
    pair_row = torch.randperm(tokens * top, generator=g).view(tokens, top).to(torch.int32)
    x = torch.randn(tokens, width, generator=g).to(dtype)
    shared = torch.randn(tokens, width, generator=g)
    logits = torch.randn(tokens, real + identity + 1, generator=g)       # the gate's logit is the last column
    before = torch.randn(tokens, width, generator=g)
    for with_shared, with_gate in ((True, True), (True, False), (False, False)):
        out = before.to(DEV)
        K.experts_mix(y.to(DEV), pair_row.to(DEV), ids.to(DEV), weights.to(DEV), real, x.to(DEV), out,
                      shared=shared.to(DEV) if with_shared else None,
                      shared_gate=logits.to(DEV)[:, real + identity:] if with_gate else None, store=store)
        want = torch.zeros(tokens, width, dtype=torch.float64) if store else before.double().clone()
        for t in range(tokens):
            for r in range(top):
                src = y[pair_row[t, r]].double() if ids[t, r] < real else x[t].double()
                want[t] += weights[t, r].double() * src
        if with_shared:
            gate = torch.sigmoid(logits[:, -1:].double()) if with_gate else 1.0
            want += gate * shared.double()
        assert float((out.cpu().double() - want).abs().max()) < 2e-5


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("heads, d, dr, dv, rank, few", [(3, 16, 8, 24, 40, True), (2, 24, 10, 8, 21, False),
                                                         (1, 40, 16, 48, 24, True), (5, 8, 32, 16, 96, False)])
def test_latent_rows_from_a_product_of_their_own_rotate_halves(dtype, heads, d, dr, dv, rank, few):
    """The queries come from one product and the latent with the shared key part from another;
    element i of a rotated part is paired with element i + dr/2; with few tokens the same kernel
    folds W_uk into the queries, with the bits of the per-head product."""
    from lockstep_b200 import kernels as K

    g = torch.Generator().manual_seed(heads * 100 + rank)
    tokens, page, pad = 9, 8, -(-(rank + dr) // 16) * 16
    queries = torch.randn(tokens, heads * (d + dr), generator=g).to(dtype)
    kv = torch.randn(tokens, rank + dr + 3, generator=g).to(dtype)
    gain = (1 + 0.3 * torch.randn(rank, generator=g)).to(dtype)
    positions = torch.tensor([14, 15, 16, 17, 18, 19, 0, 1, 2], dtype=torch.int32)
    slot = torch.tensor([1] * 6 + [0] * 3, dtype=torch.int32)
    table = torch.tensor([[4, -1, -1], [2, 0, 3]], dtype=torch.int32)
    scaling = {"factor": 4.0, "original": 16.0, "fast": 4.0, "slow": 0.5}
    cos, sin = plain.rotary_tables(range(24), dr, 100.0, scaling)
    w_fold = (torch.randn(heads, rank, d, generator=g) * 0.3).to(dtype)
    err = K.new_error_word(DEV)
    outs = []
    for fold_inside in ((True, False) if few else (False,)):
        pages = torch.full((5, 2, 1, page, pad), 9.0, dtype=dtype, device=DEV)
        q_out = torch.full((tokens, heads * pad), 9.0, dtype=dtype, device=DEV)
        dev_q = queries.to(DEV)
        K.latent_finish(dev_q, q_out, pages, gain.to(DEV), cos.float().to(DEV), sin.float().to(DEV), positions.to(DEV),
                        slot.to(DEV), table.to(DEV), heads, d, dr, rank, pad, 1e-5, False, True, err,
                        w_fold=w_fold.to(DEV) if fold_inside else None, kv=kv.to(DEV))
        if not fold_inside:
            K.heads_product(dev_q, d + dr, w_fold.to(DEV), q_out, pad)
        K.raise_on_fault(err)
        outs.append((q_out.cpu(), pages.cpu()))
    if few:
        assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    q_out, pages = outs[0]
    pc, ps = cos[positions.long()], sin[positions.long()]
    q = queries.double().view(tokens, heads, d + dr)
    c = plain.unit_rms(kv.double()[:, :rank], 1e-5) * gain.double()
    k_rot = plain.rotate_halves(kv.double()[:, None, rank:rank + dr], pc, ps)[:, 0]
    tol = 4e-6 if dtype == F32 else 3e-2
    got_q = q_out.double().view(tokens, heads, pad)
    folded = torch.einsum("thd,hrd->thr", q[..., :d], w_fold.double())
    assert float((got_q[..., :rank] - folded).abs().max()) < tol * (1 + float(folded.abs().max()))
    assert float((got_q[..., rank:rank + dr] - plain.rotate_halves(q[..., d:], pc, ps)).abs().max()) < tol * 4
    assert float(got_q[..., rank + dr:].abs().sum()) == 0.0
    for t in range(tokens):
        pg = int(table[slot[t], positions[t] // page])
        row = pages[pg, :, 0, int(positions[t]) % page].double()
        assert float((row[0, :rank] - c[t]).abs().max()) < tol * 4 and float((row[1, :rank] - c[t]).abs().max()) < tol * 4
        assert float((row[0, rank:rank + dr] - k_rot[t]).abs().max()) < tol * 4
        assert float(row[0, rank + dr:].abs().sum()) == 0.0 and float(row[1, rank:].abs().sum()) == 0.0
    # halves, not neighbours: the other pairing gives other numbers
    raw = kv.double()[:, rank:rank + dr]
    u, v = raw[:, 0::2], raw[:, 1::2]
    neighbours = torch.stack([u * pc - v * ps, v * pc + u * ps], -1).flatten(1)
    assert float((neighbours - k_rot).abs().max()) > 0.1


# ---------------------------------------------------------------------------
# models: one or two layers of each mechanism, then whole models, in four cuttings
# ---------------------------------------------------------------------------

_STRETCH = (4.0, 32, 8.0, 1.0)
SMALL = {
    "latent": [M.with_moe(M.latent(3, 16, 8, 24, 40, 20, scaling=_STRETCH))],
    "latent_wide_rotation": [M.with_moe(M.latent(2, 8, 24, 8, 8, 56, base=300.0))],
    "latent_borrowed": [M.with_moe(M.latent(2, 16, 8, 16, 24, 16, scaling=_STRETCH)),
                        M.with_moe(M.latent(5, 8, 8, 24, 24, 40, kv_from=0, scaling=_STRETCH, scale=0.4))],
    "gla": [M.with_moe(M.gla(2, 24, 40, tau=4.0))],
    "gla_one_head": [M.with_moe(M.gla(1, 72, 8, tau=1.0, decay_rank=1))],
    "experts": [M.with_moe(M.gla(1, 16, 16), experts=6, identity=0, top=2, ff=24)],
    "experts_identity": [M.with_moe(M.gla(1, 16, 16), experts=2, identity=4, top=3, ff=40, limit=0.8)],
    "experts_shared": [M.with_moe(M.latent(1, 16, 8, 16, 24, 8), experts=40, identity=3, top=4, ff=8, limit=3.0, shared=(56, 0.5))],
    "experts_all_chosen": [M.with_moe(M.gla(2, 8, 8), experts=1, identity=1, top=2, ff=16, shared=(8, 2.0))],
}


@pytest.fixture(scope="module")
def zoo(tmp_path_factory):
    cache = {}

    def get(config, dtype, lengths, seed=7, edit=None, key=None):
        key = (key or str(config), dtype, tuple(lengths))
        if key not in cache:
            folder = M.make_folder(tmp_path_factory.mktemp("kemirax"), config, seed=seed, dtype=dtype, edit=edit)
            requests = {f"r{i}": H.random_tokens(n, config["vocab"], seed=50 + i) for i, n in enumerate(lengths)}
            cache[key] = (folder, requests, {u: M.plain_logits(folder, t).float() for u, t in requests.items()})
        return cache[key]

    return get


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(SMALL))
def test_small_models_in_every_cutting(zoo, name, dtype):
    folder, requests, want = zoo(M.layers_model(SMALL[name]), dtype, [45, 130, 9, 77])
    rows = {}
    for plan_name, plan in PLANS.items():
        steps = plan(requests)
        runner = make_runner(folder, dtype, 8, steps)
        rows[plan_name] = H.run_plan(runner, steps)
        # (without real experts no choice is a close call: every row is held to its bound)
        M.assert_close(rows[plan_name], want, dtype, f"{name}, {plan_name}", None if name.startswith("experts") else 0.0)
        runner.cache.audit()
    if dtype == "float32":
        # a row's arithmetic does not depend on how its request was cut or on the batch
        for plan_name in PLANS:
            for key, row in rows["whole"].items():
                assert torch.equal(row, rows[plan_name][key]), (name, plan_name, key)


LENGTHS = {"S": [70, 300, 37, 150, 129], "T": [45, 210, 90, 33, 260], "U": [40, 190, 75, 131]}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("plan_name", sorted(PLANS))
@pytest.mark.parametrize("model", sorted(M.MODELS))
def test_whole_models_in_every_cutting(zoo, model, plan_name, dtype):
    config, page = M.MODELS[model]
    folder, requests, want = zoo(config, dtype, LENGTHS[model])
    steps = PLANS[plan_name](requests)
    runner = make_runner(folder, dtype, page, steps)
    rows = H.run_plan(runner, steps)
    M.assert_close(rows, want, dtype, f"model {model}, {plan_name}")
    runner.cache.audit()
    if plan_name == "mixed":
        assert runner.cache.reused_pages() > 0           # more requests than slots, and few pages
    if plan_name == "then_single" and runner.graphs is not None:
        assert runner.graphs.replays > 100               # decoded tokens ran as recorded steps


@pytest.mark.parametrize("seed", [1, 4, 12])
def test_configurations_drawn_from_a_seed(zoo, seed):
    """Larger models of sizes nobody chose (see ``kemirax_models.random_config``), stored without the rank of the
    decay's map (it is the tensors' own), in float32: five requests of up to 520 tokens on four slots, portions of
    some beside single tokens of others.  How far float32 rounding moves the logits depends on the drawn weights
    (ten or twelve layers of random matrices amplify it, and a router's close call, a gap between two choice scores
    below the rounding of a sum, changes a row and, through a linear layer's state, hundreds after it), so the bound
    is what the plain implementation itself loses when it runs in float32: the engine may lose twice that."""
    config = M.random_config(seed)
    folder, requests, want = zoo(config, "float32", [70, 520, 37, 150, 260], seed=seed, key=f"drawn{seed}")
    stored = json.loads((folder / "config.json").read_text())
    for layer in stored["layers"]:
        layer["mixer"].pop("decay_rank", None)
    (folder / "config.json").write_text(json.dumps(stored))

    def spread(rows):
        errors = [float((got - want[uid][pos]).abs().max()) / (1.0 + float(want[uid].abs().max())) for (uid, pos), got in rows.items()]
        errors = torch.tensor(errors).sort().values
        return float(errors[len(errors) // 2]), float(errors[int(0.97 * len(errors))])

    plain32 = {u: plain.model_logits(folder, t, torch.float32) for u, t in requests.items()}
    allowed = spread({(u, p): plain32[u][p] for u, t in requests.items() for p in range(len(t))})
    assert allowed[0] < 1e-4                                   # (the drawn model is not beyond float32 altogether)
    for plan_name in ("whole", "mixed"):
        steps = PLANS[plan_name](requests) if plan_name == "whole" else H.plan_mixed(requests, max_live=4)
        runner = make_runner(folder, "float32", 16, steps, max_live=4)
        rows = H.run_plan(runner, steps)
        assert len(rows) == sum(len(t) for t in requests.values())
        median, bulk = spread(rows)
        assert median <= 2 * allowed[0] + 2e-6 and bulk <= 2 * allowed[1] + 1e-5, (seed, plan_name, median, bulk, allowed)
        runner.cache.audit()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sublayers_on_streams_of_their_own_give_the_bits_of_sublayers_in_turn(zoo, dtype):
    """In steps of few tokens the feed-forward and the gates' product run on streams of their own beside the mixer
    (recorded: branches of the graph).  The logits are those of a runner that takes them one after the other, bit
    for bit, in decoding (recorded steps), in portions of a few tokens and in mixed batches."""
    config, page = M.MODELS["S"]
    folder, requests, want = zoo(config, dtype, LENGTHS["S"])
    for plan_name in ("then_single", "portions", "mixed"):
        steps = PLANS[plan_name](requests)
        rows = {}
        for streams in (True, False):
            runner = make_runner(folder, dtype, page, steps)
            runner.rt.options["branch_streams"] = streams
            rows[streams] = H.run_plan(runner, steps)
            if plan_name == "then_single" and runner.graphs is not None:
                assert runner.graphs.replays > 100
        for key, row in rows[True].items():
            assert torch.equal(row, rows[False][key]), (plan_name, key)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_plain_model_reproduces_its_stream_layer_by_layer(zoo, dtype):
    """The residual stream after every layer run of the engine's own program against the plain
    model's: the first layer that differs is named."""
    from lockstep_b200.engine.batch import StepContext, StepEntry

    config, page = M.MODELS["S"]
    folder, requests, _ = zoo(config, dtype, LENGTHS["S"])
    tokens = requests["r2"]
    cfg, w = plain.read_model_folder(folder)
    trace = []
    plain.forward(cfg, w, tokens, trace=trace)
    runner = make_runner(folder, dtype, page, num_pages=8, use_graphs=False)
    runner.open("s")
    runner.cache.reserve("s", len(tokens))
    runner.cache.sync()
    ctx = StepContext([StepEntry("s", tokens, 0, [len(tokens) - 1])], [runner.cache.slots["s"]], runner.device,
                      runner.err, runner.split_size)
    h = None
    for i, (_, fn) in enumerate(runner.program):
        h = fn(h, ctx)
        if 1 <= i <= len(trace):
            err = float((h.double().cpu() - trace[i - 1]).abs().max()) / (1 + float(trace[i - 1].abs().max()))
            assert err < (1e-5 if dtype == "float32" else 5e-2), f"the stream differs after layer {i - 1}: {err:.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_of_a_repeating_shape_are_recorded_and_replayed(zoo, dtype):
    """Portions of 300 tokens with one wanted row: from its third occurrence the step is a
    recorded one (the portion list, the experts' work lists, the slots of the states and of the
    carried rows are all read on the device at replay), with the bits of an unrecorded step."""
    config, page = M.MODELS["S"]
    folder, requests, want = zoo(config, dtype, [900, 900, 601], key="recorded")
    steps = []
    for uid, toks in requests.items():
        for i in range(0, len(toks) - 1, 300):
            n = min(300, len(toks) - i)
            steps.append({"entries": [(uid, toks[i:i + n], [n - 1, 0])], "end": [uid] if i + n == len(toks) else []})
    steps.append({"entries": [("r2", requests["r2"][600:601], [0])], "end": ["r2"]})
    runner = make_runner(folder, dtype, page, steps, max_live=2)
    rows = H.run_plan(runner, steps)
    assert runner.graphs is not None and runner.graphs.mixed_replays >= 4
    M.assert_close(rows, want, dtype, "recorded steps of 300 tokens")
    fresh = make_runner(folder, dtype, page, steps, max_live=2, use_graphs=False)
    plain_rows = H.run_plan(fresh, steps)
    for key, row in rows.items():
        assert torch.equal(row, plain_rows[key]), key


# ---------------------------------------------------------------------------
# weights that make a fault show
# ---------------------------------------------------------------------------

def _sharpen(tensors):
    # large query weights make every row of a softmax pick one or two keys: a far key that is lost, or
    # a latent read from the wrong layer's pages, then changes the output by as much as a value
    for name in tensors:
        if name.endswith("mix.uq"):
            tensors[name] = (tensors[name].float() * 5.0).to(tensors[name].dtype)


def _softmax_weights(folder, tokens, at):
    """The softmax's weights [heads, n, n] of latent layer ``at`` of the plain model."""
    cfg, w = plain.read_model_folder(folder)
    x = w["embed"][torch.tensor(tokens)]
    caches = {}
    for i in range(at):
        x = plain.layer_forward(x, w, i, cfg, caches)
    eps = cfg["norm"]["eps"]
    h = plain.shifted(plain.scalar_rms_norm(x, w[f"l{at}.norm1"], eps), w[f"l{at}.shift"])
    m = cfg["layers"][at]["mixer"]
    src = m.get("kv_from")
    return plain.latent_attention_mixer(h, w, f"l{at}.mix", m, eps, None if src is None else caches[src], weights=True)[0]


def _tensor_core_attention_launches():
    from lockstep_b200 import kernels as K

    counts = K.kernel_counts()
    return counts.get("attention_prefill_tc", 0), counts.get("attention_decode_mma", 0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rank", [24, 56])
def test_sharp_latent_attention_reaches_far_keys_also_through_a_borrowed_cache(zoo, rank, dtype):
    # (a latent of 56 and a rotated part of 8 make a cached row of 64: in bfloat16 the tensor-core kernels)
    config = M.layers_model([M.with_moe(M.latent(4, 16, 8, 16, rank, 24, scale=0.5)),
                             M.with_moe(M.gla(1, 16, 16)),
                             M.with_moe(M.latent(2, 8, 8, 24, rank, 40, kv_from=0, scale=0.5))])
    folder, requests, want = zoo(config, dtype, [620, 300], edit=_sharpen, key=f"sharp{rank}")
    before = _tensor_core_attention_launches()
    for at in (0, 2):
        p = _softmax_weights(folder, requests["r0"], at)
        rows = torch.arange(p.shape[-1])[None, :]
        assert float(p.max(-1).values.median()) > 0.3             # most rows lean on one key
        assert int((p.argmax(-1) < rows - 200).sum()) >= 20        # for some it lies more than 200 tokens back
    # the reader's own keys matter: with the rows of its W_uk in another order the logits move
    cfg, w = plain.read_model_folder(folder)
    moved = plain.forward(cfg, dict(w, **{"l2.mix.uk": w["l2.mix.uk"].flip(0)}), requests["r0"])[-1]
    assert float((moved - want["r0"][-1].double()).abs().max()) > 1e-2
    for plan_name in ("whole", "then_single", "portions", "mixed"):
        steps = PLANS[plan_name](requests)
        runner = make_runner(folder, dtype, 16, steps)
        M.assert_close(H.run_plan(runner, steps), want, dtype, f"sharp latent attention, {plan_name}", slack=3.0)
    after = _tensor_core_attention_launches()
    if rank == 56 and dtype == "bfloat16":
        assert after[0] > before[0] and after[1] > before[1]       # both tensor-core attention kernels ran
    else:
        assert after == before


def _lean_back(tensors):
    # a shift of nearly one: the mixers read the token before, so a carried row that is lost, cleared or
    # taken from another slot at the start of a portion changes that portion's first row
    for name in tensors:
        if name.endswith(".shift"):
            tensors[name] = torch.full_like(tensors[name], 0.95)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_shift_of_nearly_one_shows_a_lost_row(zoo, dtype):
    config = M.layers_model([M.with_moe(M.latent(2, 16, 8, 16, 24, 16)), M.with_moe(M.gla(2, 16, 24)),
                             M.with_moe(M.latent(2, 16, 8, 16, 24, 16, kv_from=0), experts=3, identity=1, top=2)], width=40)
    folder, requests, want = zoo(config, dtype, [150, 61, 240, 33, 90], edit=_lean_back, key="lean-back")
    cfg, w = plain.read_model_folder(folder)
    tokens = requests["r0"]
    # in the plain model a row of the second layer on depends on the token before it through the shift alone
    x = w["embed"][torch.tensor(tokens)]
    h = plain.scalar_rms_norm(x, w["l0.norm1"], 1e-5)
    assert float((plain.shifted(h, w["l0.shift"])[1:] - h[:-1]).abs().max()) < 0.11 * float(h.abs().max())
    for plan_name in PLANS:
        steps = PLANS[plan_name](requests)
        runner = make_runner(folder, dtype, 8, steps)
        M.assert_close(H.run_plan(runner, steps), want, dtype, f"shift of nearly one, {plan_name}")
        runner.cache.audit()


def _remember(tensors):
    # decays close to one: what the first tokens wrote into the state still weighs in the last
    # token's read-out, so a state that is lost, cleared or mixed up between slots shows
    for name in tensors:
        if name.endswith("a2.b"):
            tensors[name] = torch.full_like(tensors[name], 6.0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_slow_decays_carry_the_first_tokens_through_long_decoding(zoo, dtype):
    config = M.layers_model([M.with_moe(M.gla(2, 32, 48, tau=16.0), experts=4, identity=2, top=2),
                             M.with_moe(M.gla(1, 24, 24, tau=8.0))], width=64, vocab=131)
    folder, requests, want = zoo(config, dtype, [420, 150, 260, 90], edit=_remember, key="remember")
    cfg, w = plain.read_model_folder(folder)
    tokens = requests["r0"]
    moved = plain.forward(cfg, w, [(tokens[0] + 1) % 131] + tokens[1:])[-1]
    assert float((moved - want["r0"][-1].double()).abs().max()) > 1e-3      # the plain model itself remembers
    plans = dict(PLANS, long_decoding=lambda r: H.plan_bulk_then_single(r, tail=200))
    for plan_name, plan in plans.items():
        steps = plan(requests)
        runner = make_runner(folder, dtype, 16, steps)
        M.assert_close(H.run_plan(runner, steps), want, dtype, f"slow decays, {plan_name}")


# ---------------------------------------------------------------------------
# the entry point, the scheduler, the command line, the trace runner
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(tmp_path, dtype):
    from lockstep_b200 import Engine, Request

    config, page = M.MODELS["S"]
    folder = M.make_folder(tmp_path, config, seed=21, dtype=dtype)
    engine = Engine(folder, dtype=dtype, num_pages=64, page_size=page, max_running=12, max_step_tokens=96,
                    max_seq_len=512)
    prompts = {f"g{i}": H.random_tokens(n, config["vocab"], seed=300 + i)
               for i, n in enumerate([33, 7, 120, 1, 64, 18, 45, 2, 90, 11])}
    got = engine.generate([Request(uid=u, prompt=p, max_new_tokens=8) for u, p in prompts.items()])
    cfg, w = plain.read_model_folder(folder)
    wrong = []
    for uid, prompt in prompts.items():
        assert len(got[uid]) == 8
        rows = plain.forward(cfg, w, list(prompt) + got[uid])     # causal: one pass gives every step's logits
        for i, tok in enumerate(got[uid]):
            row = rows[len(prompt) + i - 1]
            margin = 2 * M.TOLERANCE[dtype] * (1 + float(row.abs().max()))
            if not float(row[tok]) >= float(row.max()) - margin:
                wrong.append((uid, i, tok))
    # (in bfloat16 a router's close call may change a row: see kemirax_models.CLOSE_CALLS)
    assert len(wrong) <= int(M.CLOSE_CALLS[dtype] * 80), (dtype, wrong)
    # ten requests decode as recorded steps of sixteen rows: the padding rows share the padding slot
    assert engine.runner.graphs is not None and engine.runner.graphs.replays > 0
    engine.cache.audit()
    assert engine.cache.live == 0


def test_the_command_line_writes_a_random_model_and_runs_a_workload(tmp_path):
    """``bin/lockstep random-model`` from a configuration, then ``bin/lockstep run``: greedy tokens are the plain
    model's, and sampled requests (temperature, top-p) come out whole."""
    config, page = M.MODELS["U"]
    (tmp_path / "config.json").write_text(json.dumps(config))
    folder = tmp_path / "model"
    lockstep = [sys.executable, str(ROOT / "bin" / "lockstep")]
    proc = subprocess.run(lockstep + ["random-model", "--config", str(tmp_path / "config.json"), "--out", str(folder),
                                      "--seed", "5", "--init-std", "0.15", "--gain-std", "0.1"],
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    prompts = {f"c{i}": H.random_tokens(n, config["vocab"], 95 + i) for i, n in enumerate([4, 23, 50])}
    workload = tmp_path / "workload.json"
    requests = [{"uid": u, "prompt": p, "max_new_tokens": 10} for u, p in prompts.items()]
    requests += [{"uid": "s0", "prompt": prompts["c1"], "max_new_tokens": 12, "temperature": 0.8, "top_p": 0.9, "seed": 3},
                 {"uid": "s1", "prompt": prompts["c1"], "max_new_tokens": 12, "temperature": 0.8, "top_p": 0.9, "seed": 3}]
    workload.write_text(json.dumps(requests))
    proc = subprocess.run(lockstep + ["run", "--model", str(folder), "--dtype", "float32", "--workload", str(workload),
                                      "--policy", "fixed-chunk:16", "--num-blocks", "40", "--block-size", str(page),
                                      "--max-running", "3"], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = {l["uid"]: l for l in (json.loads(x) for x in proc.stdout.splitlines() if x.startswith("{"))}
    assert set(lines) == set(prompts) | {"s0", "s1"}
    cfg, w = plain.read_model_folder(folder)
    for uid, prompt in prompts.items():
        got = lines[uid]["generated"]
        assert len(got) == 10
        rows = plain.forward(cfg, w, list(prompt) + got)
        for i, tok in enumerate(got):
            row = rows[len(prompt) + i - 1]
            assert float(row[tok]) >= float(row.max()) - 2 * M.TOLERANCE["float32"] * (1 + float(row.abs().max()))
    assert len(lines["s0"]["generated"]) == 12 and all(0 <= t < config["vocab"] for t in lines["s0"]["generated"])


def test_trace_runner_replays_a_trace(tmp_path):
    config, page = M.MODELS["T"]
    folder = M.make_folder(tmp_path, config, seed=9, dtype="bfloat16")
    requests = {f"t{i}": H.random_tokens(n, config["vocab"], seed=70 + i) for i, n in enumerate([40, 130, 25, 61, 90])}
    steps = H.plan_mixed(requests, max_live=4)
    out = tmp_path / "out"
    for dtype in ("bfloat16", "float32"):
        proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype,
                               "--out", str(out / dtype), "--max-tokens", str(H.max_live_tokens(steps, 64))],
                              input=H.plan_to_jsonl(steps), capture_output=True, text=True, timeout=900)
        assert proc.returncode == 0, proc.stderr[-2000:]
        assert [l for l in proc.stdout.splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(len(steps))]
        want = {u: M.plain_logits(folder, t).float() for u, t in requests.items()}
        at = {u: 0 for u in requests}
        rows = {}
        for i, step in enumerate(steps):
            got = np.fromfile(out / dtype / f"{i}.f32", dtype="<f4").reshape(-1, config["vocab"])
            r = 0
            for uid, toks, wanted in step["entries"]:
                for wpos in wanted:
                    rows[(uid, at[uid] + wpos)] = torch.from_numpy(got[r].copy())
                    r += 1
                at[uid] += len(toks)
            assert r == got.shape[0]
        M.assert_close(rows, want, dtype, f"trace runner, {dtype}")
