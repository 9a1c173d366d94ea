"""Kemirax without a device: the configuration class and its errors, tensor names and shapes, the
schedule of layers that read another layer's cache, what the cache manager makes of a layer's two
parts (the mixer's pages or state, and the row its shift carries), the stretched rotary tables in
the halves layout, and properties of the plain implementation itself."""

from __future__ import annotations

import copy
import math

import pytest
import torch

import kemirax_models as M
from plain import kemirax_plain as plain

from lockstep_b200.cache import CacheManager
from lockstep_b200.config import ConfigError, KemiraxConfig, config_from_dict
from lockstep_b200.config.spec import PartSpec
from lockstep_b200.engine.model import Model, expected_weights
from lockstep_b200.parts import Runtime
from lockstep_b200.parts.base import build_part


def cpu_runtime(max_positions=64):
    return Runtime(device=torch.device("cpu"), dtype=torch.float32, page_size=8, max_positions=max_positions,
                   err=torch.zeros(2, dtype=torch.int32))


def test_registry_picks_the_class_by_the_architecture_key():
    cfg = config_from_dict(M.MODEL_S)
    assert isinstance(cfg, KemiraxConfig) and cfg.to_dict() == M.MODEL_S
    assert (cfg.width, cfg.vocab, cfg.eps) == (72, 193, 1e-5)


def test_readers_of_another_layers_cache_borrow_its_first_part():
    spec = config_from_dict(M.MODEL_S).model_spec()
    runs = [(r.layer, r.cache, r.borrows) for r in spec.schedule]
    assert runs == [(0, 0, ()), (1, 1, ()), (2, 2, ((0, 0),)), (3, 3, ()), (4, 4, ((0, 0),)), (5, 5, ())]
    assert [l.mixer.kind for l in spec.layers] == ["latent_attention", "gated_linear", "latent_attention", "gated_linear",
                                                   "latent_attention", "latent_attention"]
    assert [bool(l.mixer.get("borrows_kv")) for l in spec.layers] == [False, False, True, False, True, False]
    assert spec.layers[3].feed_forward.kind == "none"
    f = spec.layers[0].feed_forward
    assert (f["experts"], f["identity"], f["top"], f["score"], f["scale"], f["limit"]) == (5, 2, 2, "softmax", "output", 1.2)
    assert f["shared"] == {"ff": 40, "limit": 0.7, "gate": True} and spec.layers[1].feed_forward["shared"] is None


def test_tensor_names_and_shapes():
    w = expected_weights(config_from_dict(M.MODEL_S).model_spec())
    assert w["embed"].shape == (193, 72) and w["head"].shape == (193, 72) and w["final.norm"].shape == ()
    assert w["l0.norm1"].shape == () and w["l0.shift"].shape == (72,)
    assert w["l0.rg1"].shape == (72, 72) and w["l0.rg1.b"].shape == (72,) and w["l0.rg2.b"].shape == (72,)
    assert w["l0.mix.dq"].shape == (20, 72) and w["l0.mix.dq.norm"].shape == (20,) and w["l0.mix.uq"].shape == (3 * 24, 20)
    assert w["l0.mix.dkv"].shape == (48, 72) and w["l0.mix.dkv.norm"].shape == (40,)
    assert w["l0.mix.uk"].shape == (48, 40) and w["l0.mix.uv"].shape == (72, 40) and w["l0.mix.o"].shape == (72, 72)
    assert "l0.mix.q" not in w and "l0.mix.sink" not in w
    # a reader has queries, W_uk, W_uv and W_o of its own and no down-projection
    assert "l2.mix.dkv" not in w and "l2.mix.dkv.norm" not in w
    assert w["l2.mix.uk"].shape == (2 * 24, 40) and w["l2.mix.uv"].shape == (2 * 16, 40) and w["l2.mix.dq"].shape == (36, 72)
    assert w["l1.mix.q"].shape == (48, 72) and w["l1.mix.v"].shape == (80, 72) and w["l1.mix.g"].shape == (80, 72)
    assert w["l1.mix.a1"].shape == (5, 72) and w["l1.mix.a2"].shape == (48, 5) and w["l1.mix.a2.b"].shape == (48,)
    assert w["l1.mix.norm"].shape == (40,) and w["l1.mix.o"].shape == (72, 80)
    # experts: the router has a row per real and per identity expert; identity experts have no tensors
    assert w["l0.mlp.router"].shape == (7, 72) and w["l0.mlp.correction"].shape == (7,)
    assert w["l0.mlp.e4.gate"].shape == (24, 72) and w["l0.mlp.e4.down"].shape == (72, 24) and "l0.mlp.e5.gate" not in w
    assert w["l0.mlp.shared.up"].shape == (40, 72) and w["l0.mlp.shared.sg"].shape == (1, 72)
    assert "l1.mlp.shared.up" not in w and "l1.mlp.shared.sg" not in w
    # a layer without a feed-forward has no second gate (stored ones are tolerated)
    assert "l3.mlp.router" not in w and "l3.rg2" not in w and "l3.rg1" in w
    # a rank the configuration does not name is whatever the stored tensors have
    raw = copy.deepcopy(M.MODEL_S)
    del raw["layers"][1]["mixer"]["decay_rank"]
    w = expected_weights(config_from_dict(raw).model_spec())
    assert w["l1.mix.a1"].shape == (-1, 72) and w["l1.mix.a1"].fits((9, 72))


@pytest.mark.parametrize("edit, message", [
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c["layers"][0].update(type="attention"), "not one of"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=6), "rot_dim"),
    (lambda c: c["layers"][0]["mixer"].pop("q_rank"), "q_rank"),
    (lambda c: c["layers"][1]["mixer"].update(tau=0.0), "tau"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1), "kv_from"),          # a linear layer caches no latents
    (lambda c: c["layers"][4]["mixer"].update(kv_from=2), "kv_from"),          # a reader has none of its own
    (lambda c: c["layers"][2]["mixer"].update(kv_from=5), "kv_from"),          # a later layer
    (lambda c: c["layers"][2]["mixer"].update(kv_rank=24), "kv_rank"),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(base=7.0), "rot"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "moe"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=8), "top"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(identity=-1), "identity"),
    (lambda c: c["layers"][0]["mlp"]["shared"].pop("limit"), "limit"),
])
def test_configuration_errors_name_the_key(edit, message):
    raw = copy.deepcopy(M.MODEL_S)
    edit(raw)
    with pytest.raises(ConfigError, match=message):
        config_from_dict(raw)


def test_a_layer_keeps_its_mixers_cache_and_the_row_its_shift_carries():
    spec = config_from_dict(M.MODEL_S).model_spec()
    model = Model(spec, cpu_runtime())
    needs = model.cache_needs()
    assert [n.kind for n in needs] == ["several"] * 6
    pages, row = needs[0].parts
    assert (pages.kind, pages.kv_heads, pages.head_dim, pages.window) == ("paged_kv", 1, 48, 0)
    assert row.kind == "state" and row.state_shape == (72,) and row.state_dtype == torch.float32
    state, row = needs[1].parts
    assert state.kind == "state" and state.state_shape == (2 * 24 * 40,)
    # a reader holds no pages of its own, only its row
    assert needs[2].parts[0] is None and needs[2].parts[1].state_shape == (72,)
    assert needs[4].parts[0] is None and needs[5].parts[0].head_dim == 48
    cache = CacheManager(needs, num_pages=8, page_size=16, max_live=2, max_seq_len=128, allocate=False)
    lender, reader = cache.view(0), cache.view(2, True, ((0, 0),))
    assert [p.kind for p in lender.parts] == ["paged_kv", "state"] and [p.kind for p in reader.parts] == ["paged_kv", "state"]
    assert lender.parts[0].writes and not reader.parts[0].writes and reader.parts[1].writes
    assert reader.parts[0].group is lender.parts[0].group
    cache.create("a")
    cache.reserve("a", 100)
    cache.advance("a", 100)
    cache.audit()
    cache.release("a")
    cache.audit()
    assert cache.live == 0


@pytest.mark.parametrize("dims, base, scaling", [(16, 40000.0, (3.0, 1024, 16.0, 2.0)), (8, 100.0, (4.0, 64, 8.0, 1.0)),
                                                 (6, 77.0, (1.5, 40, 6.0, 0.7)), (24, 300.0, None)])
def test_stretched_rotary_tables_in_halves(dims, base, scaling):
    named = dict(zip(("factor", "original", "fast", "slow"), scaling)) if scaling else None
    part = build_part("position", PartSpec("scaled_rotary", {"dim": dims, "theta": base, "scaling": named,
                                                             "interleaved": False}), cpu_runtime(50))
    cos, sin, rotated = part.rotary()
    assert rotated == dims and not part.rotary_interleaved
    want_cos, want_sin = plain.rotary_tables(range(50), dims, base, named)
    assert float((cos.double() - want_cos).abs().max()) < 1e-6 and float((sin.double() - want_sin).abs().max()) < 1e-6
    f, mag = plain.stretched_frequencies(dims, base, named)
    plain_f = base ** (-2.0 * torch.arange(dims // 2, dtype=torch.float64) / dims)
    if scaling:
        assert mag == pytest.approx(0.1 * math.log(scaling[0]) + 1.0)
        assert float(f[0]) == pytest.approx(1.0)                                 # the fastest pair keeps its frequency
        assert bool((f <= plain_f + 1e-15).all()) and bool((f >= plain_f / scaling[0] - 1e-15).all())
        assert float(f[-1]) < float(plain_f[-1])                                 # the slowest is stretched
    else:
        assert mag == 1.0 and torch.equal(f, plain_f)


def test_plain_mechanisms_have_the_properties_the_design_names():
    g = torch.Generator().manual_seed(2)
    # one number as gain, eps inside the root
    x = torch.randn(5, 12, generator=g, dtype=torch.float64)
    y = plain.scalar_rms_norm(x, torch.tensor(2.5, dtype=torch.float64), 1e-3)
    assert torch.allclose(y, 2.5 * x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-3))
    # the shift: a mix of zero changes nothing, a mix of one gives the row before (zeros first), and a
    # continuation from the carried row gives what the whole sequence gives
    mix = torch.rand(12, generator=g, dtype=torch.float64)
    assert torch.equal(plain.shifted(x, torch.zeros(12, dtype=torch.float64)), x)
    back = plain.shifted(x, torch.ones(12, dtype=torch.float64))
    assert torch.allclose(back[1:], x[:-1], atol=1e-14) and float(back[0].abs().max()) < 1e-14
    whole = plain.shifted(x, mix)
    assert torch.allclose(torch.cat([plain.shifted(x[:2], mix), plain.shifted(x[2:], mix, before=x[1])]), whole)
    # the recurrence continues from a state
    q, k, a = (torch.randn(7, 2, 4, generator=g, dtype=torch.float64) for _ in range(3))
    v = torch.randn(7, 2, 3, generator=g, dtype=torch.float64)
    a = torch.sigmoid(a)
    o, s = plain.decayed_outer_product_rule(q, k, v, a)
    o1, s1 = plain.decayed_outer_product_rule(q[:3], k[:3], v[:3], a[:3])
    o2, s2 = plain.decayed_outer_product_rule(q[3:], k[3:], v[3:], a[3:], s1)
    assert torch.allclose(torch.cat([o1, o2]), o) and torch.allclose(s2, s)
    assert torch.allclose(o[0], torch.einsum("hk,hv,hk->hv", k[0], v[0], q[0]))   # the token's own pair is read undecayed
    # routing: the correction changes the choice and not the weight; identity experts return the input
    w = {"r.router": torch.eye(4, dtype=torch.float64), "r.correction": torch.tensor([0.0, 0.0, 0.0, 1.0], dtype=torch.float64)}
    logits = torch.tensor([[3.0, 2.0, 1.0, 0.0]], dtype=torch.float64)
    ids, weights = plain.route(logits, w, "r", {"top": 2})
    scores = torch.softmax(logits, -1)
    assert ids.tolist() == [[3, 0]] and torch.allclose(weights, scores[:, [3, 0]])
    f = {"router": {"experts": 0, "identity": 4, "top": 2}, "expert": {"limit": 1.0}}
    out = plain.expert_mixture(logits, w, "r", f)
    assert torch.allclose(out, logits * (scores[0, 3] + scores[0, 0]))
    # an expert's clamps: a large gate is cut from above only, a large up from both sides
    we = {"e.gate": torch.tensor([[1.0]], dtype=torch.float64), "e.up": torch.tensor([[1.0]], dtype=torch.float64),
          "e.down": torch.tensor([[1.0]], dtype=torch.float64)}
    big = plain.clamped_expert(torch.tensor([[50.0]], dtype=torch.float64), we, "e", 2.0)
    assert float(big) == pytest.approx(2.0 * torch.sigmoid(torch.tensor(1.702 * 2.0, dtype=torch.float64)).item() * 3.0)
    low = plain.clamped_expert(torch.tensor([[-50.0]], dtype=torch.float64), we, "e", 2.0)
    assert float(low) == pytest.approx(-50.0 * torch.sigmoid(torch.tensor(-1.702 * 50.0, dtype=torch.float64)).item() * -1.0)
