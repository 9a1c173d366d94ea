"""Pikurax without a device: the configuration and its errors, names and shapes of the tensors, the schedule of a
loop and the cache needs of its parts in the cache manager, the plain implementation's own properties."""

from __future__ import annotations

import copy

import pytest
import torch

import pikurax_models as M
from plain import pikurax_plain as plain

from lockstep_b200.cache import CacheManager
from lockstep_b200.config import ConfigError, config_from_dict
from lockstep_b200.engine.batch import first_key, plan_attention
from lockstep_b200.engine.model import Model, expected_weights
from lockstep_b200.parts import Runtime


def _model(config):
    rt = Runtime(device=torch.device("cpu"), dtype=torch.float32, page_size=16, max_positions=64,
                 err=torch.zeros(2, dtype=torch.int32))
    return Model(config_from_dict(config).model_spec(), rt)


def test_names_and_shapes():
    w = expected_weights(config_from_dict(M.MODEL_S).model_spec())
    assert w["embed"].shape == (193, 72) and w["bigram"].shape == (62, 72) and w["loop.in"].shape == (72, 144)
    assert w["l0.mix.left.k"].shape == (48, 72) and "l0.mix.left.v" not in w          # the values are the keys
    assert w["l0.mix.right.ra"].shape == (5, 8, 8) and w["l0.mix.right.conv"].shape == (40, 4)
    assert w["l0.mix.left.out"].shape == (72,) and w["l0.norm1b"].shape == (72,)
    assert w["l1.mix.left.q.b"].shape == (96,) and w["l1.mix.left.q.norm"].shape == (24,) and w["l1.mix.left.sink"].shape == (4,)
    assert "l1.mix.left.o.b" not in w and w["l1.mix.left.v"].shape == (32, 72)
    assert w["l1.mix.right.g"].shape == (72, 72) and w["l1.mlp.shared.sg"].shape == (1, 72)
    assert "l2.mlp.shared.gate" not in w and "l3.mlp.gate" not in w and "l3.norm2" not in w
    assert "head" not in w and "head.weight" not in w                                  # the head is the embedding table
    u = expected_weights(config_from_dict(M.MODEL_U).model_spec())
    assert "bigram" not in u and "loop.in" not in u


def test_schedule_of_a_loop_and_cache_entries():
    spec = config_from_dict(M.MODEL_S).model_spec()
    assert [(r.layer, r.inject) for r in spec.schedule] == [
        (0, False), (1, True), (2, False), (1, True), (2, False), (1, True), (2, False), (3, False)]
    assert [r.cache for r in spec.schedule] == list(range(8))
    one_pass = copy.deepcopy(M.MODEL_S)
    one_pass["loop"] = {"start": 0, "stop": 4, "times": 1}
    assert [r.inject for r in config_from_dict(one_pass).model_spec().schedule] == [True, False, False, False]
    assert not any(r.inject for r in config_from_dict(M.MODEL_U).model_spec().schedule)


def test_cache_needs_in_the_manager():
    model = _model(M.MODEL_S)
    needs = model.cache_needs()
    assert len(needs) == 9 and model.embedding_entry == 8               # eight runs and the embedding's last token
    assert needs[8].kind == "state" and needs[8].state_dtype == torch.int32
    assert needs[0].kind == "several" and needs[0].parts[0].window == 0  # a chunked layer keeps every page
    assert needs[0].parts[1].state_shape == (4 * 40,)                    # S and three carried inputs
    assert needs[1].parts[0].head_dim == 32 and needs[1].parts[1].state_shape == (3 * 8 * 24,)
    cm = CacheManager(needs, num_pages=8, page_size=16, max_live=2, max_seq_len=64, allocate=False)
    assert len(cm.paged) == 4 and len(cm.states) == 5
    assert _model(M.MODEL_U).embedding_entry is None


@pytest.mark.parametrize("change, message", [
    (lambda c: c["layers"][0].update(type="serial"), "type"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(vdim=8), "vdim must equal dim"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=18), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["left"].pop("mask"), "mask"),
    (lambda c: c["layers"][0]["mixer"]["right"].update(blocks=3), "blocks must divide"),
    (lambda c: c["layers"][1]["mixer"]["right"].update(decay=[0.5]), "decay"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c["layers"][1]["mlp"].update(kind="sparse"), "kind"),
    (lambda c: c["loop"].update(stop=9), "loop"),
    (lambda c: c["embedding"]["bigram"].update(buckets=0), "buckets"),
    (lambda c: c["norm"].update(eps=0), "eps"),
])
def test_configuration_errors(change, message):
    cfg = copy.deepcopy(M.MODEL_S)
    change(cfg)
    with pytest.raises(ConfigError, match=message):
        config_from_dict(cfg)


def test_first_key_of_windows_and_chunks():
    assert [first_key(p, -5) for p in (0, 4, 5, 9, 10)] == [0, 0, 5, 5, 10]
    assert [first_key(p, 4) for p in (0, 3, 4, 9)] == [0, 0, 1, 6] and first_key(77, 0) == 0
    # a decoded token at position 300 of a layer with chunks of 40 reads the split that holds position 280 only
    _, split, combine, slots = plan_attention([(0, 0, 300, 1)], -40, 256)
    assert split[:, 4].tolist() == [1] and slots == 1
    _, split, _, slots = plan_attention([(0, 0, 300, 1)], -200, 256)
    assert split[:, 4].tolist() == [0, 1]


def test_plain_pieces():
    torch.manual_seed(0)
    x = torch.randn(5, 12, dtype=torch.float64)
    y = plain.layer_norm(x, torch.ones(12, dtype=torch.float64), 0.0)
    assert torch.allclose(y.mean(-1), torch.zeros(5, dtype=torch.float64), atol=1e-12)
    assert torch.allclose((y * y).mean(-1), torch.ones(5, dtype=torch.float64), atol=1e-12)
    assert plain.bigram_rows([3, 4, 5], {"buckets": 7, "mul_prev": 2, "mul_cur": 3}) == [7, (6 + 12) % 7, (8 + 15) % 7]
    # chunks: with every score equal, the weights of a row are uniform over its chunk's earlier keys
    q = torch.zeros(7, 1, 4, dtype=torch.float64)
    pr = plain.softmax_attention(q, q, q, 1.0, chunk=3, weights=True)[0]
    assert torch.allclose(pr[4], torch.tensor([0, 0, 0, .5, .5, 0, 0], dtype=torch.float64))
    assert torch.allclose(pr[6], torch.tensor([0, 0, 0, 0, 0, 0, 1.], dtype=torch.float64))
    # a sink of zero beside three zero scores takes a quarter
    pr = plain.softmax_attention(q, q, q, 1.0, sinks=torch.zeros(1, dtype=torch.float64), weights=True)[0]
    assert torch.allclose(pr[2, :3].sum(), torch.tensor(0.75, dtype=torch.float64))
    # the recurrence of the unit continues from its state
    u, r, i = (torch.rand(9, 6, dtype=torch.float64) for _ in range(3))
    lam = torch.randn(6, dtype=torch.float64)
    whole, _ = plain.gated_unit_recurrence(u, r, i, lam)
    _, s = plain.gated_unit_recurrence(u[:4], r[:4], i[:4], lam)
    rest, _ = plain.gated_unit_recurrence(u[4:], r[4:], i[4:], lam, s)
    assert torch.allclose(whole[4:], rest, atol=1e-14)
    # the chosen experts' weights sum to one
    w = {"m.router": torch.randn(6, 12, dtype=torch.float64)}
    ids, weights, z = plain.route(x, w, "m", 3)
    assert torch.allclose(weights.sum(-1), torch.ones(5, dtype=torch.float64)) and (z.gather(1, ids)[:, 0] == z.max(-1).values).all()
