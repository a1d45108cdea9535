"""Dezelorn on the CPU: config keys and refusals, the spec it turns into, the tensors it
declares, and what its mixer asks of the cache."""

import copy
import json
import os

import pytest
import torch

import dezelorn_cases as C
import plain_dezelorn as plain
from servelab_b200.cache import CacheManager, FixedStateRequest, PagedKVRequest
from servelab_b200.cache.storage import bytes_per_page, plan_groups
from servelab_b200.config import ConfigError, DezelornConfig, config_from_dict, load_config
from servelab_b200.models.causal_lm import declare_tensors
from servelab_b200.parts import BLOCKS, part_class


def test_round_trip_and_registry(tmp_path):
    for cfg, _, _ in C.CASES.values():
        typed = config_from_dict(cfg)
        assert isinstance(typed, DezelornConfig) and typed.to_dict() == cfg
    with open(tmp_path / "config.json", "w") as f:
        json.dump(C.P, f)
    assert load_config(str(tmp_path)).to_dict() == C.P


def test_every_size_and_constant_reaches_the_spec():
    spec = config_from_dict(C.Q).to_model_spec()
    assert spec.vocab_size == 300 and spec.hidden_size == 80 and spec.embedding_scale == 9.0
    assert not spec.tie_word_embeddings and len(spec.layers) == 4
    m = spec.layers[2].mixer
    assert (m.num_heads, m.num_kv_heads, m.head_dim, m.conv_taps, m.window) == (8, 2, 32, 6, 17)
    assert (m.q_temp_coef, m.q_temp_every, m.scale) == (0.25, 64, 0.15)
    assert m.tied_values and m.distance_bias and m.talking_heads and m.output_gate
    assert spec.layers[2].feed_forward is None and spec.layers[2].ff_norm is None
    assert spec.layers[1].feed_forward.intermediate_size == 96
    assert spec.layers[0].kind == "sandwich_norm" and spec.final_norm.kind == "dynamic_tanh"


@pytest.mark.parametrize("change, text", [
    (lambda c: c.update(rope=1), "unknown key"),
    (lambda c: c["layers"][0].update(type="recurrent"), "not known"),
    (lambda c: c["layers"][0]["mixer"].update(vdim=8), "vdim"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=4), "multiple"),
    (lambda c: c["layers"][0]["mixer"].update(sink=2), "unknown key"),
    (lambda c: c["layers"][0]["mlp"].update(kind="routed"), "not known"),
    (lambda c: c["layers"][1]["mixer"]["mask"].update(size=0), "positive"),
    (lambda c: c.pop("width"), "missing"),
])
def test_what_the_config_refuses(change, text):
    cfg = copy.deepcopy(C.P)
    change(cfg)
    with pytest.raises(ConfigError, match=text):
        config_from_dict(cfg)


def test_declared_tensors():
    decls = {d.name: tuple(d.shape) for d in declare_tensors(config_from_dict(C.P).to_model_spec())}
    assert decls["embed"] == (211, 48) and decls["head"] == (211, 48)
    assert decls["final.norm"] == (48,) and decls["final.norm.b"] == (48,) and decls["final.norm.alpha"] == ()
    assert decls["l0.mix.q"] == (96, 48) and decls["l0.mix.k"] == (48, 48) and decls["l0.mix.g"] == (96, 48)
    assert decls["l0.mix.o"] == (48, 96) and decls["l0.mix.q.conv"] == (96, 3) and decls["l0.mix.k.conv"] == (48, 3)
    assert decls["l0.mix.r1"] == (6,) and decls["l0.mix.talk"] == (6, 6)
    assert decls["l0.mlp.gate"] == (72, 48) and decls["l0.mlp.down"] == (48, 72)
    assert "l1.mlp.gate" not in decls and "l1.norm2" not in decls and "l1.norm1b.alpha" in decls
    assert decls["l2.mix.q.conv"] == (64, 1) and decls["l2.mix.k.conv"] == (64, 1)     # one tap: a factor per channel


def test_cache_requests_pages_with_tied_values_and_a_state_record():
    spec = config_from_dict(C.P).to_model_spec()
    reqs = [part_class(BLOCKS, b).cache_request(b) for b in spec.layers]
    pages, state = reqs[0]
    assert pages == PagedKVRequest(3, 16, 12, tied_values=True) and state == FixedStateRequest((2, 144))
    assert reqs[2] == PagedKVRequest(4, 16, 1000, tied_values=True)          # one tap: a factor per channel, no record
    groups, of_layer = plan_groups(reqs)
    assert len(groups) == 3 and of_layer == {0: 0, 1: 1, 2: 2}
    assert bytes_per_page(groups, 8, torch.bfloat16) == (3 * 16 + 32 + 4 * 16) * 8 * 2   # keys only
    mgr = CacheManager([g.request.window for g in groups], 6, 8, 2)
    assert mgr.open("a") and mgr.ensure("a", 40)
    mgr.trim("a", 40)
    assert mgr.block_table("a", 0)[:3] == [-1, -1, -1] and -1 not in mgr.block_table("a", 2)
    mgr.release("a")
    mgr.check_invariants()


def test_plain_mechanisms():
    """The oracle's own pieces, on cases worked by hand."""
    taps = torch.tensor([[1.0, 10.0, 100.0]], dtype=torch.float64)
    u = torch.tensor([[1.0], [2.0], [3.0], [4.0]], dtype=torch.float64)
    assert plain.causal_conv(u, taps).flatten().tolist() == [100.0, 210.0, 321.0, 432.0]
    t = plain.query_temperature(9, 0.5, 4, torch.float64)
    assert t[2] == 1.0 and abs(float(t[3]) - (1 + 0.5 * 0.6931471805599453)) < 1e-12 and t[6] == t[3]
    q = torch.zeros(5, 1, 2, dtype=torch.float64)
    w = plain.attention_weights(q, q.clone(), 1.0, torch.tensor([0.0]), torch.tensor([1.0]), 2)
    assert w[0, 4].tolist() == [0.0, 0.0, 0.0, 0.5, 0.5] and w[0, 0].tolist() == [1.0, 0, 0, 0, 0]
    w = plain.attention_weights(q, q.clone(), 1.0, torch.tensor([1.0]), torch.tensor([1.0]), 2)
    assert abs(float(w[0, 4, 3]) - 1 / 3) < 1e-12           # exp(-ln 2) = 1/2 against 1
    y = plain.dynamic_tanh(torch.tensor([0.0, 100.0]), torch.tensor([2.0, 2.0]), torch.tensor([1.0, 1.0]), 0.5)
    assert y.tolist() == [1.0, 3.0]
