"""Daferax on the CPU: config keys and refusals, the spec it turns into, the tensors it declares,
what its mixers ask of the cache, and the oracle's own pieces on cases worked by hand."""

import copy
import json
import math

import pytest
import torch

import daferax_cases as C
import plain_daferax as plain
from servelab_b200.cache import CacheManager, PagedKVRequest
from servelab_b200.cache.storage import bytes_per_page, plan_groups
from servelab_b200.config import ConfigError, DaferaxConfig, config_from_dict, load_config
from servelab_b200.models.causal_lm import declare_tensors
from servelab_b200.parts import BLOCKS, part_class


def test_round_trip_and_registry(tmp_path):
    for cfg, _, _ in C.CASES.values():
        typed = config_from_dict(cfg)
        assert isinstance(typed, DaferaxConfig) and typed.to_dict() == cfg
        assert hash(typed) == hash(config_from_dict(copy.deepcopy(cfg)))
    with open(tmp_path / "config.json", "w") as f:
        json.dump(C.U, f)
    assert load_config(str(tmp_path)).to_dict() == C.U


def test_every_size_and_constant_reaches_the_spec():
    spec = config_from_dict(C.V).to_model_spec()
    assert spec.vocab_size == 300 and spec.hidden_size == 80 and spec.tie_word_embeddings
    assert [b.mixer.kind for b in spec.layers] == ["latent_attention", "normed_attention", "latent_attention",
                                                   "normed_attention", "normed_attention"]
    a = spec.layers[1].mixer
    assert (a.num_heads, a.num_kv_heads, a.head_dim, a.value_dim, a.window, a.scale) == (6, 2, 32, 16, None, 0.12)
    assert a.qk_norm and a.qk_norm_eps == 1e-5 and a.head_gate and a.value_mix == "source"
    assert (a.position.dims, a.position.theta, a.position.yarn_factor) == (16, 1000000.0, None)
    assert spec.layers[3].mixer.value_mix == "mix" and spec.layers[3].mixer.window == 70
    assert spec.layers[4].mixer.value_mix is None
    m = spec.layers[2].mixer
    assert (m.num_heads, m.head_dim, m.rope_dim, m.value_dim, m.kv_rank, m.window) == (2, 8, 2, 24, 40, 1)
    assert (m.position.yarn_factor, m.position.yarn_original, m.position.yarn_fast, m.position.yarn_slow) == (2.0, 32.0, 4.0, 1.0)
    f = spec.layers[0].feed_forward
    assert (f.num_experts, f.top, f.expert_size, f.num_groups, f.keep_groups, f.route_scale) == (8, 3, 32, 4, 3, 2.0)
    assert f.shared.intermediate_size == 24 and not f.renormalize
    g = spec.layers[3].feed_forward
    assert (g.num_groups, g.keep_groups, g.top) == (1, 1, 5)
    assert spec.layers[1].feed_forward.kind == "gated_mlp" and spec.layers[4].feed_forward is None
    assert spec.layers[0].kind == "result_norm" and spec.final_norm.kind == "layernorm"


@pytest.mark.parametrize("change, text", [
    (lambda c: c.update(rope=1), "unknown key"),
    (lambda c: c["layers"][0].update(type="recurrent"), "not known"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"].update(sink=2), "unknown key"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "even"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=6), "must equal rot_dim"),
    (lambda c: c["layers"][0]["mlp"].update(kind="routed"), "not known"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "fit into the kept groups"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4), "equal groups"),
    (lambda c: c["layers"][1]["mixer"]["mask"].update(size=0), "positive"),
    (lambda c: c["layers"][2]["mixer"].update(vdim=16), "agree"),
    (lambda c: c.pop("width"), "missing"),
])
def test_what_the_config_refuses(change, text):
    cfg = copy.deepcopy(C.U)
    change(cfg)
    with pytest.raises(ConfigError, match=text):
        config_from_dict(cfg)


def test_declared_tensors():
    decls = {d.name: tuple(d.shape) for d in declare_tensors(config_from_dict(C.U).to_model_spec())}
    assert decls["embed"] == (211, 48) and "head" not in decls
    assert decls["final.norm"] == (48,) and decls["final.norm.b"] == (48,)
    assert decls["l0.mix.q"] == (64, 48) and decls["l0.mix.k"] == (32, 48) and decls["l0.mix.v"] == (16, 48)
    assert decls["l0.mix.g"] == (4, 48) and decls["l0.mix.o"] == (48, 32)
    assert decls["l0.mix.q.norm"] == (16,) and decls["l0.mix.k.norm"] == (16,)
    assert "l0.mix.vmix" not in decls and decls["l2.mix.vmix"] == ()       # the first such layer mixes nothing
    assert decls["l1.mix.q"] == (36, 48) and decls["l1.mix.dkv"] == (24, 48) and decls["l1.mix.dkv.norm"] == (20,)
    assert decls["l1.mix.uk"] == (24, 20) and decls["l1.mix.uv"] == (36, 20)
    assert decls["l1.mix.g"] == (36, 48) and decls["l1.mix.o"] == (48, 36)
    assert decls["l0.mlp.router"] == (6, 48) and decls["l0.mlp.e5.gate"] == (24, 48) and decls["l0.mlp.e0.down"] == (48, 24)
    assert decls["l0.mlp.shared.up"] == (40, 48) and "l2.mlp.shared.up" not in decls
    assert "l1.mlp.router" not in decls and "l1.norm2" not in decls and decls["l1.norm1.b"] == (48,)
    assert decls["l3.mlp.gate"] == (56, 48)


def test_cache_requests_values_of_their_own_size_and_latent_rows():
    spec = config_from_dict(C.U).to_model_spec()
    reqs = [part_class(BLOCKS, b).cache_request(b) for b in spec.layers]
    assert reqs[0] == PagedKVRequest(2, 16, None, value_dim=8)
    assert reqs[1] == PagedKVRequest(1, 24, 9, tied_values=True)           # latent 20 + rotated 4, keys only
    assert reqs[2] == PagedKVRequest(2, 8, 5, value_dim=8)
    groups, of_layer = plan_groups(reqs)
    assert len(groups) == 4 and of_layer == {0: 0, 1: 1, 2: 2, 3: 3}
    assert bytes_per_page(groups, 8, torch.bfloat16) == (2 * (16 + 8) + 24 + 2 * (8 + 8) + 32) * 8 * 2
    mgr = CacheManager([g.request.window for g in groups], 6, 8, 2)
    assert mgr.open("a") and mgr.ensure("a", 40)
    mgr.trim("a", 40)
    assert mgr.block_table("a", 1)[:3] == [-1, -1, -1] and -1 not in mgr.block_table("a", 0)
    mgr.release("a")
    mgr.check_invariants()


def test_plain_mechanisms():
    """The oracle's own pieces, on cases worked by hand."""
    y = plain.layer_norm(torch.tensor([[1.0, 3.0]], dtype=torch.float64), torch.tensor([2.0, 2.0]),
                         torch.tensor([0.5, 0.5]), 0.0)
    assert y.tolist() == [[-1.5, 2.5]]
    y = plain.rms_norm(torch.tensor([[3.0, 4.0]], dtype=torch.float64), torch.tensor([1.0, 2.0]), 0.0)
    assert torch.allclose(y, torch.tensor([[3.0, 8.0]], dtype=torch.float64) / math.sqrt(12.5))
    # neighbouring pairs: a quarter turn at position 1 with frequency pi/2 would need base tricks;
    # with dims 2 the only frequency is 1, so position p rotates (1, 0) to (cos p, sin p)
    x = torch.tensor([[[1.0, 0.0, 5.0]]], dtype=torch.float64).repeat(3, 1, 1)
    r = plain.rotate_pairs(x, torch.arange(3), 2, 10000.0)
    assert torch.allclose(r[2, 0], torch.tensor([math.cos(2.0), math.sin(2.0), 5.0], dtype=torch.float64))
    # scaled frequencies: the fastest pair keeps its frequency, the slowest is divided by the factor
    f, mag = plain.rotary_frequencies(8, 100.0, {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0})
    f0, _ = plain.rotary_frequencies(8, 100.0, None)
    assert f[0] == f0[0] and abs(float(f[3]) - float(f0[3]) / 4) < 1e-15 and abs(mag - (0.1 * math.log(4) + 1)) < 1e-15
    # the window counts the query's own position
    assert plain.visible(4, 2).int().tolist() == [[1, 0, 0, 0], [1, 1, 0, 0], [0, 1, 1, 0], [0, 0, 1, 1]]
    # routing: groups (0,1) (2,3) (4,5); the best two groups are the first and the last, so
    # expert 3, although third best overall... is second best, is barred
    W = {"m.router": torch.eye(6, dtype=torch.float64)}
    h = torch.log(torch.tensor([[0.30, 0.05, 0.10, 0.25, 0.28, 0.02]], dtype=torch.float64))
    idx, w = plain.route(h, W, "m.", {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 2}, "scale": 2.0})
    assert idx.tolist() == [[0, 4]] and torch.allclose(w, torch.tensor([[0.60, 0.56]], dtype=torch.float64))
    idx, _ = plain.route(h, W, "m.", {"experts": 6, "top": 3})
    assert idx.tolist() == [[0, 4, 3]]
