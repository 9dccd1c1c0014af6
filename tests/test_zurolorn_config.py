"""Zurolorn on the CPU: what its configuration class reads and refuses, the run list of a loop, the tensor names the
assembled model asks for, and properties of the plain implementation's mechanisms."""
import copy

import pytest
import torch

import plain_zurolorn as pz
import zurolorn_models as zm
from cisr_b200.config import ConfigError, architecture_for
from cisr_b200.engine.model import Model


def spec_of(cfg):
    return architecture_for(cfg).config_class.from_dict(cfg).to_spec()


def test_registry_picks_the_design_by_its_architecture_key():
    assert architecture_for(zm.ZA).name == "Zurolorn"
    with pytest.raises(ConfigError):
        architecture_for({"architecture": "Nothing"})


@pytest.mark.parametrize("case", list(zm.CASES))
def test_model_asks_for_exactly_the_checkpoint_tensors(case):
    cfg, _ = zm.CASES[case]
    needs = Model(spec_of(cfg), "bfloat16", config=cfg, device=None).tensor_needs()
    assert {k: tuple(v.shape) for k, v in needs.items()} == zm.tensor_shapes(cfg)


def test_run_list_of_a_loop_and_its_pass_vectors():
    spec = spec_of(zm.ZA)
    assert [(e.layer, e.pass_step) for e in spec.run] == [(0, 0), (1, None), (0, 1), (1, None), (0, 2), (1, None), (2, None)]
    assert [(e.layer, e.pass_step) for e in spec_of(zm.ZC).run] == [(0, None), (1, 0)]
    assert spec_of(zm.ZB).pass_steps is None and [e.layer for e in spec_of(zm.ZB).run] == [0, 1]
    assert pz.layer_order(zm.ZA) == [(e.layer, e.pass_step) for e in spec.run]


def test_every_run_entry_has_a_cache_of_its_own_and_rows_are_padded():
    model = Model(spec_of(zm.ZB), "float32", config=zm.ZB, device=None)
    uses = model.cache_uses()
    assert [u.head_dim for u in uses] == [64, 128] and all(u.planes == 1 and u.kv_heads == 1 for u in uses)
    cache = Model(spec_of(zm.ZA), "float32", config=zm.ZA, device=None).make_cache(8, 16, 2)
    assert sorted(len(g.entries) for g in cache.page_groups) == [1, 3, 3]      # three passes of layers 0 and 1, then layer 2


def test_parts_take_their_constants_from_the_configuration():
    spec = spec_of(zm.ZA)
    first, second = spec.layers[0], spec.layers[1]
    assert first.mixer["gate"] and not first.mixer["q_rank"] and first.mixer["position"].kind == "rotary_half"
    assert not second.mixer["gate"] and second.mixer["q_rank"] == 56 and second.mixer["position"].kind == "rotary_interleaved"
    assert second.feed_forward is None and second.feed_forward_norm is None and "feed_forward_scale" not in second.extras
    assert first.feed_forward["groups"] == 4 and first.feed_forward["keep"] == 2 and first.feed_forward["route_scale"] == 1.5
    assert spec.layers[2].feed_forward["groups"] == 0
    assert spec.embedding["scale"] == 3.0 and spec.head["scale"] == 0.5


@pytest.mark.parametrize("change, message", [
    (lambda c: c["layers"][0].__setitem__("type", "hyena"), "not a mixer"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 8), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"].pop("q_rank"), "q_rank"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "dense"), "moe only"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].__setitem__("count", 3), "groups"),
    (lambda c: c["layers"][0]["mlp"]["router"].__setitem__("top", 9), "top"),
    (lambda c: c["loop"].__setitem__("stop", 7), "loop"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("kv_rank", 400), "not supported"),
    (lambda c: c.pop("logit_scale"), "logit_scale"),
])
def test_refusals(change, message):
    cfg = copy.deepcopy(zm.ZA)
    change(cfg)
    with pytest.raises(ConfigError, match=message):
        spec_of(cfg)


# ------------------------------------------------------------------ the plain implementation's mechanisms
def test_rotation_keeps_lengths_and_depends_on_distance_only():
    g = torch.Generator().manual_seed(0)
    a, b = torch.randn(1, 1, 24, generator=g, dtype=torch.float64), torch.randn(1, 1, 24, generator=g, dtype=torch.float64)
    for interleaved in (False, True):
        def dot(p, q):
            ra = pz.rotate(a, torch.tensor([p]), 1000.0, 16, interleaved)
            rb = pz.rotate(b, torch.tensor([q]), 1000.0, 16, interleaved)
            return float((ra * rb).sum())
        assert abs(dot(7, 3) - dot(104, 100)) < 1e-9 and abs(dot(7, 3) - dot(7, 4)) > 1e-6
        r = pz.rotate(a, torch.tensor([9]), 1000.0, 16, interleaved)
        assert torch.allclose(r.norm(), a.norm()) and torch.equal(r[..., 16:], a[..., 16:])
    half, inter = pz.rotate(a, torch.tensor([5]), 1000.0, 16, False), pz.rotate(a, torch.tensor([5]), 1000.0, 16, True)
    assert not torch.allclose(half, inter)


def test_router_opens_only_the_best_groups():
    router = {"experts": 6, "top": 2, "scale": 2.0, "groups": {"count": 3, "keep": 1}}
    # scores by expert: group 0 = (0.9, 0.1), group 1 = (0.6, 0.6), group 2 = (0.7, 0.2): group 1 wins on its two best
    z = torch.logit(torch.tensor([[0.9, 0.1, 0.6, 0.6, 0.7, 0.2]], dtype=torch.float64))
    chosen, weight = pz.route(torch.eye(6, dtype=torch.float64)[:1] * 0 + 1, torch.diag(z[0]) , router)
    assert sorted(chosen[0].tolist()) == [2, 3] and torch.allclose(weight, torch.full((1, 2), 1.2, dtype=torch.float64))
    router["groups"]["keep"] = 3
    chosen, weight = pz.route(torch.ones(1, 6, dtype=torch.float64), torch.diag(z[0]), router)
    assert chosen[0].tolist() == [0, 4] and torch.allclose(weight[0], torch.tensor([1.8, 1.4], dtype=torch.float64))


@pytest.mark.parametrize("case", list(zm.CASES))
def test_plain_model_is_causal(case):
    cfg, seed = zm.CASES[case]
    w = zm.make_weights(cfg, seed)
    tokens = zm.random_tokens(cfg, 21, 1)
    whole = pz.forward(cfg, w, tokens)
    assert torch.allclose(pz.forward(cfg, w, tokens[:13]), whole[:13], atol=1e-9)
    assert torch.isfinite(whole).all() and float(whole.std()) > 1e-3
