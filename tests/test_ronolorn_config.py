"""Ronolorn on the CPU: what its configuration class reads and refuses, the tensor names the assembled model asks for,
the caches its mixers ask for, the stretched rotary frequencies, and properties of the plain implementation."""
import copy
import math

import pytest
import torch

import plain_ronolorn as pr
import ronolorn_models as rm
from cisr_b200.config import ConfigError, PartSpec, architecture_for
from cisr_b200.engine.model import Model


def spec_of(cfg):
    return architecture_for(cfg).config_class.from_dict(cfg).to_spec()


def test_registry_picks_the_design_by_its_architecture_key():
    assert architecture_for(rm.RA).name == "Ronolorn"


@pytest.mark.parametrize("case", list(rm.CASES))
def test_model_asks_for_exactly_the_checkpoint_tensors(case):
    cfg, _ = rm.CASES[case]
    needs = Model(spec_of(cfg), "bfloat16", config=cfg, device=None).tensor_needs()
    assert {k: tuple(v.shape) for k, v in needs.items() if v.alias is None} == rm.tensor_shapes(cfg)
    assert needs["head"].alias == "embed"          # the head is the embedding table itself


def test_preset_builds():
    from cisr_b200.config import preset_dict
    spec = spec_of(preset_dict("ronolorn-small"))
    assert [l.mixer.kind for l in spec.layers] == ["windowed_attention", "gated_delta", "windowed_attention"]


def test_parts_take_their_constants_from_the_configuration():
    spec = spec_of(rm.RA)
    first, second, third = spec.layers[0].mixer, spec.layers[1].mixer, spec.layers[2].mixer
    assert first.kind == "windowed_attention" and first["window"] == 19 and first["sink"] is None and first["qk_norm"] is None
    assert set(first["bias"]) == {"q", "k", "v", "o"} and not first["values_from_keys"] and first["scale"] == 0.2
    assert first["position"].kind == "rotary_interleaved" and first["position"]["dim"] == 8 and "scaling" not in first["position"].params
    assert second.kind == "gated_delta" and second["conv"] == 3 and second["eps"] == 1e-5
    assert third["sink"] == 0.0 and third["qk_norm"] == "whole" and third["values_from_keys"] and set(third["bias"]) == {"q", "k"}
    assert third["position"]["scaling"]["factor"] == 4.0
    assert spec.layers[2].feed_forward is None and "feed_forward_hyper" not in spec.layers[2].extras
    assert spec.stream.kind == "hyper" and spec.stream["streams"] == 3 and spec.embedding["scale"] == 5.0
    plain = spec_of(rm.RB)
    assert plain.stream["streams"] == 1 and not plain.layers[0].extras
    assert plain.layers[0].mixer["window"] is None and plain.layers[2].mixer["position"].kind == "none"
    assert spec_of(rm.RC).layers[0].extras["mixer_hyper"]["streams"] == 1


def test_caches_windows_get_pools_of_their_own_and_the_recurrence_a_state_slot():
    model = Model(spec_of(rm.RA), "float32", config=rm.RA, device=None)
    uses = model.cache_uses()
    assert [(u.kind, u.head_dim, u.window) for u in uses if u.kind == "pages"] == [("pages", 48, 19), ("pages", 48, 33), ("pages", 16, 7)]
    d1, d2 = uses[1], uses[3]
    assert d1.kind == "state" and d1.state_shape == (4 * 20 * 24 + 2 * (2 * 2 * 20 + 4 * 24),)
    assert d2.state_shape == (3 * 40 * 16 + 4 * (2 * 3 * 40 + 3 * 16),)
    cache = model.make_cache(8, 16, 2)
    assert len(cache.page_groups) == 3 and len(cache.state_groups) == 2


@pytest.mark.parametrize("change, message", [
    (lambda c: c["layers"][0].__setitem__("type", "hyena"), "not a mixer"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 7), "rot"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("kv_heads", 4), "multiple"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("vdim", 32), "vdim"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("dim", 300), "dim"),
    (lambda c: c["layers"][1]["mixer"].pop("conv"), "conv"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "moe"), "dense"),
    (lambda c: c.__setitem__("streams", 40), "streams"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("dim", 272), "256"),
])
def test_refusals_come_before_any_weight_is_read(change, message):
    cfg = copy.deepcopy(rm.RA)
    change(cfg)
    with pytest.raises(ConfigError, match=message):
        architecture_for(cfg).config_class.from_dict(cfg)


@pytest.mark.parametrize("rot", [{"base": 70000.0, "dims": 32, "scaling": rm.YARN}, {"base": 400000.0, "dims": 40,
                                  "scaling": {"factor": 16.0, "original": 1024, "fast": 24.0, "slow": 2.0}},
                                 {"base": 100.0, "dims": 6, "scaling": {"factor": 1.5, "original": 8, "fast": 1.0, "slow": 1.0}}])
def test_stretched_frequencies_match_the_plain_ones(rot):
    from cisr_b200.parts.rotary import scaled_frequencies
    plain, magnitude = pr.rotary_frequencies(rot, torch.float64)
    base = rot["base"] ** (-torch.arange(rot["dims"] // 2, dtype=torch.float64) * 2.0 / rot["dims"])
    got, got_magnitude = scaled_frequencies(base, rot["base"], rot["dims"], dict(rot["scaling"], kind="yarn"))
    assert torch.allclose(got, plain, rtol=1e-14, atol=0) and got_magnitude == magnitude
    assert magnitude == 0.1 * math.log(rot["scaling"]["factor"]) + 1.0


def test_plain_delta_rule_reads_its_own_write_and_forgets_by_its_decay():
    """With beta = 1 and no decay the state returns v for the key just written; q = k reads it back at once."""
    d, dv = 6, 4
    g = torch.Generator().manual_seed(0)
    k = torch.nn.functional.normalize(torch.randn(d, generator=g, dtype=torch.float64), dim=0)
    v = torch.randn(dv, generator=g, dtype=torch.float64)
    S = torch.randn(d, dv, generator=g, dtype=torch.float64)
    u = 1.0 * (v - S.T @ k)
    S = S + torch.outer(k, u)
    assert torch.allclose(S.T @ k, v)


def test_plain_sink_takes_weight_from_the_keys():
    g = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn(5, 2, 8, generator=g, dtype=torch.float64) for _ in range(3))
    plain = pr.attend(q, k, v, 0.3, None, sink=False)
    sunk = pr.attend(q, k, v, 0.3, None, sink=True)
    assert (sunk.abs() < plain.abs() + 1e-12).all() and not torch.allclose(sunk, plain)
    # the first token sees itself alone: weight e^s / (1 + e^s) with the sink, 1 without
    s = (q[0, 0] @ k[0, 0]) * 0.3
    assert torch.allclose(sunk[0, :8], v[0, 0] * torch.exp(s) / (1 + torch.exp(s)))
    assert torch.allclose(plain[0, :8], v[0, 0])


def test_plain_window_edges():
    ok = pr.visible(6, 3)
    assert ok[5].tolist() == [False, False, False, True, True, True] and ok[1].tolist() == [True, True, False, False, False, False]
    assert pr.visible(4, None)[3].all() and pr.visible(4, 1).sum() == 4


def test_chunk_plan_of_the_delta_rule():
    """Portions of a chunk and more are cut into chunks (the last may be short); shorter ones and single tokens have none
    and are counted for the token-by-token kernel; every request knows where its chunks start."""
    from cisr_b200.parts.delta import CHUNKED_FROM, chunk_plan
    assert CHUNKED_FROM == 64
    chunk_req, chunk_t0, req_chunk0, short = chunk_plan([130, 1, 64, 63, 200])
    assert chunk_req == [0, 0, 0, 2, 4, 4, 4, 4] and chunk_t0 == [0, 64, 128, 0, 0, 64, 128, 192]
    assert req_chunk0 == [0, 3, 3, 4, 4] and short == 2
    assert chunk_plan([1, 1, 1]) == ([], [], [0, 0, 0], 3)


def test_the_delta_mixer_plans_with_the_step():
    from cisr_b200.engine.batch import HostBatch
    model = Model(spec_of(rm.RA), "float32", config=rm.RA, device=None)
    keys = {type(p).__name__: p.plan_key() for p in model.planners()}
    assert set(keys) == {"WindowedAttention", "GatedDelta"}          # one plan per key, whatever the number of layers
    delta = [p for p in model.planners() if type(p).__name__ == "GatedDelta"][0]
    plan = delta.step_plan(HostBatch(["a", "b"], [0, 1], [0, 70], [70, 1], [70, 9], 71, []))
    assert plan.info == {"n_chunks": 2, "n_short": 1} and plan.arrays["chunk_t0"].tolist() == [0, 64]
