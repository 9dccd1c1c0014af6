"""Zurolorn through the engine against the plain implementation (tests/plain_zurolorn.py).

Each mechanism alone (router, experts, the kernels around the latent mixer, one-layer models), then whole models under
every way of cutting and batching: whole prompts, prefill against token-by-token decoding, portions down to two tokens,
unequal requests side by side with pages and slots used again, long decoding across many pages, the first tokens of a
sequence, single far keys made to stand out, and greedy generation through the scheduler and the command line.

float32 runs are held to the float64 plain implementation with the routers as configured.  In bfloat16 a token whose
router scores (or group scores) lie close takes another expert once the router's input is rounded, and with it another
path through the model, which is no fault of the arithmetic; among hundreds of tokens some always do.  The bfloat16
runs of whole models therefore use the same shapes with routers that have no choice to make (every expert is taken,
every group kept; the scores still weight the experts), and the choice itself is tested in bfloat16 where the inputs
are equal to the bit: in the router kernel's own test.
"""
import json
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_zurolorn as pz
import replay
import zurolorn_models as zm

pytestmark = pytest.mark.gpu
F = torch.float64
LENGTHS = {"a": 150, "b": 70, "c": 33, "d": 200, "e": 90, "f": 3, "g": 129, "h": 64, "i": 47, "j": 111}
_cache = {}


# ------------------------------------------------------------------ helpers
def without_choice(cfg):
    """The same shapes with routers that take every expert (and keep every group)."""
    cfg = json.loads(json.dumps(cfg))
    for spec in cfg["layers"]:
        if spec.get("mlp"):
            router = spec["mlp"]["router"]
            router["top"] = router["experts"]
            if router.get("groups"):
                router["groups"]["keep"] = router["groups"]["count"]
    return cfg


def setup(case, dtype, tmp_path_factory, gain=1.0, lengths=None):
    key = (case, dtype, gain, None if lengths is None else tuple(sorted(lengths.items())))
    if key not in _cache:
        from cisr_b200 import Model

        cfg, seed = zm.CASES[case]
        if dtype == "bfloat16":
            cfg = without_choice(cfg)
        weights = zm.make_weights(cfg, seed, gain=gain)
        path = zm.write_model_dir(tmp_path_factory.mktemp(f"{case}_{dtype}"), cfg, weights)
        model = Model.from_pretrained(path, dtype=dtype)
        requests = {rid: zm.random_tokens(cfg, n, 100 + i) for i, (rid, n) in enumerate((lengths or LENGTHS).items())}
        reference = {rid: pz.forward(cfg, weights, tokens).numpy() for rid, tokens in requests.items()}
        _cache[key] = (cfg, weights, path, model, requests, reference)
    return _cache[key]


def stepper_for(model, steps, slack_pages=0):
    from cisr_b200 import Stepper
    return Stepper(model, n_pages=replay.max_live_tokens(steps) // 16 + slack_pages, page_size=16, max_slots=4)


# ------------------------------------------------------------------ each mechanism alone
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts, top, groups, keep, hidden", [(8, 2, 4, 2, 128), (6, 1, 0, 0, 72), (9, 2, 3, 1, 40), (16, 4, 8, 3, 192),
                                                                (4, 4, 2, 2, 64), (12, 3, 12, 5, 96)])
def test_router_kernel(dtype, experts, top, groups, keep, hidden):
    """The router part alone (logits by the engine's product, choice by the selection kernel), inputs equal to the bit."""
    from cisr_b200.config import PartSpec
    from cisr_b200.parts import FEED_FORWARDS, build_part
    g = torch.Generator().manual_seed(experts * 100 + top)
    h = torch.randn(57, hidden, generator=g).to(dtype)
    w = (3.0 / hidden ** 0.5 * torch.randn(experts, hidden, generator=g)).to(dtype)
    router = {"experts": experts, "top": top, "scale": 1.75}
    if groups:
        router["groups"] = {"count": groups, "keep": keep}
    want_ids, want_w = pz.route(h.to(F), w.to(F), router)
    part = build_part(FEED_FORWARDS, PartSpec("routed_experts", {"hidden_size": hidden, "expert_size": 8, "experts": experts, "top": top,
                                                                 "groups": groups, "keep": keep, "route_scale": 1.75}), dtype, "feed-forward")
    from cisr_b200.ops import build
    build.compile_many(part.kernel_jobs())
    tensors = {"router.weight": w.cuda()}
    for e in range(experts):
        tensors[f"experts.{e}.up.weight"] = torch.zeros(8, hidden, dtype=dtype, device="cuda")
        tensors[f"experts.{e}.down.weight"] = torch.zeros(hidden, 8, dtype=dtype, device="cuda")
    part.load(tensors)
    chosen, weight = part.route(h.cuda())
    assert torch.equal(chosen.cpu().long(), want_ids), "the router chose other experts (inputs are equal to the bit, float sums differ in the last place only)"
    assert torch.allclose(weight.cpu().to(F), want_w, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens, experts, top, ff, hidden", [(1, 4, 2, 40, 72), (13, 8, 3, 96, 128), (150, 6, 1, 24, 64), (300, 16, 4, 64, 192),
                                                              (700, 5, 2, 200, 328), (3, 40, 2, 136, 72)])
def test_expert_kernels(dtype, tokens, experts, top, ff, hidden):
    from cisr_b200.ops import kernels
    g = torch.Generator().manual_seed(tokens)
    h = torch.randn(tokens, hidden, generator=g).to(dtype)
    up = (torch.randn(experts, ff, hidden, generator=g) / hidden ** 0.5).to(dtype)
    down = (torch.randn(experts, hidden, ff, generator=g) / ff ** 0.5).to(dtype)
    chosen = torch.stack([torch.randperm(experts, generator=g)[:top] for _ in range(tokens)]).to(torch.int32)
    weight = torch.rand(tokens, top, generator=g) * 2
    want = torch.zeros(tokens, hidden, dtype=F)
    for t in range(tokens):
        for k in range(top):
            e = int(chosen[t, k])
            act = torch.relu(up[e].to(F) @ h[t].to(F)) ** 2
            want[t] += weight[t, k].to(F) * (down[e].to(F) @ (act.to(dtype).to(F)))
    act = torch.empty((tokens * top, ff), dtype=dtype, device="cuda")
    out = torch.empty((tokens, hidden), dtype=torch.float32, device="cuda")
    kernels.moe_rows(h.cuda(), up.cuda(), down.cuda(), chosen.cuda(), weight.cuda(), act, out)
    err = (out.cpu().to(F) - want).abs().max() / want.abs().max()
    assert err < (2e-6 if dtype == torch.float32 else 8e-3), f"relative error {err:.2e}"
    if dtype == torch.bfloat16 and hidden % 8 == 0 and ff % 8 == 0:
        # the same sum by the path for many tokens: sorted by expert, grouped tensor-core products (here also with experts
        # that no token chose, blocks of one row, and row tiles that stay unused)
        grouped = torch.full((tokens, hidden), 7.0, dtype=torch.float32, device="cuda")
        kernels.moe_grouped(h.cuda(), up.cuda(), down.cuda(), chosen.cuda(), weight.cuda(), grouped)
        err = (grouped.cpu().to(F) - want).abs().max() / want.abs().max()
        assert err < 8e-3, f"grouped products: relative error {err:.2e}"
        kernels.raise_if_kernel_gave_up()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("interleaved", [False, True])
def test_latent_row_and_query_kernels(dtype, interleaved):
    """Unit norms, rotation and the cache row layout, with a token at an offset inside a page that is not the request's first."""
    from cisr_b200.ops import kernels
    T, q_rank, kv_rank, rot, heads, plain, row, page = 5, 24, 40, 12, 3, 20, 64, 8
    g = torch.Generator().manual_seed(3)
    proj = torch.randn(T, q_rank + kv_rank + rot + 7, generator=g)
    qn, cn = 1 + 0.1 * torch.randn(q_rank, generator=g), 1 + 0.1 * torch.randn(kv_rank, generator=g)
    positions = torch.tensor([9, 10, 11, 12, 30], dtype=torch.int32)
    angle = positions.to(F)[:, None] * torch.tensor([777.0 ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=F)
    cos, sin = torch.cos(angle).float().cuda(), torch.sin(angle).float().cuda()
    cache = torch.full((6, 1, page, row), 9.0, dtype=dtype, device="cuda")
    table = torch.tensor([[-1, 4, 2, 5, -1, -1], [0, 1, -1, 3, -1, -1]], dtype=torch.int32, device="cuda")
    token_req = torch.tensor([0, 0, 0, 0, 0], dtype=torch.int32, device="cuda")
    req_slot = torch.tensor([1], dtype=torch.int32, device="cuda")
    cq = torch.empty((T, q_rank), dtype=dtype, device="cuda")
    kernels.latent_rows(proj.cuda(), 0, q_rank, qn.cuda(), cq, q_rank, kv_rank, cn.cuda(), 1e-5, cos, sin, rot // 2, interleaved, cache,
                        token_req, positions.cuda(), req_slot, table, page)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert torch.allclose(cq.cpu().to(F), pz.rms_norm(proj[:, :q_rank].to(F), qn.to(F), 1e-5), atol=tol, rtol=tol)
    want_c = pz.rms_norm(proj[:, q_rank:q_rank + kv_rank].to(F), cn.to(F), 1e-5)
    want_k = pz.rotate(proj[:, None, q_rank + kv_rank:q_rank + kv_rank + rot].to(F), positions, 777.0, rot, interleaved)[:, 0]
    for t, pos in enumerate(positions.tolist()):
        got = cache[int(table[1, pos // page]), 0, pos % page].cpu().to(F)
        assert torch.allclose(got[:kv_rank], want_c[t], atol=tol, rtol=tol) and torch.allclose(got[kv_rank:kv_rank + rot], want_k[t], atol=tol, rtol=tol)
        assert (got[kv_rank + rot:] == 0).all()
    assert (cache[2] == 9).all() and (cache[4] == 9).all() and (cache[5] == 9).all()      # pages of the other slot's row stay untouched
    q = torch.randn(T, heads * (plain + rot) + 3, generator=g)
    q_plain = torch.empty((T, heads, plain), dtype=dtype, device="cuda")
    q_rows = torch.full((T, heads, row), 7.0, dtype=dtype, device="cuda")
    kernels.latent_query(q.cuda(), 0, heads, plain, cos, sin, rot // 2, interleaved, q_plain, q_rows, kv_rank)
    qh = q[:, :heads * (plain + rot)].view(T, heads, plain + rot).to(F)
    assert torch.allclose(q_plain.cpu().to(F), qh[..., :plain], atol=tol, rtol=tol)
    assert torch.allclose(q_rows[..., kv_rank:kv_rank + rot].cpu().to(F), pz.rotate(qh[..., plain:], positions, 777.0, rot, interleaved), atol=tol, rtol=tol)
    assert (q_rows[..., kv_rank + rot:] == 0).all() and (q_rows[..., :kv_rank] == 7).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("interleaved, gate", [(False, True), (True, False)])
def test_few_token_kernels_around_the_attention(dtype, interleaved, gate):
    """The row kernels of decode steps: queries carried into the latent's basis (with their rotated part), and the value
    matrix applied to the weighted sum of cache rows (with the gate), against the plain formulas."""
    from cisr_b200.ops import kernels
    T, heads, plain, rot, kv_rank, vdim, row = 3, 5, 24, 12, 40, 28, 64
    g = torch.Generator().manual_seed(11)
    q = torch.randn(T, heads * (plain + rot) + 5, generator=g)
    k_up = (torch.randn(heads, plain, kv_rank, generator=g) / plain ** 0.5).to(dtype)
    positions = torch.tensor([0, 77, 1030])
    angle = positions.to(F)[:, None] * torch.tensor([500.0 ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=F)
    cos, sin = torch.cos(angle).float().cuda(), torch.sin(angle).float().cuda()
    q_rows = torch.full((T, heads, row), 3.0, dtype=dtype, device="cuda")
    kernels.latent_absorb(q.cuda(), 0, heads, plain, cos, sin, rot // 2, interleaved, k_up.cuda(), q_rows, kv_rank)
    qh = q[:, :heads * (plain + rot)].view(T, heads, plain + rot)
    want = torch.einsum("thd,hdr->thr", qh[..., :plain].to(dtype).to(F), k_up.to(F))
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert torch.allclose(q_rows[..., :kv_rank].cpu().to(F), want, atol=tol, rtol=tol)
    assert torch.allclose(q_rows[..., kv_rank:kv_rank + rot].cpu().to(F), pz.rotate(qh[..., plain:].to(F), positions, 500.0, rot, interleaved), atol=tol, rtol=tol)
    assert (q_rows[..., kv_rank + rot:] == 0).all()
    mixed = torch.randn(T, heads, row, generator=g).to(dtype)
    v_up = (torch.randn(heads, vdim, kv_rank, generator=g) / kv_rank ** 0.5).to(dtype)
    gates = torch.randn(T, 9 + heads * vdim, generator=g)
    out = torch.empty((T, heads * vdim), dtype=dtype, device="cuda")
    kernels.latent_values(mixed.cuda(), v_up.cuda(), gates.cuda() if gate else None, 9, out)
    want = torch.einsum("thr,hjr->thj", mixed[..., :kv_rank].to(F), v_up.to(F)).reshape(T, heads * vdim)
    if gate:
        want = want * torch.sigmoid(gates[:, 9:].to(F))
    assert torch.allclose(out.cpu().to(F), want, atol=tol, rtol=tol)


def one_layer(kind, mlp, loop=None):
    m = zm.mixer(kind, 3, 24, 8, 40, 48, 4321.0, q_rank=36)
    cfg = {"architecture": "Zurolorn", "vocab": 50, "width": 88, "embedding": {"scale": 2.0}, "norm": {"eps": 1e-5}, "logit_scale": 2.0,
           "layers": [zm.layer(kind, m, mlp)]}
    if loop:
        cfg["loop"] = loop
    return cfg


@pytest.mark.parametrize("name, cfg", [
    ("mixer with direct queries and gate", one_layer("latent_attention", None)),
    ("mixer with latent queries", one_layer("latent_attention_2", None)),
    ("experts", one_layer("latent_attention", zm.moe(6, 2, 32, 1.5, groups=(3, 2)))),
    ("one layer run four times", one_layer("latent_attention_2", zm.moe(4, 1, 16, 0.5), loop={"start": 0, "stop": 1, "times": 4})),
])
def test_one_layer_models_float32(name, cfg, tmp_path):
    """A model of one layer isolates each mechanism: prompt in one step, then in two-token portions, then token by token."""
    from cisr_b200 import Model, Stepper
    weights = zm.make_weights(cfg, 5)
    model = Model.from_pretrained(zm.write_model_dir(tmp_path, cfg, weights), dtype="float32")
    requests = {"p": zm.random_tokens(cfg, 41, 1), "q": zm.random_tokens(cfg, 18, 2)}
    reference = {rid: pz.forward(cfg, weights, t).numpy() for rid, t in requests.items()}
    for steps in (replay.trace_whole(requests), replay.trace_portions(requests, (2,)), replay.trace_portions(requests, (1,))):
        replay.compare(replay.run_steps(Stepper(model, n_pages=8, page_size=16, max_slots=2), steps), requests, reference, "float32")


# ------------------------------------------------------------------ whole models under every cut
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", list(zm.CASES))
@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed"])
def test_replay_matches_plain(case, dtype, mode, tmp_path_factory):
    cfg, weights, path, model, requests, reference = setup(case, dtype, tmp_path_factory)
    steps = {"whole": lambda: replay.trace_whole(requests), "tail": lambda: replay.trace_tail_decode(requests, 32),
             "portions": lambda: replay.trace_portions(requests, (7, 2, 13, 5, 2, 31, 64, 3)),
             "mixed": lambda: replay.trace_mixed(requests, seed=7)}[mode]()
    stepper = stepper_for(model, steps)
    got = replay.run_steps(stepper, steps)
    assert len(got) == sum(LENGTHS.values())
    replay.compare(got, requests, reference, dtype)
    assert not stepper.cache.requests
    for group in stepper.cache.page_groups:
        assert group.pool.n_free == group.pool.n_pages
        if mode == "mixed":
            assert group.pool.taken > group.pool.n_pages       # pages were used again


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_request_is_the_same_alone_and_in_a_crowd(dtype, tmp_path_factory):
    """Unequal requests side by side (portions beside single tokens) against each alone: equal up to rounding."""
    cfg, weights, path, model, requests, reference = setup("zc", dtype, tmp_path_factory)
    crowd = replay.run_steps(stepper_for(model, replay.trace_mixed(requests, seed=11)), replay.trace_mixed(requests, seed=11))
    alone = replay.run_steps(stepper_for(model, replay.trace_whole(requests)), replay.trace_whole(requests))
    bound = 2e-5 if dtype == "float32" else 0.03
    for key, row in crowd.items():
        assert replay.relative_rms(row, alone[key].astype(np.float64)) < bound, f"request {key[0]} position {key[1]} depends on its neighbours"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_crosses_many_pages(dtype, tmp_path_factory):
    cfg, weights, path, model, _, _ = setup("za", dtype, tmp_path_factory)
    tokens = zm.random_tokens(cfg, 330, 77)
    reference = {"long": pz.forward(cfg, weights, tokens).numpy()}
    steps = [{"step": 0, "entries": [{"id": "long", "tokens": tokens[:3], "want": [0, 1, 2]}], "end": []}]
    steps += [{"step": i - 2, "entries": [{"id": "long", "tokens": [tokens[i]], "want": [0]}], "end": []} for i in range(3, len(tokens))]
    got = replay.run_steps(stepper_for(model, steps), steps)
    replay.compare(got, {"long": tokens}, reference, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decoding_from_captured_graphs(dtype, tmp_path_factory):
    """Decode steps replayed from CUDA graphs (two requests side by side, contexts crossing a graph's context bucket) give the
    plain implementation's logits like steps launched directly."""
    from cisr_b200 import StepEntry, Stepper
    cfg, weights, path, model, _, _ = setup("zc", dtype, tmp_path_factory)
    requests = {"u": zm.random_tokens(cfg, 90, 5), "v": zm.random_tokens(cfg, 61, 6)}
    reference = {rid: pz.forward(cfg, weights, t).numpy() for rid, t in requests.items()}
    stepper = Stepper(model, n_pages=12, page_size=16, max_slots=2, graph=True)
    assert stepper.graphs is not None, "the mixers of this design are safe to capture"
    got, heads = {}, {"u": 40, "v": 11}
    for rid, tokens in requests.items():
        stepper.create(rid)
        stepper.step([StepEntry(rid, tokens[:heads[rid]], [])])
    for i in range(50):
        logits = stepper.step([StepEntry(rid, [requests[rid][heads[rid] + i]], [0]) for rid in requests]).cpu().numpy()
        for row, rid in enumerate(requests):
            got[(rid, heads[rid] + i)] = logits[row].copy()
    stepper.check_kernels()
    replay.compare(got, requests, reference, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_of_a_sequence(dtype, tmp_path_factory):
    """Prompts of one, two and three tokens, alone and side by side, and logits wanted only at some places."""
    cfg, weights, path, model, _, _ = setup("zb", dtype, tmp_path_factory)
    requests = {f"s{n}": zm.random_tokens(cfg, n, n) for n in (1, 2, 3, 17)}
    reference = {rid: pz.forward(cfg, weights, t).numpy() for rid, t in requests.items()}
    side_by_side = [{"step": 0, "entries": [{"id": rid, "tokens": t, "want": [len(t) - 1]} for rid, t in requests.items()],
                     "end": list(requests)}]
    got = replay.run_steps(stepper_for(model, side_by_side), side_by_side)
    assert sorted(got) == sorted((rid, len(t) - 1) for rid, t in requests.items())
    check = lambda rows: replay.compare(rows, requests, reference, dtype)
    check(got)
    check(replay.run_steps(stepper_for(model, replay.trace_portions(requests, (1,))), replay.trace_portions(requests, (1,))))
    nothing_wanted = [{"step": 0, "entries": [{"id": "s17", "tokens": requests["s17"][:9], "want": []}], "end": []},
                      {"step": 1, "entries": [{"id": "s17", "tokens": requests["s17"][9:], "want": [7]}], "end": ["s17"]}]
    got = replay.run_steps(stepper_for(model, nothing_wanted), nothing_wanted)
    assert list(got) == [("s17", 16)]
    check(got)


def test_sharp_attention_depends_on_single_far_keys(tmp_path_factory):
    """With every matrix of the mixers scaled up the softmax is peaked and each query's weight sits on one or two keys
    anywhere in its past (hundreds of tokens back, across page borders, in decoding and in prompts): a wrong, missing
    or stale cache row shows in the logits.  float32 only: a peaked model amplifies bfloat16 rounding."""
    lengths = {"x": 300, "y": 170, "z": 61}
    cfg, weights, path, model, requests, reference = setup("zb", "float32", tmp_path_factory, gain=2.5, lengths=lengths)
    for steps in (replay.trace_whole(requests), replay.trace_mixed(requests, seed=3), replay.trace_tail_decode(requests, 70),
                  replay.trace_portions(requests, (16, 2, 15, 17, 3, 64, 33))):
        replay.compare(replay.run_steps(stepper_for(model, steps), steps), requests, reference, "float32", scale=4.0)


def test_one_far_key_stands_out(tmp_path):
    """One key that carries weight, placed at the start, around a page border and around the border of the decode
    kernel's key ranges, hundreds of positions before the query that is compared.  For each place the token is picked
    (by the plain implementation) whose presence there moves the last logits most, and it occurs nowhere else; the test
    makes sure that it matters (replacing it moves the logits fifty times beyond the comparison's bound), then holds
    the engine to the plain implementation with the prompt whole, decoded, and in portions."""
    from cisr_b200 import Model, Stepper
    cfg = one_layer("latent_attention_2", None)
    cfg["layers"][0]["mixer"]["scale"] = 0.6
    weights = zm.make_weights(cfg, 9)
    model = Model.from_pretrained(zm.write_model_dir(tmp_path, cfg, weights), dtype="float32")
    rng = np.random.default_rng(0)
    n = 420
    for place in (0, 15, 16, 17, 255, 256):
        filler = [int(t) for t in rng.integers(0, cfg["vocab"] - 8, size=n)]        # the last eight tokens are kept for the key
        without = pz.forward(cfg, weights, filler)[-1].numpy()
        effect = {}
        for b in range(cfg["vocab"] - 8, cfg["vocab"]):
            tokens = list(filler)
            tokens[place] = b
            effect[b] = replay.relative_rms(pz.forward(cfg, weights, tokens)[-1].numpy(), without)
        key = max(effect, key=effect.get)
        assert effect[key] > 1e-3, f"no token at place {place} matters for the last position: the test would show nothing"
        tokens = list(filler)
        tokens[place] = key
        requests, reference = {"r": tokens}, {"r": pz.forward(cfg, weights, tokens).numpy()}
        for steps in (replay.trace_whole(requests), replay.trace_tail_decode(requests, 40), replay.trace_portions(requests, (33, 2, 100))):
            replay.compare(replay.run_steps(Stepper(model, n_pages=28, page_size=16, max_slots=2), steps), requests, reference, "float32")


# ------------------------------------------------------------------ generation through the scheduler and the command line
@pytest.mark.parametrize("graph", [False, True])
def test_greedy_generation_through_the_scheduler(graph, tmp_path_factory):
    """More requests than slots, few pages: requests wait, run in portions under a token budget, decode side by side, end,
    and their pages and slots serve the next ones.  float32 tokens equal the plain implementation's greedy choice."""
    from cisr_b200 import Engine, Request
    cfg, weights, path, model, _, _ = setup("za", "float32", tmp_path_factory)
    prompts = {f"g{i}": zm.random_tokens(cfg, n, 50 + i) for i, n in enumerate((19, 5, 40, 2, 27, 11))}
    new = 7

    def plain_greedy(prompt):
        seq = list(prompt)
        for _ in range(new):
            seq.append(int(pz.forward(cfg, weights, seq)[-1].argmax()))
        return seq[len(prompt):]

    engine = Engine.for_model(model, pages=6, page_size=16, max_active=3, token_budget=24, prefill_chunk=9, policy="decode_first", graph=graph)
    for key, prompt in prompts.items():
        engine.submit(Request(key, prompt, max_new_tokens=new))
    got = {r.key: r.generated for r in engine.run()}
    assert got == {k: plain_greedy(p) for k, p in prompts.items()}
    assert not engine.stepper.cache.requests and all(g.pool.n_free == g.pool.n_pages for g in engine.stepper.cache.page_groups)
    assert all(g.pool.taken > g.pool.n_pages for g in engine.stepper.cache.page_groups)


def test_command_line_and_trace_program(tmp_path_factory, tmp_path):
    cfg, weights, path, model, requests, reference = setup("zb", "float32", tmp_path_factory)
    short = {k: requests[k] for k in ("c", "f", "i")}
    steps = replay.trace_mixed(short, seed=5, max_live=2)
    got = replay.run_trace_program(path, "float32", steps, tmp_path / "out", replay.max_live_tokens(steps), cfg["vocab"])
    replay.compare(got, short, reference, "float32")
    listing = tmp_path / "requests.json"
    listing.write_text(json.dumps([{"key": "only", "prompt": requests["c"][:9], "max_new_tokens": 4}]))
    proc = subprocess.run([sys.executable, "-m", "cisr_b200", "--config", "zurolorn-small", "--dtype", "float32", "--requests", str(listing),
                           "--pages", "16"], capture_output=True, text=True, timeout=900, cwd=str(replay.ROOT))
    assert proc.returncode == 0, proc.stderr[-3000:]
    out = json.loads(proc.stdout[proc.stdout.index("{"):])
    assert out["weights"] == "random-zurolorn-small" and len(out["requests"][0]["generated"]) == 4
