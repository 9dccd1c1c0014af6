"""Ronolorn through the engine against the plain implementation (tests/plain_ronolorn.py).

Each mechanism alone (the stream kernel, the rows of the attention projection, the delta rule's kernels, the sink and
the window in every attention kernel, one-layer models), then whole models under every way of cutting and batching:
whole prompts, prefill against token-by-token decoding, portions down to one and two tokens, unequal requests side
by side with pages and state slots used again, long decoding, the first tokens of a sequence, keys made to stand out
just inside and just outside a window, and greedy generation through the scheduler, the command line and the trace
program.
"""
import json
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_ronolorn as pr
import replay
import ronolorn_models as rm

pytestmark = pytest.mark.gpu
F = torch.float64
LENGTHS = {"a": 150, "b": 70, "c": 33, "d": 200, "e": 90, "f": 3, "g": 129, "h": 64, "i": 47, "j": 1}
_cache = {}


# ------------------------------------------------------------------ helpers
def plain(cfg, weights, tokens):
    return pr.forward(cfg, weights, tokens).numpy()


def setup(case, dtype, tmp_path_factory, gain=1.0, lengths=None):
    key = (case, dtype, gain, None if lengths is None else tuple(sorted(lengths.items())))
    if key not in _cache:
        from cisr_b200 import Model

        cfg, seed = rm.CASES[case]
        weights = rm.make_weights(cfg, seed, gain=gain)
        path = rm.write_model_dir(tmp_path_factory.mktemp(f"{case}_{dtype}"), cfg, weights)
        model = Model.from_pretrained(path, dtype=dtype)
        requests = {rid: rm.random_tokens(cfg, n, 100 + i) for i, (rid, n) in enumerate((lengths or LENGTHS).items())}
        reference = {rid: plain(cfg, weights, tokens) for rid, tokens in requests.items()}
        _cache[key] = (cfg, weights, path, model, requests, reference)
    return _cache[key]


def compare(got, requests, reference, dtype, scale=1.0):
    """float32: every logit within the replay tests' bound.  bfloat16: every row's relative RMS error below twice the
    replay tests' bound, and at most one row in a hundred (or one) above the bound itself.  The delta rule divides each
    head's read-out by its root mean square; where a read-out is nearly zero (a few positions among hundreds, found
    the same under every cut) the rounding of the layer's input is magnified tenfold there, in the plain
    implementation's arithmetic as in the engine's, while the float32 run of the same model stays inside its bound."""
    if dtype == "float32":
        return replay.compare(got, requests, reference, dtype, scale=scale)
    assert got, "nothing was compared"
    errors = {key: replay.relative_rms(row, reference[key[0]][key[1]]) for key, row in got.items()}
    assert all(np.isfinite(row).all() for row in got.values())
    worst = max(errors, key=errors.get)
    assert errors[worst] < 2 * replay.RRMS16, f"bfloat16 logits differ for request {worst[0]} at position {worst[1]}: {errors[worst]:.4f}"
    over = sorted(k for k, e in errors.items() if e >= replay.RRMS16)
    assert len(over) <= max(1, len(errors) // 100), f"bfloat16 rows over the bound: {over[:10]}"


def stepper_for(model, steps, slack_pages=0):
    from cisr_b200 import Stepper
    return Stepper(model, n_pages=replay.max_live_tokens(steps) // 16 + slack_pages, page_size=16, max_slots=4)


def model_of(cfg, weights, tmp_path, dtype="float32"):
    from cisr_b200 import Model
    return Model.from_pretrained(rm.write_model_dir(tmp_path, cfg, weights), dtype=dtype)


# ------------------------------------------------------------------ each mechanism alone
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("streams, hidden, kind", [(1, 64, "layer"), (3, 96, "layer"), (4, 200, "rms"), (7, 72, "layer"), (16, 40, "rms")])
def test_stream_kernel(dtype, streams, hidden, kind):
    """Write-back of an output with its bias, the mixing table read [from, to], the mixture and its norm; in place;
    rows picked; the first call that spreads one row over all streams."""
    from cisr_b200.ops import kernels
    g = torch.Generator().manual_seed(streams * 10 + hidden)
    T, eps = 9, 1e-5
    X = torch.randn(T, streams, hidden, generator=g, dtype=F)
    y, bias = torch.randn(T, hidden, generator=g, dtype=F), torch.randn(hidden, generator=g, dtype=F)
    mix, a, b = (torch.randn(n, generator=g, dtype=F).reshape(shape) for n, shape in
                 ((streams * streams, (streams, streams)), (streams, (streams,)), (streams, (streams,))))
    w = (1 + 0.1 * torch.randn(hidden, generator=g)).to(dtype)

    def normed(u):
        return (pr.layer_norm(u, w.to(F), eps) if kind == "layer" else pr.rms(u, eps) * w.to(F))

    want_X = torch.einsum("sr,tsw->trw", mix, X) + b[None, :, None] * (y + bias)[:, None, :]
    want_h = normed(torch.einsum("s,tsw->tw", a, want_X))
    f32 = lambda t: t.float().cuda().contiguous()
    streams_dev = f32(X)
    h = torch.empty((T, hidden), dtype=dtype, device="cuda")
    kernels.hyper_mix_norm(streams_dev, streams_dev, streams, y=f32(y), bias=f32(bias), mix=f32(mix), out_w=f32(b), in_w=f32(a),
                           norm_w=w.cuda(), eps=eps, norm_kind=kind, h=h)
    tol = 2e-5 if dtype == torch.float32 else 1.2e-2
    assert (streams_dev.cpu().to(F) - want_X).abs().max() < 1e-5 * want_X.abs().max()
    assert (h.cpu().to(F) - want_h).abs().max() < tol * want_h.abs().max()
    # rows picked, nothing stored, no output pending, plain sum as the mixture: what the final norm does
    rows = torch.tensor([7, 2, 2], dtype=torch.int32, device="cuda")
    before = streams_dev.clone()
    h = torch.empty((3, hidden), dtype=dtype, device="cuda")
    kernels.hyper_mix_norm(streams_dev, streams_dev, streams, norm_w=w.cuda(), eps=eps, norm_kind=kind, h=h, rows=rows, store=False)
    assert torch.equal(before, streams_dev)
    want = normed(want_X.sum(1))[[7, 2, 2]]
    assert (h.cpu().to(F) - want).abs().max() < tol * want.abs().max()
    # one row read as every stream
    row = torch.randn(T, hidden, generator=g, dtype=F)
    spread = torch.empty((T, streams, hidden), dtype=torch.float32, device="cuda")
    h = torch.empty((T, hidden), dtype=dtype, device="cuda")
    kernels.hyper_mix_norm(f32(row), spread, streams, in_w=f32(a), norm_w=w.cuda(), eps=eps, norm_kind=kind, h=h)
    assert torch.equal(spread.cpu(), row.float()[:, None, :].expand(T, streams, hidden))
    want = normed(a.sum() * row.float().to(F))
    assert (h.cpu().to(F) - want).abs().max() < 3 * tol * want.abs().max()
    assert torch.allclose(kernels.hyper_sum(spread, torch.empty((T, hidden), dtype=torch.float32, device="cuda")).cpu().to(F),
                          streams * row.float().to(F), rtol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("from_keys, norm, interleaved, key_dim, value_dim, rot_dims",
                         [(False, False, True, 24, 40, 8), (True, True, True, 48, 48, 32), (False, True, False, 16, 16, 16),
                          (True, False, True, 20, 20, 0), (False, False, True, 64, 32, 16)])
def test_attention_rows_kernel(dtype, from_keys, norm, interleaved, key_dim, value_dim, rot_dims):
    """Bias, norm over the whole projection, rotation, padding and the cache rows, with tokens at offsets inside pages
    that are not the request's first."""
    from cisr_b200.ops import kernels
    T, hq, hkv, page, eps = 5, 4, 2, 8, 1e-5
    D = -(-max(key_dim, value_dim) // 16) * 16
    g = torch.Generator().manual_seed(key_dim + value_dim)
    nq, nk, nv = hq * key_dim, hkv * key_dim, 0 if from_keys else hkv * value_dim
    proj = torch.randn(T, nq + nk + nv + 3, generator=g)
    bias = torch.randn(nq + nk + nv + 3, generator=g)
    wq, wk = 1 + 0.2 * torch.randn(nq, generator=g), 1 + 0.2 * torch.randn(nk, generator=g)
    positions = torch.tensor([9, 10, 11, 12, 30], dtype=torch.int32)
    rot = {"base": 777.0, "dims": rot_dims} if rot_dims else None
    half = rot_dims // 2
    cos = sin = None
    if rot:
        angle = positions.to(F)[:, None] * pr.rotary_frequencies(rot, F)[0]
        cos, sin = torch.cos(angle).float().cuda(), torch.sin(angle).float().cuda()
    row = (proj + bias).to(F)
    q, k = row[:, :nq], row[:, nq:nq + nk]
    v = k.reshape(T, hkv, key_dim) if from_keys else row[:, nq + nk:nq + nk + nv].reshape(T, hkv, value_dim)
    if norm:
        q, k = pr.rms(q, eps) * wq.to(F), pr.rms(k, eps) * wk.to(F)
    q, k = q.reshape(T, hq, key_dim), k.reshape(T, hkv, key_dim)
    if rot and interleaved:
        q, k = pr.rotate(q, positions, rot), pr.rotate(k, positions, rot)
    elif rot:                                  # split-half pairs: the engine's other rotation, restated here
        def turn(x):
            c, s = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
            out = x.clone()
            out[..., :half] = x[..., :half] * c - x[..., half:2 * half] * s
            out[..., half:2 * half] = x[..., half:2 * half] * c + x[..., :half] * s
            return out
        q, k = turn(q), turn(k)
    table = torch.full((3, 6), -1, dtype=torch.int32)
    table[1, 1], table[1, 3] = 4, 2               # positions 8..15 -> page 4, 24..31 -> page 2
    q_out = torch.full((T, hq, D), 7.0, dtype=dtype, device="cuda")
    kc = torch.zeros((6, hkv, page, D), dtype=dtype, device="cuda")
    vc = torch.zeros_like(kc)
    kernels.attention_rows(proj.cuda(), nq, -1 if from_keys else nq + nk, bias=bias.cuda(), q_norm=wq.cuda() if norm else None,
                           k_norm=wk.cuda() if norm else None, eps=eps, cos=cos, sin=sin, rot_half=half, interleaved=interleaved,
                           q_out=q_out, k_cache=kc, v_cache=vc, token_req=torch.zeros(T, dtype=torch.int32, device="cuda"),
                           positions=positions.cuda(), req_slot=torch.tensor([1], dtype=torch.int32, device="cuda"),
                           block_table=table.cuda(), page_size=page, hq=hq, hkv=hkv, key_dim=key_dim, value_dim=value_dim)
    tol = 3e-6 if dtype == torch.float32 else 8e-3
    got_q = q_out.cpu().to(F)
    assert (got_q[..., :key_dim] - q).abs().max() < tol * q.abs().max() and (got_q[..., key_dim:] == 0).all()
    for t, pos in enumerate(positions.tolist()):
        pg, off = (4, pos - 8) if pos < 16 else (2, pos - 24)
        got_k, got_v = kc[pg, :, off].cpu().to(F), vc[pg, :, off].cpu().to(F)
        assert (got_k[:, :key_dim] - k[t]).abs().max() < tol * k.abs().max() and (got_k[:, key_dim:] == 0).all()
        assert (got_v[:, :value_dim] - v[t]).abs().max() < tol * v.abs().max() and (got_v[:, value_dim:] == 0).all()
    assert int((kc != 0).any(-1).sum()) == T * hkv, "rows of other pages and offsets were touched"
    # the output bias, where no arrangement takes it into its own kernel
    y = torch.randn(T, 24, generator=g).cuda()
    b = torch.randn(24, generator=g).cuda()
    assert torch.equal(kernels.bias_add(y.clone(), b), y + b)


@pytest.mark.parametrize("lanes, long", [(0, False), (4, False), (8, False), (16, False), (32, False), (0, True), (8, True)])
@pytest.mark.parametrize("heads, kvh, dk, dv, taps", [(4, 2, 20, 24, 3), (2, 1, 32, 64, 4), (3, 3, 72, 40, 1), (1, 1, 130, 9, 2),
                                                       (2, 2, 128, 16, 5), (2, 1, 200, 8, 2), (1, 1, 256, 3, 2)])
def test_delta_kernels_carry_their_state_across_portions(heads, kvh, dk, dv, taps, lanes, long):
    """The recurrence, the convolution with kept inputs, decay, beta, unit norms and the gated output norm against the
    plain mixer on whole sequences; two requests side by side in portions down to one token (shorter than the taps),
    one of them in a slot that held another request's state before; with every number of lanes per column of the state
    that the recurrence kernel can be launched with (0: its own choice).  `long`: portions of a chunk and more, which
    run the chunked form (whole chunks, a chunk's tail, a chunk after single tokens) beside a request that stays with the
    token-by-token kernel in the same step."""
    from cisr_b200.parts.delta import CHUNKED_FROM, chunk_plan
    from cisr_b200.ops import kernels
    hidden, eps = 48, 1e-5
    g = torch.Generator().manual_seed(dk * 7 + dv)
    m = {"heads": heads, "kv_heads": kvh, "dim": dk, "vdim": dv, "conv": taps}
    W = {"q": torch.randn(kvh * dk, hidden, generator=g) / 4, "k": torch.randn(kvh * dk, hidden, generator=g) / 4,
         "v": torch.randn(heads * dv, hidden, generator=g) / 4, "q.conv": torch.randn(kvh * dk, taps, generator=g),
         "k.conv": torch.randn(kvh * dk, taps, generator=g), "v.conv": torch.randn(heads * dv, taps, generator=g),
         "b": torch.randn(heads, hidden, generator=g) / 4, "a": torch.randn(heads, hidden, generator=g) / 4,
         "A_log": torch.randn(heads, generator=g) - 1, "dt_bias": torch.randn(heads, generator=g),
         "g": torch.randn(heads * dv, hidden, generator=g) / 4, "norm": 1 + 0.1 * torch.randn(dv, generator=g),
         "o": torch.eye(heads * dv)}
    W64 = {k: v.to(F) for k, v in W.items()}
    lengths = {0: 237, 1: 140} if long else {0: 37, 1: 12}
    hs = {r: torch.randn(n, hidden, generator=g) for r, n in lengths.items()}
    want = {r: pr.mixer_delta(h.to(F), W64, "", m, eps) for r, h in hs.items()}
    stacked = torch.cat([W[k] for k in ("q", "k", "v", "g", "b", "a")]).to(F)
    conv = torch.cat([W[k] for k in ("q.conv", "k.conv", "v.conv")]).cuda().contiguous()
    channels = 2 * kvh * dk + heads * dv
    state = torch.randn(4, heads * dk * dv + (taps - 1) * channels, generator=g).cuda()     # slots hold an older request's state
    slot = {0: 2, 1: 0}
    for s in slot.values():
        state[s].zero_()                          # what the cache manager does when a request takes a slot
    cuts = {0: [70, 1, 64, 2, 100], 1: [1, 3, 129, 7]} if long else {0: [5, 1, 1, 2, 9, 1, 18], 1: [1, 1, 3, 7]}
    at = {0: 0, 1: 0}
    got = {0: [], 1: []}
    while any(cuts.values()):
        batch = [r for r in (1, 0) if cuts[r]]    # request 1 first: rows of the step are not in slot order
        sizes = [cuts[r].pop(0) for r in batch]
        rows = torch.cat([hs[r][at[r]:at[r] + n] for r, n in zip(batch, sizes)])
        proj = (rows.to(F) @ stacked.T).float().cuda().contiguous()
        q_start = np.cumsum([0] + sizes[:-1]).astype(np.int32)
        token_req = np.concatenate([np.full(n, i, dtype=np.int32) for i, n in enumerate(sizes)])
        out = torch.empty((rows.shape[0], heads * dv), dtype=torch.float32, device="cuda")
        dev = lambda a: torch.from_numpy(np.asarray(a, dtype=np.int32)).cuda()
        chunk_req, chunk_t0, req_chunk0, short = chunk_plan(sizes)
        chunks = (dev(chunk_req), dev(chunk_t0), dev(req_chunk0), len(chunk_req), short, CHUNKED_FROM) if chunk_req else None
        kernels.delta_step(proj, conv, taps, state, W["A_log"].cuda(), W["dt_bias"].cuda(), W["norm"].cuda(), eps, 1e-6,
                           dev(token_req), dev([slot[r] for r in batch]), dev(q_start), dev(sizes), len(batch), heads, kvh, dk, dv, out,
                           lanes=lanes, chunks=chunks)
        for i, (r, n) in enumerate(zip(batch, sizes)):
            got[r].append(out[q_start[i]:q_start[i] + n].cpu())
            at[r] += n
    for r in lengths:
        err = (torch.cat(got[r]).to(F) - want[r]).abs().max() / want[r].abs().max()
        assert err < 2e-5, f"request {r}: relative error {err:.2e}"


def one_attention(kind, dim, vdim, window, heads=4, kv_heads=2, scale=None, streams=2, width=64, rot_dims=None):
    rot = {"base": 2000.0, "dims": rot_dims if rot_dims is not None else dim // 2 * 2}
    return rm.one_layer(kind, rm.attention(heads, kv_heads, dim, vdim, scale or dim ** -0.5, window=window, rot=rot), ff=None,
                        streams=streams, width=width)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind, dim, vdim, window", [("attention_2", 64, 64, 45), ("attention_2", 96, 96, None), ("attention", 64, 32, 200),
                                                     ("attention_2", 128, 128, 131), ("attention", 24, 40, 17), ("attention_2", 160, 160, 64),
                                                     ("attention_2", 64, 64, 3), ("attention_2", 96, 96, 2), ("attention_2", 128, 128, 3)])
def test_every_attention_kernel_has_the_sink_and_the_window(dtype, kind, dim, vdim, window, tmp_path):
    """One attention layer, prompts long enough for every prompt kernel (128-query tensor-memory tiles at widths 64 and
    128, 64-query tiles at the others, CUDA cores in float32 and beyond 128) and decoding for the split kernels and
    their merge.  The layer's output is the whole model, so a sink left out of one kernel shows directly: the test
    first makes sure that the plain logits without the sink differ far beyond the bound.  Among dozens of keys the sink
    takes a few hundredths of the weight, which float32 shows and bfloat16 does not; the windows of two and three keys
    are there for bfloat16 (the sink then holds a quarter of the weight or more)."""
    cfg = one_attention(kind, dim, vdim, window, width=128)
    weights = rm.make_weights(cfg, dim + vdim)
    model = model_of(cfg, weights, tmp_path, dtype)
    requests = {"p": rm.random_tokens(cfg, 300, 1), "q": rm.random_tokens(cfg, 140, 2)}
    reference = {k: plain(cfg, weights, t) for k, t in requests.items()}
    if kind == "attention_2":
        real = pr.attend
        try:
            pr.attend = lambda q, k, v, scale, window, sink: real(q, k, v, scale, window, False)
            other = plain(cfg, weights, requests["q"])
        finally:
            pr.attend = real
        moved = replay.relative_rms(other[-1], reference["q"][-1])
        if window is not None and window <= 3:
            assert moved > 0.06, "the sink would not show in this test"
        elif dtype == "float32":
            assert moved > 1e-3, "the sink would not show in this test"
    for steps in (replay.trace_whole(requests), replay.trace_tail_decode(requests, 20), replay.trace_portions(requests, (130, 2, 64, 1))):
        compare(replay.run_steps(stepper_for(model, steps, slack_pages=2), steps), requests, reference, dtype, scale=2.0)


# ------------------------------------------------------------------ whole models under every cut
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", list(rm.CASES))
def test_whole_prompts(case, dtype, tmp_path_factory):
    cfg, weights, path, model, requests, reference = setup(case, dtype, tmp_path_factory)
    steps = replay.trace_whole(requests)
    compare(replay.run_steps(stepper_for(model, steps), steps), requests, reference, dtype, scale=4.0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", list(rm.CASES))
def test_prefill_against_token_by_token_decoding(case, dtype, tmp_path_factory):
    cfg, weights, path, model, requests, reference = setup(case, dtype, tmp_path_factory)
    steps = replay.trace_tail_decode(requests, 60)           # longer than every window of the models
    compare(replay.run_steps(stepper_for(model, steps), steps), requests, reference, dtype, scale=4.0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case, sizes", [("ra", (16, 2, 15, 17, 3, 64, 33)), ("rb", (2, 2, 1, 5)), ("rc", (128, 7, 2, 130)), ("ra", (1,))])
def test_portions_of_several_sizes(case, sizes, dtype, tmp_path_factory):
    cfg, weights, path, model, requests, reference = setup(case, dtype, tmp_path_factory)
    if sizes == (1,) or sizes == (2, 2, 1, 5):
        requests = {k: requests[k] for k in ("b", "c", "f", "j")}
    steps = replay.trace_portions(requests, sizes)
    compare(replay.run_steps(stepper_for(model, steps), steps), requests, reference, dtype, scale=4.0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", list(rm.CASES))
def test_unequal_requests_side_by_side_with_pages_and_slots_used_again(case, dtype, tmp_path_factory):
    cfg, weights, path, model, requests, reference = setup(case, dtype, tmp_path_factory)
    steps = replay.trace_mixed(requests, seed=7)
    stepper = stepper_for(model, steps)
    compare(replay.run_steps(stepper, steps), requests, reference, dtype, scale=4.0)
    assert not stepper.cache.requests and len(stepper.cache.free_slots) == 4
    assert all(g.pool.n_free == g.pool.n_pages for g in stepper.cache.page_groups)
    assert any(g.pool.taken > g.pool.n_pages for g in stepper.cache.page_groups), "no page was used twice"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sizes_that_are_no_multiples_of_eight(dtype, tmp_path):
    """Width, feed-forward width, head widths and vocabulary that fit no 16-byte group: the products take the paths
    that have no alignment to rely on, the padded operands stay zero where they are padding."""
    cfg = {"architecture": "Ronolorn", "vocab": 83, "width": 100, "embedding": {"scale": 3.0}, "norm": {"eps": 1e-5}, "streams": 5,
           "layers": [rm.layer("attention", rm.attention(3, 1, 10, 6, 0.3, window=21, rot={"base": 900.0, "dims": 6}), 50),
                      rm.layer("delta", rm.delta(3, 1, 7, 5, 2), 33),
                      rm.layer("attention_2", rm.attention(2, 2, 18, 18, 0.2, window=9, rot={"base": 5000.0, "dims": 18, "scaling": rm.YARN}), 27)]}
    weights = rm.make_weights(cfg, 77)
    model = model_of(cfg, weights, tmp_path, dtype)
    requests = {"u": rm.random_tokens(cfg, 140, 1), "v": rm.random_tokens(cfg, 37, 2)}
    reference = {k: plain(cfg, weights, t) for k, t in requests.items()}
    for steps in (replay.trace_whole(requests), replay.trace_mixed(requests, seed=2, max_live=2), replay.trace_portions(requests, (2, 15, 1))):
        compare(replay.run_steps(stepper_for(model, steps, slack_pages=2), steps), requests, reference, dtype, scale=4.0)


@pytest.mark.parametrize("kinds", [("delta", "delta"), ("attention_2",), ("attention", "attention")])
def test_models_of_one_kind_of_mixer(kinds, tmp_path):
    """Only recurrent layers (no pages at all, state slots alone), only attention (no state): the cache manager, the
    launch plans and the trace of mixed steps must not count on the other kind being there."""
    mixers = {"delta": rm.delta(2, 1, 24, 20, 3), "attention": rm.attention(2, 1, 24, 20, 0.2, window=11, rot={"base": 800.0, "dims": 10}),
              "attention_2": rm.attention(3, 1, 32, 32, 0.2, window=13, rot={"base": 800.0, "dims": 32})}
    cfg = {"architecture": "Ronolorn", "vocab": 61, "width": 48, "embedding": {"scale": 2.0}, "norm": {"eps": 1e-5}, "streams": 2,
           "layers": [rm.layer(k, mixers[k], 40 if i == 0 else None) for i, k in enumerate(kinds)]}
    weights = rm.make_weights(cfg, 3)
    model = model_of(cfg, weights, tmp_path)
    requests = {"m": rm.random_tokens(cfg, 90, 1), "n": rm.random_tokens(cfg, 30, 2), "o": rm.random_tokens(cfg, 5, 3)}
    reference = {k: plain(cfg, weights, t) for k, t in requests.items()}
    for steps in (replay.trace_whole(requests), replay.trace_mixed(requests, seed=4, max_live=3)):
        compare(replay.run_steps(stepper_for(model, steps, slack_pages=2), steps), requests, reference, "float32", scale=4.0)


def test_a_request_alone_and_in_a_crowd(tmp_path_factory):
    """The same request by itself and beside three others of other lengths, portion by portion and token by token:
    float32 logits agree far inside the comparison's bound (the products may choose another kernel by the step's
    token count; everything else is the same arithmetic in the same order)."""
    from cisr_b200 import StepEntry, Stepper
    cfg, weights, path, model, requests, reference = setup("ra", "float32", tmp_path_factory)
    target = requests["e"]
    cuts = [30, 2, 17, 1, 1, 1, 20, 1, 1] + [1] * 16
    alone = Stepper(model, n_pages=40, page_size=16, max_slots=4)
    crowd = Stepper(model, n_pages=40, page_size=16, max_slots=4)
    alone.create("t")
    for key in ("x", "t", "y", "z"):
        crowd.create(key)
    others = {"x": requests["a"], "y": requests["d"], "z": requests["g"]}
    at, step = 0, 0
    for n in cuts:
        want = list(range(n))
        a = alone.step([StepEntry("t", target[at:at + n], want)]).cpu().numpy()
        entries = [StepEntry("x", others["x"][3 * step:3 * step + 3], []), StepEntry("t", target[at:at + n], want),
                   StepEntry("y", others["y"][step:step + 1], [0]), StepEntry("z", others["z"][4 * step:4 * step + 4], [])]
        b = crowd.step(entries).cpu().numpy()[:n]
        for i in range(n):
            assert replay.relative_rms(a[i], b[i].astype(np.float64)) < 2e-6, f"position {at + i} depends on its neighbours"
            compare({("e", at + i): a[i]}, requests, reference, "float32", scale=4.0)
        at += n
        step += 1


def test_long_decoding_through_windows_and_state(tmp_path_factory):
    """330 tokens one by one from the first: every window passes over decoded tokens many times, pages go back to
    their pools while the request lives, and the recurrence carries its state through every step."""
    cfg, weights, path, model, _, _ = setup("ra", "float32", tmp_path_factory)
    requests = {"long": rm.random_tokens(cfg, 330, 77)}
    reference = {"long": plain(cfg, weights, requests["long"])}
    steps = replay.trace_portions(requests, (1,))
    stepper = stepper_for(model, steps)
    compare(replay.run_steps(stepper, steps), requests, reference, "float32", scale=4.0)
    assert all(g.pool.peak <= -(-g.use.window // 16) + 1 for g in stepper.cache.page_groups), "a window kept pages it had passed"


def test_first_tokens_of_a_sequence(tmp_path_factory):
    """Positions 0, 1, 2, ...: the convolution's zeros before the sequence, an empty state, windows that are not full
    yet and the sink's weight beside a single key, whole, in two-token portions and one by one, also with nothing
    wanted in a step."""
    cfg, weights, path, model, _, _ = setup("ra", "float32", tmp_path_factory)
    requests = {f"s{n}": rm.random_tokens(cfg, n, 300 + n) for n in (1, 2, 3, 4, 6, 9)}
    reference = {k: plain(cfg, weights, t) for k, t in requests.items()}
    for steps in (replay.trace_whole(requests), replay.trace_portions(requests, (2,)), replay.trace_portions(requests, (1,))):
        compare(replay.run_steps(stepper_for(model, steps), steps), requests, reference, "float32", scale=4.0)
    nothing_wanted = [{"step": 0, "entries": [{"id": "s9", "tokens": requests["s9"][:5], "want": []}], "end": []},
                      {"step": 1, "entries": [{"id": "s9", "tokens": requests["s9"][5:], "want": [3]}], "end": ["s9"]}]
    got = replay.run_steps(stepper_for(model, nothing_wanted), nothing_wanted)
    assert list(got) == [("s9", 8)]
    compare(got, requests, reference, "float32", scale=4.0)


@pytest.mark.parametrize("kind", ["attention", "attention_2"])
def test_keys_just_inside_and_just_outside_the_window(kind, tmp_path):
    """One attention layer is the whole model, so the last position sees exactly its window.  A token that occurs
    nowhere else is put at the window's oldest place and one place beyond; the plain implementation says that the
    first moves the last logits and the second does not move them at all, and the engine must agree with it with
    the prompt whole, decoded (the window passing page borders on the way) and in portions that cut at the edge."""
    from cisr_b200 import Stepper
    window, n = 37, 150
    cfg = one_attention(kind, 32, 32, window, scale=0.5, width=64)
    weights = rm.make_weights(cfg, 5, gain=2.0)
    model = model_of(cfg, weights, tmp_path)
    rng = np.random.default_rng(0)
    filler = [int(t) for t in rng.integers(0, cfg["vocab"] - 8, size=n)]
    without = plain(cfg, weights, filler)[-1]
    for distance, seen in ((window - 1, True), (window, False), (0, True), (1, True)):
        place = n - 1 - distance
        effect = {}
        for b in range(cfg["vocab"] - 8, cfg["vocab"]):
            tokens = list(filler)
            tokens[place] = b
            effect[b] = replay.relative_rms(plain(cfg, weights, tokens)[-1], without)
        key = max(effect, key=effect.get)
        if seen:
            assert effect[key] > 1e-3, f"a key {distance} back does not matter: the test would show nothing"
        else:
            assert effect[key] == 0.0, "a key beyond the window moved the plain logits"
        tokens = list(filler)
        tokens[place] = key
        requests, reference = {"r": tokens}, {"r": plain(cfg, weights, tokens)}
        for steps in (replay.trace_whole(requests), replay.trace_tail_decode(requests, 60),
                      replay.trace_portions(requests, (place, 1, window - 2, 2, 1)), replay.trace_portions(requests, (place + 1, window - 1, 5))):
            compare(replay.run_steps(Stepper(model, n_pages=12, page_size=16, max_slots=2), steps), requests, reference, "float32")


def test_sharp_attention_depends_on_single_keys(tmp_path_factory):
    """With the query and key projections scaled up the softmax is peaked: each query's weight sits on one or two keys
    somewhere in its window, so a wrong, missing or stale cache row shows.  float32 only."""
    lengths = {"x": 300, "y": 170, "z": 61}
    cfg, weights, path, model, requests, reference = setup("rc", "float32", tmp_path_factory, gain=3.0, lengths=lengths)
    for steps in (replay.trace_whole(requests), replay.trace_mixed(requests, seed=3), replay.trace_tail_decode(requests, 140),
                  replay.trace_portions(requests, (16, 2, 15, 17, 3, 64, 33))):
        compare(replay.run_steps(stepper_for(model, steps), steps), requests, reference, "float32", scale=8.0)


def test_repeated_step_shapes_replay_from_graphs_with_state_and_chunks(tmp_path_factory):
    """Portions of the same lengths recur: from the second time on the step is a graph replay.  The portions are long
    enough for the chunked recurrence (its chunk lists travel with the graph's metadata) and pass the windows; single
    tokens beside them take the token-by-token kernel in the same captured step.  The warm-up run in front of a capture
    must not advance any request's recurrent state twice."""
    from cisr_b200 import StepEntry, Stepper
    cfg, weights, path, model, _, _ = setup("ra", "float32", tmp_path_factory)
    stepper = Stepper(model, n_pages=60, page_size=16, max_slots=4, graph=True)
    tokens = {k: rm.random_tokens(cfg, 231, 20 + i) for i, k in enumerate("abcd")}
    reference = {k: plain(cfg, weights, t) for k, t in tokens.items()}
    got = {}
    for k in "abcd":
        stepper.create(k)
    plan = [[("a", 0, 100)], [("b", 0, 100)], [("c", 0, 100)], [("d", 0, 100)], [("a", 100, 100)],
            [("b", 100, 70), ("a", 200, 1)], [("c", 100, 70), ("a", 201, 1)], [("d", 100, 70), ("b", 170, 1)],
            [("a", 202, 1), ("b", 171, 1)], [("a", 203, 1), ("b", 172, 1)], [("a", 204, 1), ("b", 173, 1)]]
    for step in plan:
        entries = [StepEntry(k, tokens[k][at:at + n], [n - 1, 0] if n > 1 else [0]) for k, at, n in step]
        logits = stepper.step(entries).cpu().numpy()
        row = 0
        for k, at, n in step:
            for w in ([n - 1, 0] if n > 1 else [0]):
                got[(k, at + w)] = logits[row].copy()
                row += 1
        stepper.cache.check()
    compare(got, tokens, reference, "float32", scale=4.0)
    report = stepper.graphs.report()
    assert report["shape_entries"] >= 2 and report["hits"] >= 4


# ------------------------------------------------------------------ generation through the scheduler and the command line
@pytest.mark.parametrize("case, graph", [("ra", False), ("ra", True), ("rc", False)])
def test_greedy_generation_through_the_scheduler(case, graph, tmp_path_factory):
    """More requests than slots, few pages: requests wait, run in portions under a token budget, decode side by side,
    end, and their pages and state slots serve the next ones.  float32 tokens equal the plain greedy choice.  (A model
    with a recurrent mixer runs without captured graphs whatever is asked.)"""
    from cisr_b200 import Engine, Request
    cfg, weights, path, model, _, _ = setup(case, "float32", tmp_path_factory)
    prompts = {f"g{i}": rm.random_tokens(cfg, n, 50 + i) for i, n in enumerate((19, 5, 40, 2, 27, 11))}
    new = 7

    def plain_greedy(prompt):
        seq = list(prompt)
        for _ in range(new):
            seq.append(int(pr.forward(cfg, weights, seq)[-1].argmax()))
        return seq[len(prompt):]

    engine = Engine.for_model(model, pages=6, page_size=16, max_active=3, token_budget=24, prefill_chunk=9, policy="decode_first", graph=graph)
    for key, prompt in prompts.items():
        engine.submit(Request(key, prompt, max_new_tokens=new))
    got = {r.key: r.generated for r in engine.run()}
    assert got == {k: plain_greedy(p) for k, p in prompts.items()}
    assert not engine.stepper.cache.requests and all(g.pool.n_free == g.pool.n_pages for g in engine.stepper.cache.page_groups)


def test_command_line_and_trace_program(tmp_path_factory, tmp_path):
    cfg, weights, path, model, requests, reference = setup("rb", "float32", tmp_path_factory)
    short = {k: requests[k] for k in ("c", "f", "i", "j", "h")}
    steps = replay.trace_mixed(short, seed=5, max_live=4)
    got = replay.run_trace_program(path, "float32", steps, tmp_path / "out", replay.max_live_tokens(steps), cfg["vocab"])
    compare(got, short, reference, "float32", scale=4.0)
    got = replay.run_trace_program(path, "bfloat16", steps, tmp_path / "out16", replay.max_live_tokens(steps), cfg["vocab"])
    compare(got, short, reference, "bfloat16")
    listing = tmp_path / "requests.json"
    listing.write_text(json.dumps([{"key": "only", "prompt": requests["c"][:9], "max_new_tokens": 4}]))
    proc = subprocess.run([sys.executable, "-m", "cisr_b200", "--config", "ronolorn-small", "--dtype", "float32", "--requests", str(listing),
                           "--pages", "16"], capture_output=True, text=True, timeout=900, cwd=str(replay.ROOT))
    assert proc.returncode == 0, proc.stderr[-3000:]
    out = json.loads(proc.stdout[proc.stdout.index("{"):])
    assert out["weights"] == "random-ronolorn-small" and len(out["requests"][0]["generated"]) == 4
