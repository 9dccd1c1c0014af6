"""A plain, slow Zurolorn: one function per mechanism, whole sequences on the CPU in float64.

Nothing here is shared with the engine: no cache, no pages, no kernels.  A sequence is run as a whole
(every position sees all earlier ones), so the engine's ways of cutting a prompt can be held against it.
`weights` maps checkpoint names to tensors; `config` is the config.json dict.

With `round_to` set to torch.bfloat16, values are rounded there where the engine's serving path rounds
them (operands of matrix products), so that the twin shows what storage alone costs.
"""
from __future__ import annotations

import torch

F = torch.float64
SCORE_LOG = None      # a list here receives (scores [T, experts], router settings) of every routing, in run order


def rms_unit(x, eps):
    """x over its root mean square, eps inside the root."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x, weight, eps):
    return rms_unit(x, eps) * weight


def rotate(v, positions, base, dims, interleaved):
    """Turn the first `dims` coordinates of the last axis of v [T, ..., D] by position * base^(-2i/dims).

    Pairs are (i, i + dims/2), or (2i, 2i + 1) when interleaved; the rest passes unchanged."""
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F)
    angle = positions.to(F)[:, None] * freq[None, :]                 # [T, half]
    shape = [v.shape[0]] + [1] * (v.dim() - 2) + [half]
    cos, sin = torch.cos(angle).reshape(shape), torch.sin(angle).reshape(shape)
    out = v.clone()
    if interleaved:
        a, b = v[..., 0:dims:2], v[..., 1:dims:2]
        out[..., 0:dims:2] = a * cos - b * sin
        out[..., 1:dims:2] = b * cos + a * sin
    else:
        a, b = v[..., :half], v[..., half:dims]
        out[..., :half] = a * cos - b * sin
        out[..., half:dims] = b * cos + a * sin
    return out


def causal_softmax_attention(q, k, v, scale):
    """q, k [T, H, Dk], v [T, H, Dv]; position i sees every j <= i."""
    T = q.shape[0]
    scores = torch.einsum("ihd,jhd->hij", q, k) * scale
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    scores = scores.masked_fill(~mask, float("-inf"))
    weights = torch.softmax(scores, dim=-1)
    return torch.einsum("hij,jhd->ihd", weights, v)


def latent_attention(h, w, prefix, mixer, positions, eps, kind, rnd):
    """Both latent mixers.  `kind` "latent_attention": direct queries, split-half pairs, output gate;
    "latent_attention_2": queries through a normed latent, interleaved pairs, no gate."""
    H, dn, dr, dv, rank = mixer["heads"], mixer["dim"], mixer["rot_dim"], mixer["vdim"], mixer["kv_rank"]
    second = kind == "latent_attention_2"
    T = h.shape[0]
    g = lambda name: w[prefix + name].to(F)
    if second:
        cq = rnd(rms_norm(h @ g("dq").T, g("dq.norm"), eps))
        q = cq @ g("uq").T
    else:
        q = h @ g("q").T
    q = q.view(T, H, dn + dr)
    down = h @ g("dkv").T
    c = rnd(rms_norm(down[:, :rank], g("dkv.norm"), eps))
    k_rot = down[:, rank:rank + dr]
    base, dims = mixer["rot"]["base"], mixer["rot"]["dims"]
    q_rot = rotate(q[..., dn:], positions, base, dims, interleaved=second)
    k_rot = rnd(rotate(k_rot[:, None, :], positions, base, dims, interleaved=second))      # [T, 1, dr]
    k_plain = (c @ g("uk").T).view(T, H, dn)
    value = (c @ g("uv").T).view(T, H, dv)
    qf = torch.cat((q[..., :dn], q_rot), dim=-1)
    kf = torch.cat((k_plain, k_rot.expand(T, H, dr)), dim=-1)
    mixed = causal_softmax_attention(qf, kf, value, mixer["scale"]).reshape(T, H * dv)
    if not second:
        mixed = mixed * torch.sigmoid(h @ g("g").T)
    return rnd(mixed) @ g("o").T


def route(h, router_w, router):
    """Chosen experts [T, top] and their weights: sigmoid scores, groups of neighbours scored by their two best,
    the best `keep` groups stay open, the `top` best open experts are taken, weight = score * scale."""
    E, top = router["experts"], router["top"]
    s = torch.sigmoid(h @ router_w.to(F).T)                                   # [T, E]
    if SCORE_LOG is not None:
        SCORE_LOG.append((s, router))
    allowed = torch.ones_like(s, dtype=torch.bool)
    groups = router.get("groups")
    if groups:
        count, keep = groups["count"], groups["keep"]
        per = E // count
        grouped = s.view(-1, count, per)
        group_score = grouped.topk(min(2, per), dim=-1).values.sum(-1)       # [T, count]
        best = group_score.topk(keep, dim=-1).indices
        open_ = torch.zeros_like(group_score, dtype=torch.bool).scatter_(1, best, True)
        allowed = open_[:, :, None].expand(-1, count, per).reshape(-1, E)
    chosen = s.masked_fill(~allowed, -1.0).topk(top, dim=-1).indices
    return chosen, s.gather(1, chosen) * router["scale"]


def expert_mixture(h, w, prefix, mlp, rnd):
    router = mlp["router"]
    chosen, weight = route(h, w[prefix + "router"], router)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(chosen[t].tolist(), weight[t]):
            up = torch.relu(w[f"{prefix}e{e}.up"].to(F) @ h[t]) ** 2
            out[t] += a * (w[f"{prefix}e{e}.down"].to(F) @ rnd(up))
    return out


def layer_order(config):
    """[(layer index, pass number or None)]: pass number t where the pass's vector is added before the layer."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, None) for i in range(start)]
    for t in range(times):
        for i in range(start, stop):
            order.append((i, t if i == start else None))
    return order + [(i, None) for i in range(stop, n)]


def forward(config, weights, tokens, round_to=None, return_layers=False):
    """Logits [T, vocab] (float64) of one sequence; with return_layers also the stream after every layer run."""
    rnd = (lambda x: x) if round_to is None else (lambda x: x.to(round_to).to(F))
    eps = config["norm"]["eps"]
    ids = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(len(ids))
    x = weights["embed"].to(F)[ids] * config["embedding"]["scale"]
    after = []
    for index, step in layer_order(config):
        spec = config["layers"][index]
        p = f"l{index}."
        if step is not None:
            x = x + weights["loop.step"].to(F)[step]
        h = rnd(rms_norm(x, weights[p + "norm1"].to(F), eps))
        mixed = latent_attention(h, weights, p + "mix.", spec["mixer"], positions, eps, spec["type"], rnd)
        x = x + mixed * weights[p + "ls1"].to(F)
        if spec.get("mlp"):
            h = rnd(rms_norm(x, weights[p + "norm2"].to(F), eps))
            x = x + expert_mixture(h, weights, p + "mlp.", spec["mlp"], rnd) * weights[p + "ls2"].to(F)
        after.append(x.clone())
    h = rnd(rms_norm(x, weights["final.norm"].to(F), eps))
    logits = (h @ weights["head"].to(F).T) * config["logit_scale"]
    return (logits, torch.stack(after)) if return_layers else logits
