"""Ronolorn, plainly: whole sequences, no cache, one function per mechanism, torch on the CPU in one float type.

This file shares no code with the engine.  It is the oracle of the engine's tests: slow loops where a loop says
what happens (the recurrence walks the tokens one by one, attention builds the full score matrix).

    weights: dict name -> tensor (any float type; widened here)
    config:  the config.json dict of the design
"""
from __future__ import annotations

import math

import torch


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def layer_norm(x, w, eps):
    """(x - mean) / sqrt(var + eps) * w over the last axis; var is the mean squared deviation; no bias."""
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w


def rms(x, eps):
    """x divided by its root mean square over the last axis (eps inside the root)."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rotary_frequencies(rot, dtype):
    """One frequency per pair of the rotated part, and the factor both tables are multiplied by."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=dtype)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def turn_dim(t):          # the pair index whose wave makes t turns over the original length
        return dims * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(turn_dim(float(sc["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(sc["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x, positions, rot):
    """x [T, heads, dim]: the first rot.dims coordinates of each head turn, neighbours (2i, 2i+1) paired."""
    if not rot:
        return x
    dims = int(rot["dims"])
    f, mag = rotary_frequencies(rot, x.dtype)
    a = positions.to(x.dtype)[:, None] * f[None, :]                 # [T, dims/2]
    cos, sin = (torch.cos(a) * mag)[:, None, :], (torch.sin(a) * mag)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def visible(T, window):
    """[T, T] mask: query i sees key j when 0 <= i - j (< window, when there is one)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = (i - j) >= 0
    if window is not None:
        ok &= (i - j) < window
    return ok


def attend(q, k, v, scale, window, sink):
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H * dv].  sink: one more term exp(0) in the denominator."""
    T, H, _ = q.shape
    G = k.shape[1]
    ok = visible(T, window)
    out = []
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        s = s.masked_fill(~ok, float("-inf"))
        m = s.max(-1, keepdim=True).values
        if sink:
            m = m.clamp(min=0.0)
        e = torch.exp(s - m)
        den = e.sum(-1, keepdim=True) + (torch.exp(-m) if sink else 0.0)
        out.append((e / den) @ v[:, g])
    return torch.cat(out, dim=-1)


def mixer_attention(h, W, p, m, positions):
    """Biased projections, rotation of part of each head, a window of keys, ordinary softmax."""
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = (h @ W[p + "q"].T + W[p + "q.b"]).view(T, H, d)
    k = (h @ W[p + "k"].T + W[p + "k.b"]).view(T, G, d)
    v = (h @ W[p + "v"].T + W[p + "v.b"]).view(T, G, dv)
    q, k = rotate(q, positions, m.get("rot")), rotate(k, positions, m.get("rot"))
    window = int(m["mask"]["size"]) if m.get("mask") else None
    a = attend(q, k, v, float(m["scale"]), window, sink=False)
    return a @ W[p + "o"].T + W[p + "o.b"]


def mixer_attention_2(h, W, p, m, positions, eps):
    """Values are the keys as projected; q and k normed over their whole projection; a sink in the softmax."""
    T = h.shape[0]
    H, G, d = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
    q = h @ W[p + "q"].T + W[p + "q.b"]
    k = h @ W[p + "k"].T + W[p + "k.b"]
    v = k.view(T, G, d)
    q = (rms(q, eps) * W[p + "q.norm"]).view(T, H, d)
    k = (rms(k, eps) * W[p + "k.norm"]).view(T, G, d)
    q, k = rotate(q, positions, m.get("rot")), rotate(k, positions, m.get("rot"))
    window = int(m["mask"]["size"]) if m.get("mask") else None
    a = attend(q, k, v, float(m["scale"]), window, sink=True)
    return a @ W[p + "o"].T


def short_conv(x, w):
    """x [T, C], w [C, taps]: y[t, c] = sum_j w[c, taps-1-j] x[t-j, c], zeros before the start; then silu."""
    T, C = x.shape
    taps = w.shape[1]
    y = torch.zeros_like(x)
    for j in range(taps):
        shifted = torch.zeros_like(x)
        if j < T:
            shifted[j:] = x[: T - j]
        y = y + shifted * w[:, taps - 1 - j]
    return y * torch.sigmoid(y)


def mixer_delta(h, W, p, m, eps):
    """Gated delta rule, token by token."""
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = short_conv(h @ W[p + "q"].T, W[p + "q.conv"]).view(T, G, d)
    k = short_conv(h @ W[p + "k"].T, W[p + "k.conv"]).view(T, G, d)
    v = short_conv(h @ W[p + "v"].T, W[p + "v.conv"]).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ W[p + "b"].T)                                            # [T, H]
    decay = torch.exp(-torch.exp(W[p + "A_log"]) * torch.nn.functional.softplus(h @ W[p + "a"].T + W[p + "dt_bias"]))
    gate = (h @ W[p + "g"].T).view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hd in range(H):
        g = hd // (H // G)
        S = torch.zeros(d, dv, dtype=h.dtype)
        for t in range(T):
            S = decay[t, hd] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            out[t, hd] = S.T @ q[t, g]
    out = rms(out, eps) * W[p + "norm"] * (gate * torch.sigmoid(gate))
    return out.reshape(T, H * dv) @ W[p + "o"].T


def feed_forward(h, W, p):
    z = torch.relu(h @ W[p + "up"].T)
    return (z * z) @ W[p + "down"].T


def run_mixer(kind, h, W, p, m, positions, eps):
    if kind == "attention":
        return mixer_attention(h, W, p, m, positions)
    if kind == "attention_2":
        return mixer_attention_2(h, W, p, m, positions, eps)
    if kind == "delta":
        return mixer_delta(h, W, p, m, eps)
    raise ValueError(kind)


def forward(config, weights, tokens, dtype=torch.float64, collect=None):
    """Logits [T, vocab] of one sequence.  `collect`: a list that receives the residual stream (the sum of the
    streams) after every layer."""
    W = {k: v.to(dtype) for k, v in weights.items()}
    eps = float(config["norm"]["eps"])
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(tokens.numel())
    x = W["embed"][tokens] * float(config["embedding"]["scale"])
    streams = config.get("streams")
    X = x[None].repeat(int(streams), 1, 1) if streams else None
    for i, layer in enumerate(config["layers"]):
        L = f"l{i}."
        subs = [("1", lambda h: run_mixer(layer["type"], h, W, L + "mix.", layer["mixer"], positions, eps))]
        if layer.get("mlp") is not None:
            subs.append(("2", lambda h: feed_forward(h, W, L + "mlp.")))
        for q, fn in subs:
            if X is None:
                x = x + fn(layer_norm(x, W[L + "norm" + q], eps))
            else:
                a, b, M = W[L + f"hc{q}.in"], W[L + f"hc{q}.out"], W[L + f"hc{q}.mix"]
                u = torch.einsum("s,stw->tw", a, X)
                y = fn(layer_norm(u, W[L + "norm" + q], eps))
                X = torch.einsum("sr,stw->rtw", M, X) + b[:, None, None] * y[None]
        if collect is not None:
            collect.append(x.clone() if X is None else X.sum(0))
    if X is not None:
        x = X.sum(0)
    return layer_norm(x, W["final.norm"], eps) @ W["embed"].T
