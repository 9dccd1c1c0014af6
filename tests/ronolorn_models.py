"""Small Ronolorn configurations and seeded weights for the tests.

The shapes differ from one another in what a configuration can set: several streams, one stream with its tensors, no
stream key at all (the plain residual sum); key and value heads of different widths and widths that need padding;
grouped and ungrouped heads; windows of a few keys, of one key, and none; rotation of part of a head, of a whole
head, with and without stretched frequencies, and none; convolutions of one to five taps; layers without a
feed-forward; every order of the three mixers.
"""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import torch


def attention(heads, kv_heads, dim, vdim, scale, window=None, rot=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    if rot is not None:
        m["rot"] = rot
    return m


def delta(heads, kv_heads, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def layer(kind, mix, ff):
    return {"type": kind, "mixer": mix, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


YARN = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 0.5}

# three streams; padded heads (24 / 40 -> 48); a layer without a feed-forward; delta with grouped and ungrouped heads
RA = {
    "architecture": "Ronolorn", "vocab": 173, "width": 96, "embedding": {"scale": 5.0}, "norm": {"eps": 1e-5}, "streams": 3,
    "layers": [
        layer("attention", attention(6, 2, 24, 40, 0.2, window=19, rot={"base": 3000.0, "dims": 8}), 136),
        layer("delta", delta(4, 2, 20, 24, 3), 72),
        layer("attention_2", attention(4, 2, 48, 48, 0.15, window=33, rot={"base": 70000.0, "dims": 32, "scaling": YARN}), None),
        layer("delta", delta(3, 3, 40, 16, 5), 40),
        layer("attention", attention(2, 2, 16, 16, 0.3, window=7, rot={"base": 500.0, "dims": 16, "scaling": dict(YARN, factor=2.0)}), 64),
    ],
}

# no stream key: the plain residual sum; attention without a window, without rotation, with a window of one; one tap
RB = {
    "architecture": "Ronolorn", "vocab": 97, "width": 64, "embedding": {"scale": 1.0}, "norm": {"eps": 3e-6},
    "layers": [
        layer("attention_2", attention(5, 1, 32, 32, 0.18, rot={"base": 25000.0, "dims": 12}), 56),
        layer("delta", delta(2, 1, 72, 40, 1), None),
        layer("attention", attention(3, 3, 40, 24, 0.25), 48),
        layer("attention_2", attention(2, 1, 16, 16, 0.4, window=1), 24),
        layer("delta", delta(1, 1, 130, 9, 2), 80),
    ],
}

# one stream with its tensors; tensor-core head widths (64, 128); rotation of the whole head
RC = {
    "architecture": "Ronolorn", "vocab": 300, "width": 192, "embedding": {"scale": 8.0}, "norm": {"eps": 1e-6}, "streams": 1,
    "layers": [
        layer("attention", attention(8, 4, 64, 64, 0.125, window=130, rot={"base": 300000.0, "dims": 64}), 200),
        layer("attention_2", attention(4, 1, 128, 128, 0.09, window=50, rot={"base": 12345.0, "dims": 64, "scaling": YARN}), 128),
        layer("delta", delta(4, 2, 64, 64, 4), 96),
    ],
}

CASES = {"ra": (RA, 41), "rb": (RB, 42), "rc": (RC, 43)}


def one_layer(kind, mix, ff=None, streams=2, width=64, vocab=101, scale=2.0):
    cfg = {"architecture": "Ronolorn", "vocab": vocab, "width": width, "embedding": {"scale": scale}, "norm": {"eps": 1e-6},
           "layers": [layer(kind, mix, ff)]}
    if streams is not None:
        cfg["streams"] = streams
    return cfg


def tensor_shapes(cfg: dict) -> dict:
    w, v = cfg["width"], cfg["vocab"]
    shapes = {"embed": (v, w), "final.norm": (w,)}
    s = cfg.get("streams")
    for i, spec in enumerate(cfg["layers"]):
        p, m = f"l{i}.", spec["mixer"]
        H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        shapes[p + "norm1"] = (w,)
        if spec["type"] == "delta":
            taps = m["conv"]
            shapes.update({p + "mix.q": (G * d, w), p + "mix.k": (G * d, w), p + "mix.v": (H * dv, w),
                           p + "mix.q.conv": (G * d, taps), p + "mix.k.conv": (G * d, taps), p + "mix.v.conv": (H * dv, taps),
                           p + "mix.b": (H, w), p + "mix.a": (H, w), p + "mix.A_log": (H,), p + "mix.dt_bias": (H,),
                           p + "mix.g": (H * dv, w), p + "mix.norm": (dv,), p + "mix.o": (w, H * dv)})
        else:
            shapes.update({p + "mix.q": (H * d, w), p + "mix.q.b": (H * d,), p + "mix.k": (G * d, w), p + "mix.k.b": (G * d,),
                           p + "mix.o": (w, H * dv)})
            if spec["type"] == "attention":
                shapes.update({p + "mix.v": (G * dv, w), p + "mix.v.b": (G * dv,), p + "mix.o.b": (w,)})
            else:
                shapes.update({p + "mix.q.norm": (H * d,), p + "mix.k.norm": (G * d,)})
        if spec.get("mlp"):
            shapes.update({p + "norm2": (w,), p + "mlp.up": (spec["mlp"]["ff"], w), p + "mlp.down": (w, spec["mlp"]["ff"])})
        if s is not None:
            for q in ("1", "2") if spec.get("mlp") else ("1",):
                shapes.update({p + f"hc{q}.in": (s,), p + f"hc{q}.out": (s,), p + f"hc{q}.mix": (s, s)})
    return shapes


def make_weights(cfg: dict, seed: int, gain: float = 1.0) -> dict:
    """Seeded weights, every value representable in bfloat16 (so a bfloat16 engine and a float oracle start alike).

    Matrices N(0, gain / sqrt(inputs)) (`gain` scales the mixers' input projections only: a larger one makes the
    softmax peaked); biases, stream weights and the recurrence's constants spread widely, so that leaving one out, or
    reading the mixing table the wrong way round, moves the logits."""
    rng = np.random.default_rng(seed)
    s = cfg.get("streams") or 1
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        if name.endswith(".b") and len(shape) == 1:
            value = 0.3 * rng.standard_normal(shape)
        elif name.endswith("hc1.in") or name.endswith("hc2.in"):
            value = 1.0 / s + 0.3 / s * rng.standard_normal(shape)
        elif name.endswith(".out") and "hc" in name:
            value = 1.0 + 0.3 * rng.standard_normal(shape)
        elif name.endswith(".mix") and "hc" in name:
            value = np.eye(s) * 0.8 + 0.2 / s + 0.15 * rng.standard_normal(shape)
        elif name.endswith(".conv"):
            value = 0.6 * rng.standard_normal(shape) + (np.arange(shape[1]) == shape[1] - 1) * 0.5
        elif name.endswith("A_log"):
            value = -1.0 + 0.7 * rng.standard_normal(shape)
        elif name.endswith("dt_bias"):
            value = rng.standard_normal(shape)
        elif len(shape) == 1:
            value = 1.0 + 0.1 * rng.standard_normal(shape)
        elif name == "embed":
            value = rng.standard_normal(shape) / cfg["embedding"]["scale"]
        elif ".mix." in name and name.rsplit(".", 1)[1] in ("q", "k"):
            value = gain / np.sqrt(shape[1]) * rng.standard_normal(shape)
        else:
            value = 1.0 / np.sqrt(shape[1]) * rng.standard_normal(shape)
        out[name] = torch.from_numpy(np.asarray(value, dtype=np.float32)).to(torch.bfloat16).to(torch.float32)
    return out


def write_model_dir(path, cfg: dict, weights: dict) -> Path:
    from safetensors.torch import save_file

    path = Path(path)
    path.mkdir(parents=True, exist_ok=True)
    (path / "config.json").write_text(json.dumps(cfg, indent=1))
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in weights.items()}, str(path / "model.safetensors"))
    return path


def random_tokens(cfg: dict, n: int, seed: int) -> list:
    rng = np.random.default_rng(seed)
    return [int(t) for t in rng.integers(0, cfg["vocab"], size=n)]
