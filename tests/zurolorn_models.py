"""Small Zurolorn configurations and seeded weights for the tests.

The shapes differ from one another in everything a configuration can set: widths that are not powers of two, head,
value and latent sizes that all differ, cache rows that need padding (kv_rank + rot_dim not a multiple of 16), a
layer without a feed-forward, routers with and without groups, one and several kept groups, top 1 and more, loops
over one or several layers, a loop that runs once, and no loop at all.
"""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import torch


def mixer(kind, heads, dim, rot_dim, vdim, kv_rank, base, q_rank=None, scale=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
         "rot": {"base": base, "dims": rot_dim}, "scale": (dim + rot_dim) ** -0.5 if scale is None else scale}
    if kind == "latent_attention_2":
        m["q_rank"] = q_rank
    return m


def moe(experts, top, ff, scale, groups=None):
    router = {"experts": experts, "top": top, "scale": scale}
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router}


def layer(kind, mix, mlp):
    return {"type": kind, "mixer": mix, "mlp": mlp}


# two looped layers run three times, a layer without a feed-forward, two kept groups of four
ZA = {
    "architecture": "Zurolorn", "vocab": 211, "width": 128, "embedding": {"scale": 3.0}, "norm": {"eps": 1e-5}, "logit_scale": 0.5,
    "layers": [
        layer("latent_attention", mixer("latent_attention", 4, 32, 16, 48, 64, 10000.0), moe(8, 2, 96, 1.5, groups=(4, 2))),
        layer("latent_attention_2", mixer("latent_attention_2", 3, 48, 32, 40, 80, 70000.0, q_rank=56), None),
        layer("latent_attention_2", mixer("latent_attention_2", 2, 16, 16, 24, 32, 500.0, q_rank=24), moe(6, 1, 40, 0.7)),
    ],
    "loop": {"start": 0, "stop": 2, "times": 3},
}

# no loop; rows that need padding (40 + 12 = 52 -> 64); a router without groups and one with three groups of which one is kept
ZB = {
    "architecture": "Zurolorn", "vocab": 97, "width": 72, "embedding": {"scale": 1.0}, "norm": {"eps": 3e-6}, "logit_scale": 1.0,
    "layers": [
        layer("latent_attention_2", mixer("latent_attention_2", 5, 24, 12, 16, 40, 25000.0, q_rank=48), moe(5, 3, 56, 2.5)),
        layer("latent_attention", mixer("latent_attention", 2, 40, 24, 56, 96, 1e6, scale=0.2), moe(9, 2, 24, 1.0, groups=(3, 1))),
    ],
}

# a loop over the last layer alone that runs once; the widest row the kernels take (224 + 32 = 256); tensor-core head geometry
ZC = {
    "architecture": "Zurolorn", "vocab": 300, "width": 192, "embedding": {"scale": 8.0}, "norm": {"eps": 1e-6}, "logit_scale": 0.125,
    "layers": [
        layer("latent_attention", mixer("latent_attention", 8, 64, 32, 64, 96, 300000.0), moe(12, 4, 72, 1.25, groups=(4, 3))),
        layer("latent_attention_2", mixer("latent_attention_2", 4, 96, 32, 80, 224, 12345.0, q_rank=160), moe(4, 2, 128, 3.0, groups=(2, 2))),
    ],
    "loop": {"start": 1, "stop": 2, "times": 1},
}

CASES = {"za": (ZA, 31), "zb": (ZB, 32), "zc": (ZC, 33)}


def tensor_shapes(cfg: dict) -> dict:
    w, v = cfg["width"], cfg["vocab"]
    shapes = {"embed": (v, w), "final.norm": (w,), "head": (v, w)}
    if cfg.get("loop"):
        shapes["loop.step"] = (cfg["loop"]["times"], w)
    for i, spec in enumerate(cfg["layers"]):
        p, m = f"l{i}.", spec["mixer"]
        H, dn, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
        shapes[p + "norm1"] = (w,)
        shapes[p + "ls1"] = (w,)
        if spec["type"] == "latent_attention_2":
            shapes[p + "mix.dq"] = (m["q_rank"], w)
            shapes[p + "mix.dq.norm"] = (m["q_rank"],)
            shapes[p + "mix.uq"] = (H * (dn + dr), m["q_rank"])
        else:
            shapes[p + "mix.q"] = (H * (dn + dr), w)
            shapes[p + "mix.g"] = (H * dv, w)
        shapes[p + "mix.dkv"] = (r + dr, w)
        shapes[p + "mix.dkv.norm"] = (r,)
        shapes[p + "mix.uk"] = (H * dn, r)
        shapes[p + "mix.uv"] = (H * dv, r)
        shapes[p + "mix.o"] = (w, H * dv)
        if spec.get("mlp"):
            shapes[p + "norm2"] = (w,)
            shapes[p + "ls2"] = (w,)
            shapes[p + "mlp.router"] = (spec["mlp"]["router"]["experts"], w)
            for e in range(spec["mlp"]["router"]["experts"]):
                shapes[p + f"mlp.e{e}.up"] = (spec["mlp"]["expert"]["ff"], w)
                shapes[p + f"mlp.e{e}.down"] = (w, spec["mlp"]["expert"]["ff"])
    return shapes


def make_weights(cfg: dict, seed: int, gain: float = 1.0) -> dict:
    """Seeded weights, every value representable in bfloat16 (so a bfloat16 engine and a float oracle start alike).

    Matrices N(0, gain / sqrt(inputs)); norm weights 1 + N(0, 0.1); layer scales and per-pass vectors spread widely so
    that leaving one out, or taking the wrong pass's row, moves the logits; routers wide enough that scores differ."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        if name.endswith(("ls1", "ls2")):
            value = rng.uniform(0.3, 1.7, shape)
        elif name == "loop.step":
            value = 0.5 * rng.standard_normal(shape)
        elif len(shape) == 1:
            value = 1.0 + 0.1 * rng.standard_normal(shape)
        elif name.endswith("router"):
            value = 3.0 / np.sqrt(shape[1]) * rng.standard_normal(shape)
        elif name == "embed":
            value = rng.standard_normal(shape) / cfg["embedding"]["scale"]
        else:
            value = gain / np.sqrt(shape[1]) * rng.standard_normal(shape)
        out[name] = torch.from_numpy(value.astype(np.float32)).to(torch.bfloat16).to(torch.float32)
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
