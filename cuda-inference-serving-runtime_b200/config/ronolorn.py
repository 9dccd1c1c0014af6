"""Typed configuration of Ronolorn, a decoder whose layers mix windowed attention and a gated delta rule over several
residual streams.

config.json of this design, key by key:

    architecture        "Ronolorn"
    vocab, width        sizes of the token table and of the residual stream
    embedding.scale     the looked-up row is multiplied by it
    norm.eps            eps of every layer norm of the model, of the whole-projection query/key norm and of the delta
                        rule's output norm
    streams             optional: how many residual streams a token carries (hyper-connections, tensors l<i>.hc1.* for
                        the mixer and l<i>.hc2.* for the feed-forward); absent: one stream, the plain residual sum
    layers[i]           type: "attention" (biases on q, k, v and o; ordinary softmax), "attention_2" (biases on q and k;
                        the values are the keys as projected; q and k normed over their whole projection; a sink of
                        score 0 in the softmax) or "delta" (gated delta rule);
                        mixer: heads, kv_heads, dim, vdim; for attention also scale, rot.base, rot.dims (interleaved
                        pairs over the first rot.dims coordinates of each head), rot.scaling (factor, original, fast,
                        slow; optional), mask.size (a window of keys; optional); for delta also conv (taps);
                        mlp: null, or kind "dense" with ff (up, squared relu, down)
    max_positions       optional: longest sequence the block tables are made for

Tensor names: embed (also the output head, without the scale), l<i>.norm1 / norm2, l<i>.mix.*, l<i>.mlp.up / down,
l<i>.hc1.* / hc2.*, final.norm.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from .errors import ConfigError
from .registry import register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec

ATTENTION_TYPES = {
    # type -> (projections with a bias, values are the keys, norm over the whole projection, sink score or None)
    "attention": (("q", "k", "v", "o"), False, None, None),
    "attention_2": (("q", "k"), True, "whole", 0.0),
}
DEFAULT_MAX_POSITIONS = 1 << 17
MAX_STREAMS = 16


def _need(mapping: Mapping[str, Any], key: str, where: str):
    if not isinstance(mapping, Mapping) or key not in mapping:
        raise ConfigError(f"config.json lacks {where}{key}")
    return mapping[key]


@dataclass(frozen=True)
class RonolornConfig:
    raw: Mapping[str, Any]

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "RonolornConfig":
        config = cls(dict(raw))
        config.to_spec()          # every refusal is raised here, before any weight is read
        return config

    def to_dict(self) -> dict:
        return dict(self.raw)

    # ---------------------------------------------------------------- the parts of a layer
    @staticmethod
    def _position(m: Mapping[str, Any], at: str, dim: int) -> PartSpec:
        rot = m.get("rot")
        if not rot:
            return PartSpec("none", {})
        dims, base = int(_need(rot, "dims", at + "rot.")), float(_need(rot, "base", at + "rot."))
        if dims % 2 or not 0 < dims <= dim or not base > 1:
            raise ConfigError(f"{at}rot: dims must be even and at most dim, base above 1")
        params = {"theta": base, "dim": dims}
        scaling = rot.get("scaling")
        if scaling:
            sat = at + "rot.scaling."
            params["scaling"] = {"kind": "yarn", "factor": float(_need(scaling, "factor", sat)), "original": float(_need(scaling, "original", sat)),
                                 "fast": float(_need(scaling, "fast", sat)), "slow": float(_need(scaling, "slow", sat))}
            if not (params["scaling"]["factor"] > 0 and params["scaling"]["original"] > 0 and params["scaling"]["fast"] > 0
                    and params["scaling"]["slow"] > 0):
                raise ConfigError(f"{sat}: factor, original, fast and slow must be positive")
        return PartSpec("rotary_interleaved", params)

    def _mixer(self, layer: Mapping[str, Any], where: str, width: int, eps: float) -> PartSpec:
        kind = _need(layer, "type", where)
        m = _need(layer, "mixer", where)
        at = where + "mixer."
        heads, kv_heads = int(_need(m, "heads", at)), int(_need(m, "kv_heads", at))
        dim, vdim = int(_need(m, "dim", at)), int(_need(m, "vdim", at))
        if min(heads, kv_heads, dim, vdim) <= 0 or heads % kv_heads:
            raise ConfigError(f"{at}: sizes must be positive and heads a multiple of kv_heads")
        if kind == "delta":
            taps = int(_need(m, "conv", at))
            if taps < 1 or dim > 256:
                raise ConfigError(f"{at}: conv must be at least 1 and dim at most 256 (the recurrence kernel's limit)")
            return PartSpec("gated_delta", {"hidden_size": width, "num_heads": heads, "num_kv_heads": kv_heads, "key_dim": dim,
                                            "value_dim": vdim, "conv": taps, "eps": eps})
        if kind not in ATTENTION_TYPES:
            raise ConfigError(f"{where}type {kind!r} is not a mixer of this design; known: delta, {', '.join(sorted(ATTENTION_TYPES))}")
        bias, from_keys, qk_norm, sink = ATTENTION_TYPES[kind]
        if from_keys and vdim != dim:
            raise ConfigError(f"{at}vdim must equal dim where the values are the keys")
        if max(dim, vdim) > 256:
            raise ConfigError(f"{at}: heads wider than 256 are not supported by the attention kernels")
        mask = m.get("mask")
        window = int(_need(mask, "size", at + "mask.")) if mask else None
        if window is not None and window < 1:
            raise ConfigError(f"{at}mask.size must be at least 1")
        return PartSpec("windowed_attention", {
            "hidden_size": width, "num_heads": heads, "num_kv_heads": kv_heads, "key_dim": dim, "value_dim": vdim,
            "position": self._position(m, at, dim), "scale": float(_need(m, "scale", at)), "window": window, "sink": sink,
            "qk_norm": qk_norm, "eps": eps, "values_from_keys": from_keys, "bias": tuple(bias)})

    @staticmethod
    def _feed_forward(layer: Mapping[str, Any], where: str, width: int):
        mlp = layer.get("mlp")
        if mlp is None:
            return None
        at = where + "mlp."
        if _need(mlp, "kind", at) != "dense":
            raise ConfigError(f"{at}kind {mlp['kind']!r} is not a feed-forward of this design (dense only)")
        ff = int(_need(mlp, "ff", at))
        if ff <= 0:
            raise ConfigError(f"{at}ff must be positive")
        return PartSpec("dense_mlp", {"hidden_size": width, "intermediate_size": ff, "activation": "relu_squared"})

    # ---------------------------------------------------------------- the model
    def to_spec(self) -> ModelSpec:
        raw = self.raw
        if raw.get("architecture") != "Ronolorn":
            raise ConfigError(f"architecture {raw.get('architecture')!r} is not Ronolorn")
        vocab, width = int(_need(raw, "vocab", "")), int(_need(raw, "width", ""))
        eps = float(_need(_need(raw, "norm", ""), "eps", "norm."))
        if vocab <= 0 or width <= 0 or not eps > 0:
            raise ConfigError("vocab, width and norm.eps must be positive")
        layer_list = _need(raw, "layers", "")
        if not layer_list:
            raise ConfigError("a model needs at least one layer")
        streams = raw.get("streams")
        if streams is not None and not 1 <= int(streams) <= MAX_STREAMS:
            raise ConfigError(f"streams must be between 1 and {MAX_STREAMS}")
        norm = PartSpec("layer_norm", {"size": width, "eps": eps, "weight_name": ""})
        names = {"mixer": "mix.", "mixer_norm": "norm1", "feed_forward": "mlp.", "feed_forward_norm": "norm2",
                 "mixer_hyper": "hc1.", "feed_forward_hyper": "hc2."}
        hyper = None if streams is None else PartSpec("hyper_weights", {"streams": int(streams)})
        layers = []
        for i, layer in enumerate(layer_list):
            where = f"layers[{i}]."
            ffn = self._feed_forward(layer, where, width)
            extras = {}
            if hyper is not None:
                extras = {"mixer_hyper": hyper} | ({"feed_forward_hyper": hyper} if ffn is not None else {})
            layers.append(LayerSpec(prefix=f"l{i}.", mixer=self._mixer(layer, where, width, eps), mixer_norm=norm, feed_forward=ffn,
                                    feed_forward_norm=norm if ffn is not None else None, arrangement="hyper_connections",
                                    names=names, extras=extras))
        from .spec import RunEntry
        spec = ModelSpec(
            hidden_size=width, vocab_size=vocab, max_positions=int(raw.get("max_positions", DEFAULT_MAX_POSITIONS)),
            embedding=PartSpec("token_embedding", {"vocab_size": vocab, "hidden_size": width, "weight_name": "",
                                                   "scale": float(_need(_need(raw, "embedding", ""), "scale", "embedding."))}),
            embedding_prefix="embed", layers=tuple(layers), run=tuple(RunEntry(layer=i) for i in range(len(layers))),
            final_norm=norm, final_norm_prefix="final.norm",
            head=PartSpec("linear_head", {"vocab_size": vocab, "hidden_size": width, "tied_to": "embed", "weight_name": ""}),
            head_prefix="head",
            stream=PartSpec("hyper", {"streams": 1 if streams is None else int(streams)}))
        spec.validate()
        return spec


register_architecture("Ronolorn", RonolornConfig)
