"""Typed configuration of Zurolorn, a decoder whose layers pair a latent-attention mixer with routed experts.

config.json of this design, key by key:

    architecture        "Zurolorn"
    vocab, width        sizes of the token table and of the residual stream
    embedding.scale     the looked-up row is multiplied by it
    norm.eps            eps of every RMS norm of the model (layer norms, latent norms, final norm)
    layers[i]           type: "latent_attention" (queries straight from the input, split-half rotation pairs, sigmoid
                        output gate) or "latent_attention_2" (queries through a normed latent of q_rank, interleaved
                        pairs, no gate); mixer: heads, dim (unrotated query/key width per head), rot_dim (rotated
                        width), vdim, kv_rank, q_rank, rot.base, rot.dims, scale; mlp: null, or kind "moe" with
                        expert.ff and router.experts / top / scale / groups.count / groups.keep
    loop                layers start .. stop - 1 run `times` times in a row with the same weights (each pass with a cache
                        of its own); row t of tensor loop.step is added to the stream right before pass t
    logit_scale         the head's output is multiplied by it
    max_positions       optional: longest sequence the block tables are made for

Tensor names: embed, loop.step, l<i>.norm1 / norm2 / ls1 / ls2, l<i>.mix.*, l<i>.mlp.router, l<i>.mlp.e<j>.up / down,
final.norm, head.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from .errors import ConfigError
from .registry import register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, RunEntry

MIXER_TYPES = {
    # type -> (queries through a latent, rotation pairs interleaved, output gate)
    "latent_attention": (False, False, True),
    "latent_attention_2": (True, True, False),
}
DEFAULT_MAX_POSITIONS = 1 << 17
CACHE_ROW_STEP, CACHE_ROW_MAX = 16, 256     # the attention kernels take rows that are multiples of 16 up to 256


def _need(mapping: Mapping[str, Any], key: str, where: str):
    if not isinstance(mapping, Mapping) or key not in mapping:
        raise ConfigError(f"config.json lacks {where}{key}")
    return mapping[key]


@dataclass(frozen=True)
class ZurolornConfig:
    raw: Mapping[str, Any]

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "ZurolornConfig":
        config = cls(dict(raw))
        config.to_spec()          # every refusal is raised here, before any weight is read
        return config

    def to_dict(self) -> dict:
        return dict(self.raw)

    # ---------------------------------------------------------------- the parts of a layer
    def _mixer(self, layer: Mapping[str, Any], where: str, width: int, eps: float) -> PartSpec:
        kind = _need(layer, "type", where)
        if kind not in MIXER_TYPES:
            raise ConfigError(f"{where}type {kind!r} is not a mixer of this design; known: {', '.join(sorted(MIXER_TYPES))}")
        latent_queries, interleaved, gate = MIXER_TYPES[kind]
        m = _need(layer, "mixer", where)
        at = where + "mixer."
        heads, dim, rot_dim = int(_need(m, "heads", at)), int(_need(m, "dim", at)), int(_need(m, "rot_dim", at))
        vdim, kv_rank = int(_need(m, "vdim", at)), int(_need(m, "kv_rank", at))
        rot = _need(m, "rot", at)
        rot_dims, base = int(_need(rot, "dims", at + "rot.")), float(_need(rot, "base", at + "rot."))
        if min(heads, dim, rot_dim, vdim, kv_rank) <= 0 or not base > 0:
            raise ConfigError(f"{at}: sizes and the rotation base must be positive")
        if rot_dims != rot_dim or rot_dim % 2:
            raise ConfigError(f"{at}rot.dims must equal rot_dim and be even")
        q_rank = int(_need(m, "q_rank", at)) if latent_queries else 0
        if latent_queries and q_rank <= 0:
            raise ConfigError(f"{at}q_rank must be positive")
        row = -(-(kv_rank + rot_dim) // CACHE_ROW_STEP) * CACHE_ROW_STEP
        if row > CACHE_ROW_MAX:
            raise ConfigError(f"{at}kv_rank + rot_dim = {kv_rank + rot_dim} is not supported: the attention kernels take cache rows "
                              f"up to {CACHE_ROW_MAX} wide")
        position = PartSpec("rotary_interleaved" if interleaved else "rotary_half", {"theta": base, "dim": rot_dim})
        return PartSpec("latent_attention", {
            "hidden_size": width, "num_heads": heads, "plain_dim": dim, "rot_dim": rot_dim, "value_dim": vdim, "kv_rank": kv_rank,
            "q_rank": q_rank, "gate": gate, "position": position, "scale": float(_need(m, "scale", at)), "eps": eps,
            "names": {"q": "q", "q_down": "dq", "q_norm": "dq.norm", "q_up": "uq", "kv_down": "dkv", "kv_norm": "dkv.norm",
                      "k_up": "uk", "v_up": "uv", "gate": "g", "out": "o"}})

    def _feed_forward(self, layer: Mapping[str, Any], where: str, width: int):
        mlp = layer.get("mlp")
        if mlp is None:
            return None
        at = where + "mlp."
        if _need(mlp, "kind", at) != "moe":
            raise ConfigError(f"{at}kind {mlp['kind']!r} is not a feed-forward of this design (moe only)")
        router = _need(mlp, "router", at)
        experts, top = int(_need(router, "experts", at + "router.")), int(_need(router, "top", at + "router."))
        ff = int(_need(_need(mlp, "expert", at), "ff", at + "expert."))
        groups = router.get("groups")
        count, keep = (int(_need(groups, "count", at + "router.groups.")), int(_need(groups, "keep", at + "router.groups."))) if groups else (0, 0)
        if min(experts, top, ff) <= 0 or top > experts:
            raise ConfigError(f"{at}: experts, top and ff must be positive and top at most experts")
        if groups and (count <= 0 or experts % count or not 0 < keep <= count or keep * (experts // count) < top):
            raise ConfigError(f"{at}router.groups: count must divide experts, and the kept groups must hold at least top experts")
        return PartSpec("routed_experts", {
            "hidden_size": width, "expert_size": ff, "experts": experts, "top": top, "groups": count, "keep": keep,
            "route_scale": float(_need(router, "scale", at + "router.")), "activation": "relu_squared",
            "names": {"router": "router", "up": "e{}.up", "down": "e{}.down"}})

    # ---------------------------------------------------------------- the model
    def run_list(self, n_layers: int):
        loop = self.raw.get("loop")
        if not loop:
            return tuple(RunEntry(layer=i) for i in range(n_layers)), 0
        start, stop, times = int(_need(loop, "start", "loop.")), int(_need(loop, "stop", "loop.")), int(_need(loop, "times", "loop."))
        if not 0 <= start <= stop <= n_layers or times < 1:
            raise ConfigError("loop: need 0 <= start <= stop <= number of layers and times >= 1")
        run = [RunEntry(layer=i) for i in range(start)]
        for t in range(times):
            for i in range(start, stop):
                run.append(RunEntry(layer=i, pass_step=t if i == start else None))
        run += [RunEntry(layer=i) for i in range(stop, n_layers)]
        return tuple(run), times

    def to_spec(self) -> ModelSpec:
        raw = self.raw
        if raw.get("architecture") != "Zurolorn":
            raise ConfigError(f"architecture {raw.get('architecture')!r} is not Zurolorn")
        vocab, width = int(_need(raw, "vocab", "")), int(_need(raw, "width", ""))
        eps = float(_need(_need(raw, "norm", ""), "eps", "norm."))
        if vocab <= 0 or width <= 0 or not eps > 0:
            raise ConfigError("vocab, width and norm.eps must be positive")
        layer_list = _need(raw, "layers", "")
        if not layer_list:
            raise ConfigError("a model needs at least one layer")
        norm = PartSpec("rms_norm", {"size": width, "eps": eps, "weight_name": ""})
        scale = PartSpec("channel_scale", {"size": width})
        names = {"mixer": "mix.", "mixer_norm": "norm1", "feed_forward": "mlp.", "feed_forward_norm": "norm2",
                 "mixer_scale": "ls1", "feed_forward_scale": "ls2"}
        layers = []
        for i, layer in enumerate(layer_list):
            where = f"layers[{i}]."
            ffn = self._feed_forward(layer, where, width)
            extras = {"mixer_scale": scale} | ({"feed_forward_scale": scale} if ffn is not None else {})
            layers.append(LayerSpec(prefix=f"l{i}.", mixer=self._mixer(layer, where, width, eps), mixer_norm=norm, feed_forward=ffn,
                                    feed_forward_norm=norm if ffn is not None else None, arrangement="pre_norm_scaled",
                                    names=names, extras=extras))
        run, times = self.run_list(len(layers))
        spec = ModelSpec(
            hidden_size=width, vocab_size=vocab, max_positions=int(raw.get("max_positions", DEFAULT_MAX_POSITIONS)),
            embedding=PartSpec("token_embedding", {"vocab_size": vocab, "hidden_size": width, "weight_name": "",
                                                   "scale": float(_need(_need(raw, "embedding", ""), "scale", "embedding."))}),
            embedding_prefix="embed", layers=tuple(layers), run=run, final_norm=norm, final_norm_prefix="final.norm",
            head=PartSpec("linear_head", {"vocab_size": vocab, "hidden_size": width, "tied_to": None, "weight_name": "",
                                          "scale": float(_need(raw, "logit_scale", ""))}),
            head_prefix="head",
            pass_steps=PartSpec("pass_vectors", {"count": times, "hidden_size": width, "weight_name": ""}) if times else None,
            pass_steps_prefix="loop.step")
        spec.validate()
        return spec


register_architecture("Zurolorn", ZurolornConfig)
