"""Hyper-connections: several residual streams per token instead of one.

All streams start as the embedding output.  A sub-block q of a layer reads one mixture of the streams and writes its
output back into all of them:

    u = sum_s in_q[s] x_s;   y = sub_block(norm(u));   x_t <- sum_s mix_q[s, t] x_s + out_q[t] * y   (all t at once)

and at the end the model's x is the sum of the streams.  With one stream, in = out = [1] and mix = [[1]] this is the
ordinary pre-norm layer x += sub_block(norm(x)); the arrangement runs that case with the same kernel and no tensors.

The write-back of one sub-block and the mixture + norm of the next are one kernel (`kernels.hyper_mix_norm`), so the
streams are read and written once per sub-block: a sub-block's output stays pending in the stream object, with its
mixing weights, until the next sub-block (or the final norm) asks for its input.  Streams and sums are float.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..config.spec import LayerSpec
from ..ops import kernels
from .base import ARRANGEMENTS, FEED_FORWARDS, MIXERS, NORMS, STREAMS, Part, TensorNeed, build_part, register
from .linear import as_tensor


class HyperWeights(Part):
    """The three tensors of one sub-block: `in` [S], `out` [S], `mix` [S, S] (indexed [from, to]).  params: streams;
    names (in, out, mix)."""

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        self.streams = int(spec["streams"])
        self.names = dict({"in": "in", "out": "out", "mix": "mix"}, **dict(spec.get("names", {})))
        self.read = self.write = self.mix = None

    def tensor_needs(self) -> Dict[str, TensorNeed]:
        s = self.streams
        # seeded random weights: a read-out and a write-in of about 1 / S and 1, a mixing near the identity
        return {self.names["in"]: TensorNeed((s,), role="vector", init_mean=1.0 / s, init_std=0.1 / s),
                self.names["out"]: TensorNeed((s,), role="vector", init_mean=1.0, init_std=0.1),
                self.names["mix"]: TensorNeed((s, s), role="vector", init_mean="identity", init_std=0.05)}

    def load(self, tensors):
        # applied to float streams: kept as float whatever the compute type
        self.read = tensors[self.names["in"]].float().contiguous()
        self.write = tensors[self.names["out"]].float().contiguous()
        self.mix = tensors[self.names["mix"]].float().contiguous()


@register(STREAMS, "hyper")
class HyperStream:
    """The streams of a step's tokens, float [tokens, S, hidden], and a sub-block output that is not in them yet."""

    def __init__(self, embedded: torch.Tensor, spec):
        self.n_streams = int(spec["streams"])
        self.source = embedded                     # [tokens, hidden]: every stream, until the first write-back
        self.x = torch.empty((embedded.shape[0], self.n_streams, embedded.shape[1]), dtype=torch.float32, device=embedded.device)
        self.spread = False                        # whether self.x holds the streams yet
        self.pending: Optional[torch.Tensor] = None
        self.pending_bias: Optional[torch.Tensor] = None
        self.pending_weights: Optional[HyperWeights] = None

    def read(self, weights: Optional[HyperWeights], norm, dtype: torch.dtype, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Bring the pending output into the streams and return norm(sum_s in[s] x_s) in `dtype` (`weights` None: the
        plain sum, as the final norm reads it); `rows` picks tokens, and the streams are then left as they are."""
        n = self.x.shape[0] if rows is None else rows.numel()
        h = torch.empty((n, self.x.shape[2]), dtype=dtype, device=self.x.device)
        y, w = self.pending, self.pending_weights
        kernels.hyper_mix_norm(self.x if self.spread else self.source, self.x, self.n_streams, y=y, bias=self.pending_bias,
                               mix=w.mix if (y is not None and w is not None) else None,
                               out_w=w.write if (y is not None and w is not None) else None,
                               in_w=weights.read if weights is not None else None, norm_w=norm.weight, eps=norm.eps,
                               norm_kind=norm.kind, h=h, rows=rows, store=rows is None and (y is not None or not self.spread))
        if rows is None:
            self.spread = True
            self.pending = self.pending_bias = self.pending_weights = None
        return h

    def write(self, y: torch.Tensor, weights: Optional[HyperWeights], bias: Optional[torch.Tensor] = None) -> None:
        self.pending, self.pending_weights, self.pending_bias = y, weights, bias

    def finish(self, norm, dtype: torch.dtype, rows: torch.Tensor) -> torch.Tensor:
        """The model's last step: the normed sum of the streams at the wanted rows."""
        return self.read(None, norm, dtype, rows=rows)

    def total(self) -> torch.Tensor:
        """The sum of the streams as they are now (pending output included), float [tokens, hidden]: what a probe of a
        layer's output reads.  Leaves the stream object as it was."""
        x = self.x
        if self.pending is not None or not self.spread:
            x = torch.empty_like(self.x)
            w = self.pending_weights
            kernels.hyper_mix_norm(self.x if self.spread else self.source, x, self.n_streams, y=self.pending, bias=self.pending_bias,
                                   mix=w.mix if (self.pending is not None and w is not None) else None,
                                   out_w=w.write if (self.pending is not None and w is not None) else None)
        return kernels.hyper_sum(x, torch.empty((x.shape[0], x.shape[2]), dtype=torch.float32, device=x.device))


@register(ARRANGEMENTS, "hyper_connections")
class HyperConnectionBlock:
    """Pre-norm sub-blocks over several streams (module docstring).  The feed-forward half may be absent.  The layer's
    `extras` give the sub-blocks' weights under "mixer_hyper" and "feed_forward_hyper"; without them (one stream) the
    constants are ones.  A mixer that says `defers_output_bias` leaves the bias of its output projection in
    `output_bias` for the write-back to add."""

    def __init__(self, spec: LayerSpec, dtype: torch.dtype):
        self.spec = spec
        self.dtype = dtype
        self.mixer_norm = build_part(NORMS, spec.mixer_norm, dtype, "norm")
        self.mixer = build_part(MIXERS, spec.mixer, dtype, "mixer")
        if getattr(self.mixer, "defers_output_bias", False):
            self.mixer.bias_taken_by_arrangement = True
        self.mixer_hyper = HyperWeights(spec.extras["mixer_hyper"], dtype) if "mixer_hyper" in spec.extras else None
        self.feed_forward = self.feed_forward_norm = self.feed_forward_hyper = None
        if spec.feed_forward is not None:
            self.feed_forward_norm = build_part(NORMS, spec.feed_forward_norm, dtype, "norm")
            self.feed_forward = build_part(FEED_FORWARDS, spec.feed_forward, dtype, "feed-forward")
            self.feed_forward_hyper = (HyperWeights(spec.extras["feed_forward_hyper"], dtype)
                                       if "feed_forward_hyper" in spec.extras else None)
        for norm in (self.mixer_norm, self.feed_forward_norm):
            if norm is not None and not hasattr(norm, "kind"):
                raise ValueError("the hyper-connection arrangement takes norms that name their kind (layer_norm, rms_norm)")

    def parts(self):
        slots = ("mixer_norm", "mixer", "mixer_hyper", "feed_forward_norm", "feed_forward", "feed_forward_hyper")
        return {slot: getattr(self, slot) for slot in slots if getattr(self, slot) is not None}

    def kernel_jobs(self):
        return kernels.hyper_jobs()

    def forward(self, stream: HyperStream, ctx, cache) -> None:
        h = stream.read(self.mixer_hyper, self.mixer_norm, self.dtype)
        y = self.mixer.forward(h, ctx, cache)
        bias = self.mixer.output_bias if getattr(self.mixer, "bias_taken_by_arrangement", False) else None
        stream.write(y, self.mixer_hyper, bias)
        if self.feed_forward is not None:
            h = stream.read(self.feed_forward_hyper, self.feed_forward_norm, self.dtype)
            stream.write(self.feed_forward.forward(h, ctx), self.feed_forward_hyper)
