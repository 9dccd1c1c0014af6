"""Routed experts: many small feed-forward layers of which each token uses a few.

    scores    s = sigmoid(W_router h): float sums (one of the engine's matrix products), float sigmoid
    groups    the experts form `groups` equal groups of neighbours; a group's score is the sum of its two best members;
              only members of the `keep` best groups can be chosen (groups 0: every expert can)
    choice    the `top` best open experts, each weighted by s * route_scale (not renormalised)
    expert    W_down act(W_up h), no biases; act(z) = max(z, 0)^2 ("relu_squared")
    output    the weighted sum of the chosen experts' outputs

The experts' matrices are stacked at load ([experts, ff, hidden] and [experts, hidden, ff]) so one launch serves
whichever experts a step's tokens chose.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..ops import kernels
from .base import FEED_FORWARDS, FeedForward, TensorNeed, register
from .linear import linear

ACTIVATIONS = ("relu_squared",)
DEFAULT_NAMES = {"router": "router.weight", "up": "experts.{}.up.weight", "down": "experts.{}.down.weight"}


@register(FEED_FORWARDS, "routed_experts")
class RoutedExperts(FeedForward):
    """params: hidden_size, expert_size, experts, top, groups, keep, route_scale, activation, names (local tensor names:
    router, and up / down with {} for the expert's number)."""

    applies_output_scale = True      # forward(h, ctx, out_scale): a per-channel layer scale is the epilogue of the last kernel

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        self.hidden = int(spec["hidden_size"])
        self.ff = int(spec["expert_size"])
        self.experts = int(spec["experts"])
        self.top = int(spec["top"])
        self.groups = int(spec.get("groups") or 0)
        self.keep = int(spec.get("keep") or 0)
        self.route_scale = float(spec.get("route_scale", 1.0))
        self.activation = spec.get("activation", "relu_squared")
        self.names = {**DEFAULT_NAMES, **dict(spec.get("names") or {})}
        if self.activation not in ACTIVATIONS:
            raise ValueError(f"expert activation {self.activation!r} is not implemented; known: {', '.join(ACTIVATIONS)}")
        if not 0 < self.top <= self.experts:
            raise ValueError("top must lie between 1 and the number of experts")
        if self.groups and (self.experts % self.groups or not 0 < self.keep <= self.groups
                            or self.keep * (self.experts // self.groups) < self.top):
            raise ValueError("groups must divide the experts, and the kept groups must hold at least top experts")
        self.router = self.up = self.down = None

    def tensor_needs(self) -> Dict[str, TensorNeed]:
        # seeded random routers are drawn wide enough that a token's scores differ clearly
        needs = {self.names["router"]: TensorNeed((self.experts, self.hidden), init_std=4.0 / self.hidden ** 0.5)}
        for e in range(self.experts):
            needs[self.names["up"].format(e)] = TensorNeed((self.ff, self.hidden))
            needs[self.names["down"].format(e)] = TensorNeed((self.hidden, self.ff))
        return needs

    def load(self, tensors):
        self.router = tensors[self.names["router"]].contiguous()
        self.up = torch.stack([tensors[self.names["up"].format(e)] for e in range(self.experts)]).contiguous()
        self.down = torch.stack([tensors[self.names["down"].format(e)] for e in range(self.experts)]).contiguous()

    def kernel_jobs(self):
        return kernels.moe_jobs() + kernels.gemm_jobs(self.dtype) + (kernels.skinny_jobs() if self.dtype == torch.bfloat16 else [])

    def route(self, h: torch.Tensor):
        """(chosen experts int32 [tokens, top], best first; their weights float [tokens, top])."""
        tokens = h.shape[0]
        chosen = torch.empty((tokens, self.top), dtype=torch.int32, device=h.device)
        weight = torch.empty((tokens, self.top), dtype=torch.float32, device=h.device)
        logits = linear(h, self.router)          # float sums, by the engine's products for this many tokens
        kernels.moe_select(logits, self.top, self.groups, self.keep, self.route_scale, chosen, weight)
        return chosen, weight

    def forward(self, h, ctx, out_scale=None):
        tokens = h.shape[0]
        chosen, weight = self.route(h)
        out = torch.empty((tokens, self.hidden), dtype=torch.float32, device=h.device)
        if kernels.moe_grouped_ok(h, self.up, self.top):
            return kernels.moe_grouped(h, self.up, self.down, chosen, weight, out, out_scale)     # many tokens: sorted by expert, tcgen05
        act = torch.empty((tokens * self.top, self.ff), dtype=self.dtype, device=h.device)
        return kernels.moe_rows(h, self.up, self.down, chosen, weight, act, out, out_scale)
