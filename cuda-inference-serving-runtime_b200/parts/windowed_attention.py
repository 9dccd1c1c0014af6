"""Grouped-query attention with the options the plain mixer (`gqa_attention`) does not have: biases on the projections,
key and value heads of different widths, values that are the keys as projected, a norm over a whole projection, a
window of keys, a sink in the softmax, rotation of part of each head.

    q = W_q h (+ b_q), k = W_k h (+ b_k), v = W_v h (+ b_v)        or v = k as projected (no W_v; value_dim = key_dim)
    qk_norm "whole": q <- q / sqrt(mean(q^2) + eps) * w_q with the mean over ALL heads of the token at once; k likewise
    rotation of the first `position.dim` coordinates of each head of q and k
    score = (q . k) * scale over the keys j with 0 <= i - j (< window)
    p_j = exp(s_j) / (sum exp(s) [+ exp(sink)]);  out = W_o [heads of sum_j p_j v_j] (+ b_o)

The paged attention kernels take one head width D for queries, keys and values: D = max(key_dim, value_dim) rounded up
to 16, heads are padded with zeros on their way into q and the cache (`kernels.attention_rows`), and the columns of W_o
that would meet the padding are zero.  Keys are cached rotated (and normed), values as they are.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..config.spec import CacheUse
from ..ops import kernels
from .attention import ATTENTION_PLAN_KEY, attention_step_plan, paged_attention
from .base import MIXERS, POSITIONS, Mixer, TensorNeed, build_part, register
from .linear import as_tensor, linear

DEFAULT_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b", "o_bias": "o.b",
                 "q_norm": "q.norm", "k_norm": "k.norm"}
HEAD_STEP, HEAD_MAX = 16, 256      # the attention kernels are built per head width: multiples of 16 up to 256


@register(MIXERS, "windowed_attention")
class WindowedAttention(Mixer):
    """params: hidden_size, num_heads, num_kv_heads, key_dim, value_dim, position (PartSpec), scale, window (None or int),
    sink (None, or the score of the sink), qk_norm (None or "whole"), eps (of that norm), values_from_keys (bool),
    bias (the set of projections that have one, among "q", "k", "v", "o"), names."""

    graph_safe = True
    # An arrangement that adds the mixer's output to the stream in a kernel of its own may add `output_bias` there: it sets
    # `bias_taken_by_arrangement` when it is built.  Otherwise the mixer adds the bias itself.
    defers_output_bias = True

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        self.hidden = int(spec["hidden_size"])
        self.hq, self.hkv = int(spec["num_heads"]), int(spec["num_kv_heads"])
        self.key_dim, self.value_dim = int(spec["key_dim"]), int(spec["value_dim"])
        self.scale = float(spec["scale"])
        self.window = spec.get("window")
        self.sink = spec.get("sink")
        self.qk_norm = spec.get("qk_norm")
        self.eps = float(spec.get("eps", 0.0))
        self.values_from_keys = bool(spec.get("values_from_keys", False))
        self.bias = frozenset(spec.get("bias", ()))
        self.names = {**DEFAULT_NAMES, **dict(spec.get("names") or {})}
        if self.hq % self.hkv:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if self.qk_norm not in (None, "whole"):
            raise ValueError(f"unknown qk_norm {self.qk_norm!r}")
        if self.values_from_keys and (self.value_dim != self.key_dim or "v" in self.bias):
            raise ValueError("values taken from the keys have the keys' width and no projection of their own")
        self.width = -(-max(self.key_dim, self.value_dim) // HEAD_STEP) * HEAD_STEP
        if self.width > HEAD_MAX:
            raise ValueError(f"heads of {max(self.key_dim, self.value_dim)} are not supported: the attention kernels take up to {HEAD_MAX}")
        self.position = build_part(POSITIONS, spec["position"], dtype, "position encoding")
        if getattr(self.position, "dim", 0) > self.key_dim:
            raise ValueError("the position encoding turns more coordinates than a key head has")
        self.w_in = self.o = self.in_bias = self.output_bias = self.q_norm = self.k_norm = None
        self.bias_taken_by_arrangement = False

    # ---------------------------------------------------------------- tensors
    def tensor_needs(self) -> Dict[str, TensorNeed]:
        n = self.names
        nq, nk, nv = self.hq * self.key_dim, self.hkv * self.key_dim, self.hkv * self.value_dim
        needs = {n["q"]: TensorNeed((nq, self.hidden)), n["k"]: TensorNeed((nk, self.hidden)),
                 n["o"]: TensorNeed((self.hidden, self.hq * self.value_dim))}
        if not self.values_from_keys:
            needs[n["v"]] = TensorNeed((nv, self.hidden))
        for which, size in (("q", nq), ("k", nk), ("v", nv), ("o", self.hidden)):
            if which in self.bias:
                needs[n[which + "_bias"]] = TensorNeed((size,), role="vector", init_mean=0.0)
        if self.qk_norm:
            needs[n["q_norm"]] = TensorNeed((nq,), role="vector")
            needs[n["k_norm"]] = TensorNeed((nk,), role="vector")
        return needs

    def load(self, tensors):
        n = self.names
        stacked = [tensors[n["q"]], tensors[n["k"]]] + ([] if self.values_from_keys else [tensors[n["v"]]])
        self.w_in = torch.cat(stacked, dim=0).contiguous()
        self.k_col = stacked[0].shape[0]
        self.v_col = -1 if self.values_from_keys else self.k_col + stacked[1].shape[0]
        if self.bias & {"q", "k", "v"}:
            pieces = [tensors[n[w + "_bias"]].float() if w in self.bias else torch.zeros(m.shape[0], device=m.device)
                      for w, m in zip("qkv", stacked)]
            self.in_bias = torch.cat(pieces).contiguous()
        self.output_bias = tensors[n["o_bias"]].float().contiguous() if "o" in self.bias else None
        if self.qk_norm:
            self.q_norm = tensors[n["q_norm"]].float().contiguous()
            self.k_norm = tensors[n["k_norm"]].float().contiguous()
        o = tensors[n["o"]]
        if self.width != self.value_dim:      # zero columns where the attention's output rows are padding
            wide = torch.zeros((self.hidden, self.hq, self.width), dtype=o.dtype, device=o.device)
            wide[:, :, :self.value_dim] = o.view(self.hidden, self.hq, self.value_dim)
            o = wide.view(self.hidden, self.hq * self.width)
        self.o = o.contiguous()

    def kernel_jobs(self):
        return ([kernels.attention_jobs(self.width, self.dtype)] + kernels.attention_rows_jobs()
                + kernels.attention_tcgen05_jobs(self.width, self.dtype) + kernels.gemm_jobs(self.dtype) + self.position.kernel_jobs()
                + (kernels.skinny_jobs() if self.dtype == torch.bfloat16 else []))

    def cache_use(self) -> CacheUse:
        return CacheUse("pages", kv_heads=self.hkv, head_dim=self.width, window=self.window)

    # ---------------------------------------------------------------- the step
    def plan_key(self):
        return ATTENTION_PLAN_KEY

    def step_plan(self, host):
        return attention_step_plan(host)

    def begin_step(self, ctx) -> None:
        self.position.rotation(ctx)

    def forward(self, h, ctx, cache):
        if not cache.write:
            raise NotImplementedError("windowed_attention writes its own keys and values")
        tokens = ctx.n_tokens
        rot = self.position.rotation(ctx)
        proj = linear(as_tensor(h), self.w_in)                      # float [tokens, q | k (| v)]
        q = torch.empty((tokens, self.hq, self.width), dtype=self.dtype, device=ctx.device)
        kernels.attention_rows(proj, self.k_col, self.v_col, bias=self.in_bias, q_norm=self.q_norm, k_norm=self.k_norm, eps=self.eps,
                               cos=rot.cos if rot else None, sin=rot.sin if rot else None, rot_half=rot.rot_half if rot else 0,
                               interleaved=rot.interleaved if rot else False, q_out=q, k_cache=cache.k, v_cache=cache.v,
                               token_req=ctx.token_req, positions=ctx.positions, req_slot=ctx.req_slot,
                               block_table=cache.block_table, page_size=cache.page_size, hq=self.hq, hkv=self.hkv,
                               key_dim=self.key_dim, value_dim=self.value_dim)
        mixed = paged_attention(ctx.plan_for(self), q, cache.k, cache.v, cache, ctx, self.hq, self.hkv, self.scale, self.window,
                                sink=self.sink)
        y = linear(mixed.view(tokens, self.hq * self.width), self.o)
        if self.output_bias is not None and not self.bias_taken_by_arrangement:
            kernels.bias_add(y, self.output_bias)
        return y
