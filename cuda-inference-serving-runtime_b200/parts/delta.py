"""The gated delta rule: a recurrent mixer with a matrix state per head and a short convolution in front.

    q, k (kv_heads x key_dim) and v (heads x value_dim) = projections of h, each through a short causal convolution
    over time per channel (taps weights, the last the current token's, zeros before the sequence) and silu;
    q, k <- unit vectors per head (x / sqrt(sum x^2 + 1e-6)), q also times key_dim^-1/2;
    beta = sigmoid(W_b h), decay = exp(-exp(A_log) * softplus(W_a h + dt_bias)), one of each per head;
    per head (its q/k head is head // (heads / kv_heads)):  S <- decay S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
    out = W_o [heads of  o / sqrt(mean(o^2) + eps) * w_norm * silu(W_g h)]

A request's state is S for every head and the last taps - 1 inputs of the convolution, float, in one row of a state
tensor of the cache manager (`CacheUse("state", ...)`), zero when the request starts.  Portions of a prompt and single
decoded tokens run the same kernels (`kernels.delta_step`).  Short portions and single tokens walk a request's tokens in
order; portions of CHUNKED_FROM tokens and more run the chunked form of the same recurrence (csrc/delta.cu), which differs
from the walk by rounding only.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..config.spec import CacheUse
from ..ops import kernels
from .base import MIXERS, Mixer, TensorNeed, register
from .feedforward import pad_columns
from .linear import as_tensor, linear

CHUNKED_FROM = kernels.DELTA_CHUNK       # portions of at least this many tokens run chunk by chunk
DELTA_PLAN_KEY = ("delta_chunks", kernels.DELTA_CHUNK, CHUNKED_FROM)


def chunk_plan(q_len):
    """Which chunks the chunked recurrence runs for a step whose requests bring `q_len` tokens: per chunk its request and
    its first token inside the portion, per request the index of its first chunk; and how many requests stay with the
    token-by-token kernel.  Depends on the portion lengths alone, so steps of one shape share it."""
    chunk_req, chunk_t0, req_chunk0, short = [], [], [], 0
    for r, n in enumerate(q_len):
        req_chunk0.append(len(chunk_req))
        if n < CHUNKED_FROM:
            short += 1
            continue
        for t0 in range(0, n, kernels.DELTA_CHUNK):
            chunk_req.append(r)
            chunk_t0.append(t0)
    return chunk_req, chunk_t0, req_chunk0, short


DEFAULT_NAMES = {"q": "q", "k": "k", "v": "v", "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv", "beta": "b", "a": "a",
                 "a_log": "A_log", "dt_bias": "dt_bias", "gate": "g", "norm": "norm", "o": "o"}
UNIT_NORM_EPS = 1e-6


@register(MIXERS, "gated_delta")
class GatedDelta(Mixer):
    """params: hidden_size, num_heads, num_kv_heads, key_dim, value_dim, conv (taps), eps (of the output norm), names."""

    # forward reads the step through device tensors only.  A captured step's warm-up run outside the graph would advance the
    # state once too often: the graph code keeps the state tensors and puts them back after it (engine/graph.py).
    graph_safe = True

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        self.hidden = int(spec["hidden_size"])
        self.heads, self.kvh = int(spec["num_heads"]), int(spec["num_kv_heads"])
        self.key_dim, self.value_dim = int(spec["key_dim"]), int(spec["value_dim"])
        self.taps = int(spec["conv"])
        self.eps = float(spec["eps"])
        self.names = {**DEFAULT_NAMES, **dict(spec.get("names") or {})}
        if self.heads % self.kvh:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if self.key_dim > kernels.DELTA_MAX_KEY_DIM:
            raise ValueError(f"key heads of {self.key_dim} are not supported: the recurrence holds up to {kernels.DELTA_MAX_KEY_DIM} rows per column")
        if self.taps < 1:
            raise ValueError("the convolution needs at least one tap")
        self.channels = 2 * self.kvh * self.key_dim + self.heads * self.value_dim
        self.state_size = self.heads * self.key_dim * self.value_dim + (self.taps - 1) * self.channels
        self.w_in = self.conv = self.a_log = self.dt_bias = self.norm = self.o = None

    def tensor_needs(self) -> Dict[str, TensorNeed]:
        n = self.names
        nqk, nv = self.kvh * self.key_dim, self.heads * self.value_dim
        return {n["q"]: TensorNeed((nqk, self.hidden)), n["k"]: TensorNeed((nqk, self.hidden)), n["v"]: TensorNeed((nv, self.hidden)),
                n["q_conv"]: TensorNeed((nqk, self.taps), role="vector", init_mean=1.0 / self.taps, init_std=0.2),
                n["k_conv"]: TensorNeed((nqk, self.taps), role="vector", init_mean=1.0 / self.taps, init_std=0.2),
                n["v_conv"]: TensorNeed((nv, self.taps), role="vector", init_mean=1.0 / self.taps, init_std=0.2),
                n["beta"]: TensorNeed((self.heads, self.hidden)), n["a"]: TensorNeed((self.heads, self.hidden)),
                n["a_log"]: TensorNeed((self.heads,), role="vector", init_mean=-1.0, init_std=0.5),
                n["dt_bias"]: TensorNeed((self.heads,), role="vector", init_mean=0.0, init_std=0.5),
                n["gate"]: TensorNeed((nv, self.hidden)), n["norm"]: TensorNeed((self.value_dim,), role="vector"),
                n["o"]: TensorNeed((self.hidden, nv))}

    def load(self, tensors):
        n = self.names
        # one product for everything that reads h: q | k | v | gate | b | a, its rows padded to a multiple of 16
        stacked = torch.cat([tensors[n[key]] for key in ("q", "k", "v", "gate", "beta", "a")], dim=0)
        extra = -stacked.shape[0] % 16
        if extra:
            stacked = torch.cat((stacked, torch.zeros((extra, self.hidden), dtype=stacked.dtype, device=stacked.device)), dim=0)
        self.w_in = stacked.contiguous()
        # everything that enters the recurrence besides the projections is float
        self.conv = torch.cat([tensors[n[key]].float() for key in ("q_conv", "k_conv", "v_conv")], dim=0).contiguous()
        self.a_log = tensors[n["a_log"]].float().contiguous()
        self.dt_bias = tensors[n["dt_bias"]].float().contiguous()
        self.norm = tensors[n["norm"]].float().contiguous()
        self.o = pad_columns(tensors[n["o"]], 8)

    def kernel_jobs(self):
        return (kernels.delta_jobs() + kernels.gemm_jobs(self.dtype)
                + (kernels.skinny_jobs() if self.dtype == torch.bfloat16 else []))

    def cache_use(self) -> CacheUse:
        return CacheUse("state", state_shape=(self.state_size,), state_dtype="float32")

    # ---------------------------------------------------------------- the launch plan of a step
    def plan_key(self):
        return DELTA_PLAN_KEY

    def step_plan(self, host):
        import numpy as np

        from ..engine.batch import StepPlan
        chunk_req, chunk_t0, req_chunk0, short = chunk_plan(host.q_len)
        as_i32 = lambda values: np.asarray(values, dtype=np.int32)
        return StepPlan(arrays={"chunk_req": as_i32(chunk_req), "chunk_t0": as_i32(chunk_t0), "req_chunk0": as_i32(req_chunk0)},
                        info={"n_chunks": len(chunk_req), "n_short": short})

    def forward(self, h, ctx, cache):
        tokens = ctx.n_tokens
        proj = linear(as_tensor(h), self.w_in)                      # float [tokens, q | k | v | gate | b | a | padding]
        width = self.o.shape[1]
        make = torch.zeros if width != self.heads * self.value_dim else torch.empty
        out = make((tokens, width), dtype=self.dtype, device=ctx.device)
        plan = ctx.plan_for(self)
        chunks = None
        if plan.info["n_chunks"]:
            chunks = (plan["chunk_req"], plan["chunk_t0"], plan["req_chunk0"], plan.info["n_chunks"], plan.info["n_short"], CHUNKED_FROM)
        kernels.delta_step(proj, self.conv, self.taps, cache.state, self.a_log, self.dt_bias, self.norm, self.eps, UNIT_NORM_EPS,
                           ctx.token_req, ctx.req_slot, ctx.q_start, ctx.q_len, ctx.n_requests, self.heads, self.kvh, self.key_dim,
                           self.value_dim, out, chunks=chunks)
        return linear(out, self.o)
