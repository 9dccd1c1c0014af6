"""Token embedding and the output head.

Parity: runtime/model.py:105 (lookup, no scaling) and runtime/model.py:120 (logits =
norm(x) @ head^T, no bias, no scaling); a tied head is the embedding table itself
(runtime/checkpoint.py:38-39), held once.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..ops import kernels
from .base import EMBEDDINGS, HEADS, Embedding, Head, Part, TensorNeed, register
from .linear import linear


@register(EMBEDDINGS, "token_embedding")
class TokenEmbedding(Embedding):
    """params: vocab_size, hidden_size; scale (the looked-up row is multiplied by it, default 1); weight_name."""

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        self.vocab = int(spec["vocab_size"])
        self.hidden = int(spec["hidden_size"])
        self.scale = float(spec.get("scale", 1.0))
        self.weight_name = spec.get("weight_name", "weight")
        self.table = None

    def tensor_needs(self) -> Dict[str, TensorNeed]:
        return {self.weight_name: TensorNeed((self.vocab, self.hidden))}

    def load(self, tensors):
        self.table = tensors[self.weight_name]

    def kernel_jobs(self):
        return [("elementwise.cu", {}, ())]

    def forward(self, token_ids):
        out = torch.empty((token_ids.numel(), self.hidden), dtype=torch.float32, device=token_ids.device)
        return kernels.embedding(self.table, token_ids, out, self.scale)


@register(HEADS, "linear_head")
class LinearHead(Head):
    """params: vocab_size, hidden_size, tied_to (full name of the tensor to share, or None); scale (the logits are
    multiplied by it, default 1); weight_name."""

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        self.vocab = int(spec["vocab_size"])
        self.hidden = int(spec["hidden_size"])
        self.tied_to = spec.get("tied_to")
        self.scale = float(spec.get("scale", 1.0))
        self.weight_name = spec.get("weight_name", "weight")
        self.weight = None

    def tensor_needs(self) -> Dict[str, TensorNeed]:
        return {self.weight_name: TensorNeed((self.vocab, self.hidden), alias=self.tied_to)}

    def load(self, tensors):
        self.weight = tensors[self.weight_name]

    def kernel_jobs(self):
        return kernels.gemm_jobs(self.dtype) + (kernels.skinny_jobs() if self.dtype == torch.bfloat16 else [])

    def forward(self, h):
        logits = linear(h, self.weight)
        return logits if self.scale == 1.0 else kernels.scale_(logits, self.scale)


@register(EMBEDDINGS, "pass_vectors")
class PassVectors(Part):
    """Vectors added to the residual stream at marked places of the run list: row t before pass t of a group of layers
    that runs several times with the same weights.  params: count, hidden_size; weight_name."""

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        self.count = int(spec["count"])
        self.hidden = int(spec["hidden_size"])
        self.weight_name = spec.get("weight_name", "weight")
        self.rows = None

    def tensor_needs(self) -> Dict[str, TensorNeed]:
        return {self.weight_name: TensorNeed((self.count, self.hidden), role="vector")}

    def load(self, tensors):
        self.rows = tensors[self.weight_name].float().contiguous()     # the stream is float: the add is made there

    def kernel_jobs(self):
        return [("elementwise.cu", {}, ())]

    def add_to(self, stream, index: int) -> None:
        """stream.x += (pending output, scaled) + row `index`, in one pass; nothing stays pending."""
        scale = getattr(stream, "pending_scale", None)
        kernels.stream_add(stream.x, stream.take_pending(), scale, self.rows[index])
