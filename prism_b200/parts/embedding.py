"""Embedding and output-head parts (andre-fu/prism engine/executor.py:74-75,130)."""

from __future__ import annotations

from typing import Optional

from .base import Embedding, Head, ParamSpec, PartSpec, WeightSource, build_part, register_part
from .. import ops


@register_part("embedding", "token")
class TokenEmbedding(Embedding):
    """Row gather, times ``scale`` (in float32; 1: no scaling); the output is the
    float32 residual stream.  ``tensor``: the table's name in the model file.  ``norm``: a norm part applied to
    the gathered rows (in float32, in place)."""

    def __init__(self, vocab_size: int, hidden_size: int, scale: float = 1.0, tensor: str = "embed_tokens.weight",
                 norm: Optional[PartSpec] = None):
        self.vocab_size = int(vocab_size)
        self.hidden_size = int(hidden_size)
        self.scale = float(scale)
        self.tensor = tensor
        self.norm = self.add_child("norm", build_part("norm", norm)) if norm is not None else None

    def params(self):
        return [ParamSpec("weight", (WeightSource(self.tensor, (self.vocab_size, self.hidden_size)),))]

    def forward(self, ctx):
        out = ctx.alloc((ctx.T, self.hidden_size), ops.torch.float32)
        ops.embed(ctx.token_ids, self.w["weight"], out, ctx.err, self.scale)
        if self.norm is not None:
            # in place on the float32 rows; the same launch leaves their copy in the compute dtype for the first
            # block's matrix products (a block that norms after the sum looks for it under this key)
            h = self.norm.forward_post(ctx, out, None, 1.0)
            ctx.scratch["postnorm_rows"], ctx.scratch["postnorm_rows_of"] = h, out
        return out


@register_part("head", "linear")
class LinearHead(Head):
    """``logits = h @ W^T`` in float32, no bias, soft-cap or scale.  ``tied_to``
    names the parameter whose storage is shared when the model file has no
    head tensor (engine/weight_manager.py:84-86; the reference copies into a
    second buffer, engine/weight_pool.py:157-160: here it is one buffer)."""

    def __init__(self, vocab_size: int, hidden_size: int, tied_to: str = None, tensor: str = "weight"):
        self.vocab_size = int(vocab_size)
        self.hidden_size = int(hidden_size)
        self.tied_to = tied_to
        self.tensor = tensor

    def params(self):
        return [ParamSpec("weight", (WeightSource(self.tensor, (self.vocab_size, self.hidden_size)),),
                          optional=self.tied_to is not None, absent="none", alias_of=self.tied_to)]

    def forward(self, ctx, normed_rows):
        return ops.linear(normed_rows, self.w["weight"], None, out_dtype=ops.torch.float32)
