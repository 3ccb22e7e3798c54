"""Token embedding and output head."""
from __future__ import annotations

from typing import List, Optional

import torch

from ..config import register_part
from ..csrc import ops
from ..weights import WeightSpec
from . import linear as L
from .base import Part


EMBEDDING_OUTPUT = "embedding output in the compute dtype"          # ctx.memo key


class TokenEmbedding(Part):
    """``h[t, :] = table[id_t, :]`` into the float32 residual stream (src/ops/embedding.cu:9-18).
    An id outside the vocabulary is an error, not a clamp to 0 as in the reference.  ``scale`` multiplies the rows;
    ``keep_output`` leaves a copy of the result in the compute dtype in ``ctx.memo[EMBEDDING_OUTPUT]`` for parts that
    read the embedding again after layers have changed the stream."""

    graph_safe = True

    role = "embedding"

    def __init__(self, prefix: str, vocab_size: int, hidden_size: int, weight_name: str = "weight", scale: float = 1.0,
                 keep_output: bool = False):
        self.name = f"{prefix}.{weight_name}" if prefix else weight_name
        self.vocab_size, self.hidden_size = vocab_size, hidden_size
        self.scale, self.keep_output = float(scale), bool(keep_output)
        self.table = None

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.name, (self.vocab_size, self.hidden_size))]

    def bind(self, tensors, dtype, device) -> None:
        self.table = tensors[self.name]

    def forward(self, token_ids, ctx=None):
        out = torch.empty((token_ids.numel(), self.hidden_size), dtype=torch.float32, device=token_ids.device)
        copy = None
        if self.keep_output and ctx is not None:
            copy = torch.empty(out.shape, dtype=self.table.dtype, device=out.device)
        ops.embedding(token_ids, self.table, out, None if ctx is None else ctx.err, scale=self.scale, copy=copy)
        if copy is not None:
            if copy.dtype != ctx.dtype:          # a table stored in another precision than the activations
                kept = torch.empty(out.shape, dtype=ctx.dtype, device=out.device)
                ops.cast_add(out, kept)
                copy = kept
            ctx.memo[EMBEDDING_OUTPUT] = copy
        return out


class LMHead(Part):
    """``logits = x @ W^T`` in float32.  ``weight_name`` is the head's own matrix, or the
    embedding table's name when the two are tied (the reference always uses the table,
    src/engine/engine_server.cpp:1968,2042, whatever ``tie_word_embeddings`` says).  ``softcap`` (a positive number):
    ``logits <- softcap * tanh(logits / softcap)``."""

    graph_safe = True

    role = "head"

    def __init__(self, prefix: str, vocab_size: int, hidden_size: int, weight_name: str = "weight",
                 softcap: Optional[float] = None):
        if softcap is not None and not softcap > 0:
            raise ValueError(f"a soft cap on the logits must be positive, got {softcap}")
        self.name = f"{prefix}.{weight_name}" if prefix else weight_name
        self.vocab_size, self.hidden_size = vocab_size, hidden_size
        self.softcap = float(softcap) if softcap is not None else None
        self.weight = None

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.name, (self.vocab_size, self.hidden_size))]

    def bind(self, tensors, dtype, device) -> None:
        self.weight = tensors[self.name]

    def forward(self, x, ctx=None):
        # The norm is not folded into this contraction: with a vocabulary's worth of blocks, each would
        # repeat the norm of every row.
        logits = L.linear(x, self.weight, None, L.STORE_F32)
        if self.softcap is not None:
            ops.softcap(logits, self.softcap)
        return logits


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("head", "lm_head", LMHead)
