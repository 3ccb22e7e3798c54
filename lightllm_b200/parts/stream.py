"""Parts that rewrite the residual stream between layers (role ``stream``): a run entry may name one as its ``enter``."""
from __future__ import annotations

from typing import List

import torch

from ..config import register_part
from ..csrc import ops
from ..weights import WeightSpec
from . import linear as L
from .base import Part
from .embedding import EMBEDDING_OUTPUT


class StreamReinjection(Part):
    """``h <- W [h; e] + step[index]``: the stream is mixed again with the embedding output ``e`` (kept by the embedding
    part, ``keep_output=True``) and a learned vector is added, e.g. before every pass of a looped stretch of layers.

    ``weight_name`` is ``[hidden, 2 * hidden]`` with the stream's columns first; ``step_name`` is ``[rows, hidden]`` and
    ``index`` picks the row.  Parts of several run entries may name the same tensors (one per pass).  One kernel lays
    ``[h | e]`` side by side in the compute dtype, one contraction with the step vector as its bias writes the new float
    stream, which is never rounded to the compute dtype."""

    role = "stream"
    graph_safe = True

    def __init__(self, prefix: str, hidden_size: int, weight_name: str, step_name: str, steps: int, index: int):
        if not 0 <= index < steps:
            raise ValueError(f"step vector {index} of {steps}")
        join = lambda tail: f"{prefix}.{tail}" if prefix else tail
        self.weight_name, self.step_name = join(weight_name), join(step_name)
        self.hidden_size, self.steps, self.index = hidden_size, steps, index
        self.weight = self.step = None

    def weight_specs(self) -> List[WeightSpec]:
        D = self.hidden_size
        return [WeightSpec(self.weight_name, (D, 2 * D)), WeightSpec(self.step_name, (self.steps, D), init=("normal", 0.1))]

    def bind(self, tensors, dtype, device) -> None:
        self.weight = tensors[self.weight_name]
        self.step = tensors[self.step_name][self.index].float().contiguous()

    def forward(self, residual, ctx) -> None:
        kept = ctx.memo.get(EMBEDDING_OUTPUT)
        if kept is None:
            raise ops.KernelError("stream re-injection: the embedding part did not keep its output (keep_output=True)")
        T, D = residual.shape
        both = torch.empty((T, 2 * D), dtype=ctx.dtype, device=residual.device)
        ops.cast_concat(residual, kept, both)
        L.linear(both, self.weight, self.step, L.STORE_F32, out=residual)


register_part("stream", "reinjection", StreamReinjection)


class StreamStepVector(Part):
    """``h <- h + step[index]``: a learned vector is added to every row of the stream, e.g. before every pass of a looped
    stretch of layers.  ``step_name`` is ``[steps, hidden]`` and ``index`` picks the row; the sum is float32."""

    role = "stream"
    graph_safe = True

    def __init__(self, prefix: str, hidden_size: int, step_name: str, steps: int, index: int):
        if not 0 <= index < steps:
            raise ValueError(f"step vector {index} of {steps}")
        self.step_name = f"{prefix}.{step_name}" if prefix else step_name
        self.hidden_size, self.steps, self.index = hidden_size, steps, index
        self.step = None

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.step_name, (self.steps, self.hidden_size), init=("normal", 0.1))]

    def bind(self, tensors, dtype, device) -> None:
        self.step = tensors[self.step_name][self.index].float().contiguous()

    def forward(self, residual, ctx) -> None:
        ops.add_row(residual, self.step)


register_part("stream", "step_vector", StreamStepVector)
