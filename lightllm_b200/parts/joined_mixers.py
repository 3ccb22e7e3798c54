"""Several mixers side by side on one input, their outputs normed and averaged."""
from __future__ import annotations

import math
from typing import List, Optional, Sequence

import torch

from ..cache import CacheSpec, StateSpec
from ..config import PartSpec, part_class, register_part
from ..csrc import ops
from ..weights import WeightSpec
from .base import CacheView, LazyNorm, Mixer, Part


class JoinedMixers(Mixer):
    """``y = sum_i weight_i * rmsnorm(mixer_i(x)) * w_i``: every mixer reads the same x; each output is normed over the
    model width (``eps`` inside the root, its own plain weight ``out_norms[i]``, a full tensor name) before the sum;
    ``weights`` default to ``1 / len(mixers)`` (the mean).

    At most one of the mixers may keep pages (the run has one cache plane); their fixed-size states lie one behind the
    other in the run's state plane (flat float32), each mixer finding its own at ``CacheView.state_offset``.  The
    outputs, their norms and the sum are float32."""

    graph_safe = True
    accepts_lazy_norm = False

    def __init__(self, prefix: str, hidden_size: int, mixers: Sequence[PartSpec], out_norms: Sequence[str], eps: float,
                 weights: Optional[Sequence[float]] = None):
        if not mixers or len(out_norms) != len(mixers):
            raise ValueError("joined mixers: one norm weight's name for every mixer, at least one mixer")
        self.prefix, self.hidden_size, self.eps = prefix, hidden_size, float(eps)
        self.mixers: List[Mixer] = [part_class("mixer", m.kind)(m.prefix, **m.params) for m in mixers]
        self.out_names = list(out_norms)
        self.weights = [float(w) for w in weights] if weights is not None else [1.0 / len(mixers)] * len(mixers)
        if len(self.weights) != len(self.mixers):
            raise ValueError("joined mixers: one weight for every mixer")
        specs = [m.cache_spec() for m in self.mixers]
        paged = [i for i, s in enumerate(specs) if s is not None and s.kv is not None]
        if len(paged) > 1:
            raise ValueError("joined mixers: at most one of them may keep pages (a run has one cache plane)")
        self._kv = specs[paged[0]].kv if paged else None
        self._paged = paged[0] if paged else None
        self._offsets, total = [], 0
        for s in specs:
            self._offsets.append(total)
            if s is not None and s.state is not None:
                if s.state.dtype != "float32":
                    raise ValueError("joined mixers share one float32 state plane")
                total += math.prod(s.state.shape)
        self._state_floats = total
        self.out_w: List[Optional[torch.Tensor]] = [None] * len(self.mixers)

    def children(self) -> List[Part]:
        return list(self.mixers)

    def cache_spec(self) -> Optional[CacheSpec]:
        if self._kv is None and not self._state_floats:
            return None
        return CacheSpec(kv=self._kv, state=StateSpec((self._state_floats,), "float32") if self._state_floats else None)

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(n, (self.hidden_size,), init=("one_plus_normal", 0.1)) for n in self.out_names]

    def bind(self, tensors, dtype, device) -> None:
        self.out_w = [tensors[n] for n in self.out_names]

    def _view(self, i: int, cache: Optional[CacheView]) -> Optional[CacheView]:
        return None if cache is None else cache.at(self._offsets[i], pages=i == self._paged)

    def prepare(self, ctx, cache=None) -> None:
        for i, m in enumerate(self.mixers):
            if getattr(type(m), "prepare", None) is not Part.prepare:
                m.prepare(ctx, self._view(i, cache))

    def forward(self, x, residual, ctx, cache: Optional[CacheView]) -> None:
        if isinstance(x, LazyNorm):
            x = x.materialize()
        for i, m in enumerate(self.mixers):
            branch = torch.zeros(residual.shape, dtype=torch.float32, device=residual.device)
            m.forward(x, branch, ctx, self._view(i, cache))
            ops.rmsnorm_add(branch, self.out_w[i], self.eps, residual, self.weights[i])


register_part("mixer", "joined_mixers", JoinedMixers)
