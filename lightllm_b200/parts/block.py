"""A block: sub-blocks (norm before, a mixer or feed-forward, norm after) around the residual stream."""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from ..cache import CacheSpec, StateSpec
from ..config import LayerSpec, part_class
from ..csrc import ops
from .base import CacheView, LazyNorm, Part


_STREAM_COPY = "stream in the compute dtype"      # ctx.memo key: (the stream tensor, its copy), valid until the stream changes


def build_part(role: str, spec):
    return part_class(role, spec.kind)(spec.prefix, **spec.params)


class BuiltSubBlock:
    """The parts of one :class:`~lightllm_b200.config.SubBlock`."""

    def __init__(self, spec):
        self.role = spec.role
        self.part = build_part(spec.role, spec.part)
        self.norm_before = build_part("norm", spec.norm_before) if spec.norm_before is not None else None
        self.norm_after = build_part("norm", spec.norm_after) if spec.norm_after is not None else None
        self.after = spec.after
        self.filter = build_part("filter", spec.input_filter) if spec.input_filter is not None else None
        if self.filter is not None and self.norm_before is None:
            raise ValueError("an input filter works on a sub-block's normed input; the sub-block has no norm before it")
        self.shares_input_of: Optional[int] = None       # index of the earlier sub-block whose normed stream this one reads
        self.filter_offset = 0                            # where the filter's floats begin in the run's state slot
        self.last_reader = True                           # the last of the sub-blocks that share a normed stream

    def parts(self) -> List[Part]:
        return [p for p in (self.norm_before, self.filter, self.part, self.norm_after) if p is not None]


class Block(Part):
    """``sequential``: every sub-block reads the stream the one before it left, e.g. Qwen2's
    ``h += mixer(norm1(h)); h += ffn(norm2(h))`` (src/engine/engine_server.cpp:1530-1880);
    ``parallel``: all sub-blocks read the same h, then every branch is added.
    What a sub-block may hold is described at :class:`~lightllm_b200.config.SubBlock`."""

    role = "block"

    def __init__(self, spec: LayerSpec):
        self.arrangement = spec.arrangement
        self.branch_scale = float(spec.branch_scale)
        self.subs: List[BuiltSubBlock] = [BuiltSubBlock(sb) for sb in spec.sub_blocks]
        mixers = [sb.part for sb in self.subs if sb.role == "mixer"]
        self.mixer: Optional[Part] = mixers[0] if mixers else None
        # Sub-blocks of a parallel layer with equal norms before them read one normed stream: it is made once, and the
        # filters on it share one record of the request's earlier tokens, which the last of them brings up to date.
        if self.arrangement == "parallel":
            for i, (sb, sp) in enumerate(zip(self.subs, spec.sub_blocks)):
                for j in range(i):
                    if sp.norm_before is not None and spec.sub_blocks[j].norm_before == sp.norm_before:
                        sb.shares_input_of = self.subs[j].shares_input_of if self.subs[j].shares_input_of is not None else j
                        break
        self.filtered = any(sb.filter is not None for sb in self.subs)
        self._mixer_floats = 0
        self._state_floats = 0

    def children(self) -> List[Part]:
        return [p for sb in self.subs for p in sb.parts()]

    def cache_spec(self) -> Optional[CacheSpec]:
        """What a run of this layer asks of the cache: the mixer's pages and state, and behind the mixer's state, in the
        same (then flat, float32) state plane, what the input filters keep of earlier tokens."""
        spec = self.mixer.cache_spec() if self.mixer is not None else None
        if not self.filtered:
            return spec
        own = 0
        if spec is not None and spec.state is not None:
            if spec.state.dtype != "float32":
                raise ValueError("input filters share the mixer's state plane, which must then be float32")
            own = math.prod(spec.state.shape)
        self._mixer_floats = total = own
        offsets: Dict[int, int] = {}
        for i, sb in enumerate(self.subs):
            if sb.filter is None:
                continue
            first = sb.shares_input_of if sb.shares_input_of is not None and self.subs[sb.shares_input_of].filter is not None else i
            if first in offsets:
                if self.subs[first].filter.state_floats() != sb.filter.state_floats():
                    raise ValueError("filters on one normed stream must keep the same number of earlier tokens")
                sb.filter_offset = offsets[first]
                self.subs[first].last_reader = False
                for j in range(first + 1, i):
                    if self.subs[j].filter is not None and self.subs[j].filter_offset == offsets[first]:
                        self.subs[j].last_reader = False
            else:
                sb.filter_offset = offsets[i] = total
                total += sb.filter.state_floats()
        self._state_floats = total
        if total == 0:
            return spec
        return CacheSpec(kv=spec.kv if spec is not None else None, state=StateSpec((total,), "float32"))

    @staticmethod
    def _input(sb: BuiltSubBlock, residual, ctx, lazy: bool):
        """The part's input: the norm left to the part when it can fold it into its first kernel."""
        if sb.norm_before is None:
            dtype = ctx.dtype if ctx is not None and ctx.dtype is not None else residual.dtype
            if dtype == residual.dtype:
                return residual
            ready = ctx.memo.pop(_STREAM_COPY, None) if ctx is not None else None
            if ready is not None and ready[0] is residual and ready[1].dtype == dtype:
                return ready[1]          # the kernel that last wrote the stream left it in the compute dtype too
            x = torch.empty(residual.shape, dtype=dtype, device=residual.device)
            ops.cast_add(residual, x)
            return x
        if lazy and sb.part.accepts_lazy_norm:
            return LazyNorm(residual, sb.norm_before, ctx)
        return sb.norm_before.forward(residual, ctx)

    @staticmethod
    def _run(sb: BuiltSubBlock, x, residual, ctx, cache, into=None) -> None:
        """``into``: the float buffer that collects the layer's branches instead of the stream (a scaled layer)."""
        branch = sb.norm_after is not None and sb.after == "branch"
        if ctx is not None:
            ctx.memo.pop(_STREAM_COPY, None)          # the stream is about to change
        target = residual if into is None else into
        if into is not None and sb.norm_after is not None:
            raise ops.KernelError("a layer with a branch scale takes no norms after its branches")
        if branch:      # the part adds into a cleared buffer, which is normed and then added to the stream
            target = torch.zeros_like(residual)
        elif x is residual:      # a part without a norm before it, in float32: it must not read what it adds into
            x = residual.clone()
        if sb.role == "mixer":
            sb.part.forward(x, target, ctx, cache)
        else:
            sb.part.forward(x, target, ctx)
        if branch and hasattr(sb.norm_after, "add_into"):
            # one kernel, the sum in float32; in bfloat16 it also leaves the new stream in the compute dtype, which the
            # next branch's projections read if that branch has no norm before it
            copy = None
            if ctx is not None and ctx.dtype == torch.bfloat16 and getattr(sb.norm_after, "copies_stream", False):
                copy = torch.empty(residual.shape, dtype=torch.bfloat16, device=residual.device)
            if copy is not None:
                sb.norm_after.add_into(target, residual, ctx, copy=copy)
                ctx.memo[_STREAM_COPY] = (residual, copy)
            else:
                sb.norm_after.add_into(target, residual, ctx)
        elif branch:
            ops.cast_add(sb.norm_after.forward(target, ctx), residual, accumulate=True)
        elif sb.norm_after is not None:
            ops.cast_add(sb.norm_after.forward(residual, ctx), residual)

    def _filtered_input(self, i: int, residual, ctx, cache, normed: Dict[int, torch.Tensor]):
        """The input of sub-block i through its filter: the normed stream in float32 (made once for the sub-blocks that
        share it), then the filter, which rounds to the compute dtype."""
        sb = self.subs[i]
        first = sb.shares_input_of if sb.shares_input_of is not None else i
        h = normed.get(first)
        if h is None:
            h = normed[first] = sb.norm_before.forward(residual, ctx, dtype=torch.float32)
        if cache is None or cache.state is None:
            if sb.filter.state_floats():
                raise ops.KernelError("an input filter keeps earlier tokens in the run's state plane; the run has none")
            view = None
        else:
            view = cache.at(sb.filter_offset, pages=False)
        return sb.filter.forward(h, ctx, view, ctx.dtype if ctx is not None and ctx.dtype is not None else h.dtype,
                                 last_reader=sb.last_reader)

    def forward(self, residual, ctx, cache) -> None:
        scaled = self.branch_scale != 1.0
        into = torch.zeros_like(residual) if scaled else None          # the branches' sum, scaled as it joins the stream
        normed: Dict[int, torch.Tensor] = {}
        if self.arrangement == "parallel":
            # every branch reads the same h, so all inputs are computed before anything is added
            inputs = [self._filtered_input(i, residual, ctx, cache, normed) if sb.filter is not None
                      else self._input(sb, residual, ctx, lazy=False) for i, sb in enumerate(self.subs)]
            inputs = [x.clone() if x is residual else x for x in inputs]
            for sb, x in zip(self.subs, inputs):
                self._run(sb, x, residual, ctx, cache, into)
            if scaled:
                ops.axpy(into, residual, self.branch_scale)
        else:
            for i, sb in enumerate(self.subs):
                x = (self._filtered_input(i, residual, ctx, cache, {}) if sb.filter is not None
                     else self._input(sb, residual, ctx, lazy=True))
                self._run(sb, x, residual, ctx, cache, into)
                if scaled:
                    ops.axpy(into, residual, self.branch_scale)
                    into.zero_()
