"""A causal convolution over time on what a sub-block reads."""
from __future__ import annotations

from typing import List, Optional

import torch

from ..config import register_part
from ..csrc import ops
from ..weights import WeightSpec
from .base import CacheView, InputFilter
from .conv_attention import span_arrays


class CausalInputConv(InputFilter):
    """``x_t = h_t + sum_j w[:, j] * h_(t - taps + 1 + j)`` on every channel of the normed stream h (``residual=False``:
    without the ``h_t +``), zeros before the sequence's start.  ``weight_name`` is ``[channels, taps]``, no bias.

    h arrives in float32 and the sums are float32; the result is rounded once, to the compute dtype.  A request's last
    ``taps - 1`` rows of h live in the run's state plane (float32), so any cutting of its tokens gives the same result.
    Several filters may read one h (the sub-blocks of a parallel layer): they share that record, and the last of them
    (``last_reader``) brings it up to date.

    The kernel is the one that convolves fused projections (csrc/short_conv.cu), with the channels cut into "heads" of
    up to 64 for its warps and ``h_t +`` folded into the last tap's weight."""

    graph_safe = True

    def __init__(self, prefix: str, channels: int, taps: int, weight_name: str = "weight", residual: bool = True):
        if taps < 1:
            raise ValueError(f"a convolution has at least one tap, got {taps}")
        self.name = f"{prefix}.{weight_name}" if prefix and weight_name else (prefix or weight_name)
        self.channels, self.taps, self.residual = int(channels), int(taps), bool(residual)
        # the widest divisor of the channels up to 64, a pair of channels a lane: narrow pieces give a single token's
        # convolution to many warps instead of a few long loops
        self.piece = next(d for d in range(min(64, self.channels), 0, -1) if self.channels % d == 0)
        self.weight = None

    def state_floats(self) -> int:
        return (self.taps - 1) * self.channels

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.name, (self.channels, self.taps), init=("normal", 0.3))]

    def bind(self, tensors, dtype, device) -> None:
        w = tensors[self.name].float().clone()
        if self.residual:
            w[:, -1] += 1.0
        self.weight = w.contiguous()

    def forward(self, h, ctx, cache: Optional[CacheView], out_dtype, last_reader: bool = True):
        T, C = h.shape
        if h.dtype != torch.float32 or C != self.channels:
            raise ops.KernelError(f"input convolution: float32 [T, {self.channels}] expected, got {h.dtype} {tuple(h.shape)}")
        out = torch.empty((T, C), dtype=out_dtype, device=h.device)
        state = cache.state if cache is not None else None
        off = cache.state_offset if cache is not None else 0
        spans = span_arrays(ctx)
        fuse = bool(last_reader and ctx.decode_only and self.taps > 1)
        ops.conv_prepare(h, 0, C, self.weight, [ops.ConvSegment(0, C // self.piece, self.piece, out)], spans,
                         state if self.taps > 1 else None, off, fuse_tail=fuse)
        if last_reader and self.taps > 1 and not fuse:
            ops.conv_tail_update(h, 0, C, self.taps, spans, state, off)
        return out


register_part("filter", "causal_conv", CausalInputConv)
