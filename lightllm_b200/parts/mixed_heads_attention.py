"""Convolved attention whose heads' softmax weights are mixed before they meet the values."""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from ..cache import CacheSpec, KVSpec, StateSpec
from ..config import register_part
from ..csrc import ops
from ..weights import WeightSpec
from . import linear as L
from .base import CacheView, LazyNorm
from .conv_attention import ConvAttentionMixer, span_arrays


class MixedHeadsAttention(ConvAttentionMixer):
    """Grouped-query softmax attention over the paged cache, without rotation, in which

    * q, k and v pass a causal convolution of ``conv_taps`` taps (0: none), as in the parent;
    * q is multiplied by a temperature that grows with the position, ``1 + coef * ln(floor((p + 1) / every) + 1)``
      (``q_temperature = (coef, every)`` or ``None``);
    * every head of v is divided by its root mean square (``v_unit_rms``, ``norm_eps`` inside the root, no weight)
      and cached so;
    * after the softmax the heads' weights are mixed, ``w'_h = sum_g talk[h, g] w_g`` (``talk``: the tensor's name, or
      ``None``), and head h applies ``w'_h`` to the values of its own kv head;
    * the concatenated heads are multiplied by ``sigmoid(W_g x)`` (``gate``: the tensor's name, or ``None``) before
      the output projection.

    The mixed weights never exist: ``sum_j w'_h(j) v(j) = sum_g talk[h, g] sum_j w_g(j) v(j)``, so the attention kernels
    apply every query head's weights to the values of ALL kv heads (``value_cross``: the tensor-core kernels for
    portions and for single tokens when keys and values are 64 or 128 wide in bfloat16, else the CUDA-core kernel
    reading a slot's value row whole) and one kernel combines the ``heads x kv_heads`` results and gates them.  One
    contraction makes q | k | v | gate.
    Scores, softmax, the head sums, convolution sums, temperature and norms are float32 in both precisions."""

    def __init__(self, prefix: str, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, v_head_dim: int,
                 scale: float, conv_taps: int = 0, q_temperature: Optional[Sequence[float]] = None,
                 v_unit_rms: bool = True, norm_eps: float = 1e-6, talk: Optional[str] = "talk",
                 gate: Optional[str] = "g", names: Optional[Dict[str, str]] = None, weight_suffix: str = "",
                 conv_ending: str = "conv"):
        super().__init__(prefix, hidden_size, num_heads, num_kv_heads, head_dim, v_head_dim=v_head_dim, position=None,
                         conv_taps=conv_taps, qkv_bias=False, out_bias=False, scale=scale, names=names,
                         weight_suffix=weight_suffix, conv_ending=conv_ending)
        if q_temperature is not None and int(q_temperature[1]) < 1:
            raise ValueError(f"the query temperature steps every {q_temperature[1]} positions; at least 1")
        self.q_temperature = (float(q_temperature[0]), int(q_temperature[1])) if q_temperature is not None else None
        self.v_unit_rms, self.norm_eps = bool(v_unit_rms), float(norm_eps)
        self.talk_name = f"{prefix}.{talk}" if talk else None
        self.gate_name = f"{prefix}.{gate}" if gate else None
        self.value_cross = num_kv_heads
        self.w_fused = self.talk = None

    def cache_spec(self) -> CacheSpec:
        vd = None if self.v_head_dim == self.head_dim else self.v_head_dim
        state = StateSpec(((self.conv_taps - 1) * self.channels,), "float32") if self.conv_taps > 1 else None
        return CacheSpec(kv=KVSpec(self.num_kv_heads, self.head_dim, None, vd, None), state=state)

    def weight_specs(self) -> List[WeightSpec]:
        specs = super().weight_specs()
        H, vd, D = self.num_heads, self.v_head_dim, self.hidden_size
        if self.talk_name:
            specs.append(WeightSpec(self.talk_name, (H, H), init=("normal", 0.4)))
        if self.gate_name:
            specs.append(WeightSpec(self.gate_name, (H * vd, D)))
        return specs

    def bind(self, tensors, dtype, device) -> None:
        super().bind(tensors, dtype, device)
        if self.gate_name:
            g = tensors[self.gate_name]
            wdt = torch.float32 if torch.float32 in (g.dtype, self.w_qkv.dtype) else self.w_qkv.dtype
            self.w_fused = torch.cat([self.w_qkv.to(wdt), g.to(wdt)], dim=0).contiguous()
        else:
            self.w_fused = self.w_qkv
        self.w_qkv = None
        self.talk = tensors[self.talk_name].float().contiguous() if self.talk_name else None

    def forward(self, x, residual, ctx, cache: CacheView) -> None:
        if isinstance(x, LazyNorm):
            x = x.materialize()
        if cache is None or not cache.writes or cache.k is None or (self.conv_taps > 1 and cache.state is None):
            raise ops.KernelError("mixed-heads attention: the run needs cache planes and a state plane of its own")
        T = x.shape[0]
        H, G, hd, vd = self.num_heads, self.num_kv_heads, self.head_dim, self.v_head_dim
        fused = L.linear(x, self.w_fused, None, L.STORE)           # [T, q | k | v | gate]
        q = torch.empty((T, H * hd), dtype=x.dtype, device=x.device)
        segments = [ops.ConvSegment(0, H, hd, q, temperature=self.q_temperature),
                    ops.ConvSegment(H * hd, G, hd, cache.k, to_cache=True),
                    ops.ConvSegment((H + G) * hd, G, vd, cache.v, to_cache=True,
                                    norm="rms" if self.v_unit_rms else None, eps=self.norm_eps)]
        spans = span_arrays(ctx)
        tail_off = cache.state_offset
        ops.conv_prepare(fused, 0, self.channels, self.w_conv, segments, spans, cache.state if self.conv_taps > 1 else None,
                         tail_off, ctx.slot_mapping[cache.group], fuse_tail=ctx.decode_only and self.conv_taps > 1)
        if self.conv_taps > 1 and not ctx.decode_only:
            ops.conv_tail_update(fused, 0, self.channels, self.conv_taps, spans, cache.state, tail_off)
        # every query head over every kv head's values, float32: the heads are summed before anything is rounded
        every = torch.empty((T, H * G * vd), dtype=torch.float32, device=x.device)
        self.attend(q, cache, ctx, every)
        heads = torch.empty((T, H * vd), dtype=x.dtype, device=x.device)
        gate = fused[:, self.channels:] if self.gate_name else None
        ops.talk_mix(every, self.talk, gate, heads, H, G, vd)
        L.linear(heads, self.w_o, None, L.RESIDUAL, residual=residual)


register_part("mixer", "mixed_heads_attention", MixedHeadsAttention)
