"""Attention whose keys double as values, with soft-capped scores, a learned sink a head and a gate a head."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config import PartSpec, register_part
from ..csrc import ops
from ..weights import WeightSpec
from . import linear as L
from .attention import AttentionMixer
from .base import CacheView, LazyNorm


class KeyValuedAttentionMixer(AttentionMixer):
    """Grouped-query attention without a value projection:

        q = W_q x + b_q,  k = W_k x + b_k                       (``qk_bias``)
        v = k                                                   the keys as projected, BEFORE their rotation
        q, k <- rotate(q, k)                                    (the first ``rotary_dim`` dimensions)
        s = scale q . k;  s <- softcap tanh(s / softcap)        (``softcap``; none: the scores as they are)
        p = exp(s) / (sum over the window of exp(s) + exp(sink_h))   (``sinks``: a learned logit a head that has no
                                                                key and no value, is neither scaled nor capped)
        o_h = sigmoid(w_g,h . x) * sum p v                      (``gate``: one number a head, from the mixer's input)

    and the output projection added into the stream.  The cache keeps the rotated keys in its key plane and the
    projected ones in its value plane (with every dimension rotated nothing of the two is shared).  One contraction
    makes q, k and the gates' inputs; one kernel rotates and writes both planes; the gate is applied in place.

    ``cache_window`` as :class:`AttentionMixer`."""

    graph_safe = True
    accepts_lazy_norm = False

    def __init__(self, prefix: str, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 position: Optional[PartSpec] = None, window: Optional[int] = None, cache_window: Optional[int] = None,
                 scale: Optional[float] = None, softcap: Optional[float] = None, sinks: bool = True, gate: bool = True,
                 qk_bias: bool = True, names: Optional[Dict[str, str]] = None, weight_suffix: str = ".weight",
                 bias_ending: str = "bias"):
        if softcap is not None and not softcap > 0:
            raise ValueError(f"a soft cap on the scores must be positive, got {softcap}")
        base = {"q": "q_proj", "k": "k_proj", "o": "o_proj", "g": "g_proj", "sink": "sink"}
        base.update(names or {})
        super().__init__(prefix, hidden_size, num_heads, num_kv_heads, head_dim, position=position, qkv_bias=bool(qk_bias),
                         out_bias=False, window=window, scale=scale, names=base, weight_suffix=weight_suffix,
                         cache_window=cache_window)
        self.softcap = float(softcap) if softcap else None
        self.has_sinks, self.gate, self.bias_ending = bool(sinks), bool(gate), bias_ending
        self.w_fused = self.b_fused = None

    def _bias(self, which: str) -> str:
        return f"{self.prefix}.{self.names[which]}.{self.bias_ending}"

    def weight_specs(self) -> List[WeightSpec]:
        D, H, G, d = self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim
        specs = [WeightSpec(self._n("q", "weight"), (H * d, D)), WeightSpec(self._n("k", "weight"), (G * d, D)),
                 WeightSpec(self._n("o", "weight"), (D, H * d))]
        if self.qkv_bias:
            specs += [WeightSpec(self._bias("q"), (H * d,), init=("normal", 0.1)),
                      WeightSpec(self._bias("k"), (G * d,), init=("normal", 0.1))]
        if self.has_sinks:
            specs.append(WeightSpec(f"{self.prefix}.{self.names['sink']}", (H,), init=("normal", 1.0)))
        if self.gate:
            specs.append(WeightSpec(self._n("g", "weight"), (H, D)))
        return specs + self.position.weight_specs()

    def bind(self, tensors, dtype, device) -> None:
        H, G, d = self.num_heads, self.num_kv_heads, self.head_dim
        ws = [tensors[self._n(p, "weight")] for p in ("q", "k") + (("g",) if self.gate else ())]
        wdt = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
        rows = sum(w.shape[0] for w in ws)
        pad = -rows % 8          # whole 16-byte pieces a row of the fused output, for the contraction's staged stores
        if pad:
            ws.append(torch.zeros((pad, self.hidden_size), dtype=wdt, device=ws[0].device))
        self.w_fused = torch.cat([w.to(wdt) for w in ws], dim=0).contiguous()
        if self.qkv_bias:
            b = torch.zeros(rows + pad, dtype=torch.float32, device=ws[0].device)
            b[: H * d] = tensors[self._bias("q")].float()
            b[H * d: (H + G) * d] = tensors[self._bias("k")].float()
            self.b_fused = b.contiguous()
        self.w_o = tensors[self._n("o", "weight")]
        if self.has_sinks:
            self.sinks = tensors[f"{self.prefix}.{self.names['sink']}"].float().contiguous()
        self.position.bind(tensors, dtype, device)

    def forward(self, x, residual, ctx, cache: CacheView) -> None:
        if isinstance(x, LazyNorm):
            x = x.materialize()
        T = x.shape[0]
        H, G, d = self.num_heads, self.num_kv_heads, self.head_dim
        writes = cache.writes
        fused = L.linear(x, self.w_fused, self.b_fused, L.STORE)          # [T, q | k | gates]
        table = self.position.rotary_table()
        inv_freq, rotary_dim, interleaved = table if table is not None else (None, 0, False)
        q = torch.empty((T, H * d), dtype=x.dtype, device=x.device)
        ops.head_prepare(fused, 0, H * d, H, G, d, ctx.positions, ctx.slot_mapping[cache.group] if writes else None, q,
                         cache.k, cache.v, values="keys" if writes else None, inv_freq=inv_freq, rotary_dim=rotary_dim,
                         interleaved=interleaved)
        attn = torch.empty((T, H * d), dtype=x.dtype, device=x.device)
        self.attend(q, cache, ctx, attn)
        if self.gate:
            g0 = (H + G) * d
            ops.head_gate(attn, fused[:, g0: g0 + H], attn, H, d, True, "sigmoid")
        L.linear(attn, self.w_o, None, L.RESIDUAL, residual=residual)


register_part("mixer", "key_valued_attention", KeyValuedAttentionMixer)
