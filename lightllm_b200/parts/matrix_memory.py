"""A matrix memory with exponential gates (the mLSTM cell of xLSTM), run as a recurrence over a per-request state."""
from __future__ import annotations

from typing import Dict, List, Optional

import numpy as np
import torch

from ..cache import CacheSpec, StateSpec
from ..config import register_part
from ..csrc import ops
from ..weights import WeightSpec
from . import linear as L
from .base import CacheView, LazyNorm, Mixer
from .conv_attention import span_arrays


class MatrixMemoryMixer(Mixer):
    """Per head, with S ``[head_dim, v_head_dim]``, n ``[head_dim]`` and a running maximum m, all zero before a
    request's first token::

        i_t = cap tanh((W_i x + b_i) / cap)               f_t = logsigmoid(cap tanh((W_f x + b_f) / cap))
        m_t = max(f_t + m_(t-1), i_t)
        S_t = exp(f_t + m_(t-1) - m_t) S_(t-1) + exp(i_t - m_t) k_t v_t^T          n_t likewise with k_t alone
        o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)                      q_t = W_q x * head_dim ** -0.5

    Each head's o is divided by its root mean square (``norm_eps``), the concatenated heads are multiplied by a weight
    (``norm``: all heads' size) and by ``sigmoid(W_g x)``, then projected by ``W_o``.

    One contraction makes q | k | v | gate in the compute dtype, a second one the two gates' pre-activations in
    float32.  S (with n as one more column) and m live in float32 in the request's state slot and are carried from span
    to span, so the result does not depend on how the tokens were cut.  Gates, the maximum, exponentials, the state,
    the outputs and the head norm are float32 in both precisions."""

    graph_safe = True
    accepts_lazy_norm = False

    def __init__(self, prefix: str, hidden_size: int, num_heads: int, head_dim: int, v_head_dim: int, gate_cap: float,
                 norm_eps: float = 1e-6, names: Optional[Dict[str, str]] = None, weight_suffix: str = "",
                 bias_ending: str = "b"):
        if not gate_cap > 0:
            raise ValueError(f"the gates' cap must be positive, got {gate_cap}")
        self.prefix, self.hidden_size = prefix, hidden_size
        self.num_heads, self.head_dim, self.v_head_dim = num_heads, head_dim, v_head_dim
        self.gate_cap, self.norm_eps = float(gate_cap), float(norm_eps)
        self.names = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "i": "i", "f": "f", "norm": "norm"}
        self.names.update(names or {})
        self.weight_suffix, self.bias_ending = weight_suffix, bias_ending
        self.matrix_floats = num_heads * head_dim * (v_head_dim + 1)          # S with n as its last column
        self.w_fused = self.w_gates = self.b_i = self.b_f = self.norm_w = self.w_o = None

    def _n(self, which: str, bias: bool = False) -> str:
        base = f"{self.prefix}.{self.names[which]}"
        return f"{base}.{self.bias_ending}" if bias else base + self.weight_suffix

    def cache_spec(self) -> CacheSpec:
        return CacheSpec(state=StateSpec((self.matrix_floats + self.num_heads,), "float32"))

    def weight_specs(self) -> List[WeightSpec]:
        D, H, hd, vd = self.hidden_size, self.num_heads, self.head_dim, self.v_head_dim
        return [WeightSpec(self._n("q"), (H * hd, D)), WeightSpec(self._n("k"), (H * hd, D)),
                WeightSpec(self._n("v"), (H * vd, D)), WeightSpec(self._n("g"), (H * vd, D)),
                WeightSpec(self._n("o"), (D, H * vd)),
                WeightSpec(f"{self.prefix}.{self.names['norm']}", (H * vd,), init=("one_plus_normal", 0.1)),
                WeightSpec(self._n("i"), (H, D)), WeightSpec(self._n("i", True), (H,), init=("normal", 1.0)),
                WeightSpec(self._n("f"), (H, D)), WeightSpec(self._n("f", True), (H,), init=("normal", 1.0))]

    def bind(self, tensors, dtype, device) -> None:
        ws = [tensors[self._n(p)] for p in "qkvg"]
        wdt = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
        self.w_fused = torch.cat([w.to(wdt) for w in ws], dim=0).contiguous()
        gi, gf = tensors[self._n("i")], tensors[self._n("f")]
        gdt = torch.float32 if torch.float32 in (gi.dtype, gf.dtype) else gi.dtype
        self.w_gates = torch.cat([gi.to(gdt), gf.to(gdt)], dim=0).contiguous()
        self.b_i = tensors[self._n("i", True)].float().contiguous()
        self.b_f = tensors[self._n("f", True)].float().contiguous()
        self.norm_w = tensors[f"{self.prefix}.{self.names['norm']}"].float().contiguous()
        self.w_o = tensors[self._n("o")]

    # A span longer than this is cut into pieces that run side by side (csrc/matrix_memory.cu).
    MIN_PIECE = 32
    WARPS_PER_SM = 16

    @property
    def prepare_key(self):
        return ("matrix_memory", self.num_heads, self.head_dim, self.v_head_dim)

    def _pieces(self, ctx):
        """(item_span, item_c, span_first, num_items, chunk) for this step: which pieces the spans are cut into."""
        key = ("matrix_memory_pieces", self.num_heads, self.head_dim, self.v_head_dim)
        hit = ctx.memo.get(key)
        if hit is not None:
            return hit
        longest = max(s.length for s in ctx.spans)
        chunk = 1 << 30
        if longest > 2 * self.MIN_PIECE:
            dg = 1 if self.head_dim <= 64 else 2 if self.head_dim <= 128 else 4 if self.head_dim <= 256 else 8
            warps = self.num_heads * -(-(self.v_head_dim + 1) * dg // 32)             # of one piece
            wanted = max(1, L.num_sms(ctx.device) * self.WARPS_PER_SM // warps)         # pieces in flight
            total = sum(s.length for s in ctx.spans)
            chunk = max(self.MIN_PIECE, -(-(-(-total // wanted)) // 16) * 16)
        counts = [-(-s.length // chunk) for s in ctx.spans]
        if max(counts) == 1:
            hit = (ctx.iota, ctx.zeros, ctx.iota, len(ctx.spans), 1 << 30)
        else:
            item_span = np.repeat(np.arange(len(counts), dtype=np.int32), counts)
            first = np.concatenate([[0], np.cumsum(counts)[:-1]]).astype(np.int32)
            item_c = (np.arange(len(item_span), dtype=np.int32) - first[item_span]).astype(np.int32)
            items = ctx.stage(np.stack([item_span, item_c]))
            hit = (items[0], items[1], ctx.stage(first), int(len(item_span)), int(chunk))
        ctx.shape_key.append(("matrix_memory", hit[3], hit[4]))
        ctx.memo[key] = hit
        return hit

    def prepare(self, ctx, cache=None) -> None:
        self._pieces(ctx)

    def forward(self, x, residual, ctx, cache: CacheView) -> None:
        if isinstance(x, LazyNorm):
            x = x.materialize()
        if cache is None or cache.state is None or not cache.writes:
            raise ops.KernelError("matrix memory: the run needs a state plane of its own (the recurrence advances it)")
        T = x.shape[0]
        H, hd, vd = self.num_heads, self.head_dim, self.v_head_dim
        f32 = dict(dtype=torch.float32, device=x.device)
        fused = L.linear(x, self.w_fused, None, L.STORE)                   # [T, q | k | v | gate]
        pre = L.linear(x, self.w_gates, None, L.STORE_F32)                 # [T, z_i | z_f]
        spans = span_arrays(ctx)
        off = cache.state_offset
        gates = torch.empty((3, T, H), **f32)
        ops.memory_gates(pre, 0, H, self.b_i, self.b_f, self.gate_cap, spans, H, cache.state, off + self.matrix_floats,
                         gates[0], gates[1], gates[2])
        num = torch.empty((T, H * vd), **f32)
        den = torch.empty((T, H), **f32)
        ops.matrix_memory(fused, 0, H * hd, 2 * H * hd, hd ** -0.5, gates[0], gates[1], gates[2], spans, H, hd, vd,
                          cache.state, off, num, den, pieces=self._pieces(ctx))
        gated = torch.empty((T, H * vd), dtype=x.dtype, device=x.device)
        g0 = 2 * H * hd + H * vd
        ops.head_gate(num, fused[:, g0: g0 + H * vd], gated, H, vd, False, "sigmoid", unit_rms=True, eps=self.norm_eps,
                      norm_weight=self.norm_w, denominator=den)
        L.linear(gated, self.w_o, None, L.RESIDUAL, residual=residual)


register_part("mixer", "matrix_memory", MatrixMemoryMixer)
