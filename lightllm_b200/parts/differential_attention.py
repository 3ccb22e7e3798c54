"""Differential attention: two softmax maps a head over the same values, subtracted and normed head by head."""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from ..config import PartSpec, register_part
from ..csrc import ops
from ..weights import WeightSpec
from . import linear as L
from .attention import AttentionMixer
from .base import CacheView, LazyNorm

MAPS = 2


class DifferentialAttentionMixer(AttentionMixer):
    """Grouped-query attention in which every head has TWO score maps over the same values:

        q [T, H, 2, dim], k [T, G, 2, dim], v [T, G, vdim]      (head by head ``[map 1, map 2]``; no biases)
        q, k <- rotate(rms_norm(q or k over dim) * w)           (``qk_norm``: a weight [dim] shared by heads and maps)
        a_m = softmax(scale q_m . k_m over the window) v        for m = 1, 2
        o   = unit_rms(a_1 - lambda a_2 over vdim) * (1 - diff)
        lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff         (four vectors [dim], one number a layer)

    followed by the output projection added into the stream.

    How it runs on the attention kernels the engine has: a kv head's two key maps lie side by side in one cache row of
    ``2 dim`` numbers, and query head (h, m) is written as a row of ``2 dim`` numbers that is zero outside its own map, so
    its dot product with the row is ``q_m . k_m``.  The kernels then see ordinary grouped-query attention with ``2 H``
    query heads over ``G`` kv heads with keys ``2 dim`` and values ``vdim`` wide, and every key and value row is read once
    for a kv head's ``2 H / G`` queries.  Where ``2 dim == vdim`` is 64 or 128 this takes the tensor-core kernels in
    bfloat16.  The maps' outputs leave the kernels in float32; one kernel subtracts, norms and scales them.

    ``own_kv=False``: the mixer has no key and value projections (nor their norm) and reads the cache plane of the run
    entry its own entry names (``RunEntry.cache_of``), with queries, window and everything else of its own.
    ``cache_window``: see :class:`AttentionMixer` (the plane must keep what its widest reader sees)."""

    graph_safe = True
    accepts_lazy_norm = False

    def __init__(self, prefix: str, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, v_head_dim: int,
                 diff: float, norm_eps: float = 1e-6, position: Optional[PartSpec] = None, window: Optional[int] = None,
                 cache_window: Optional[int] = None, scale: Optional[float] = None, qk_norm: bool = True,
                 own_kv: bool = True, names: Optional[Dict[str, str]] = None, weight_suffix: str = ".weight"):
        base = {"q": "q_proj", "k": "k_proj", "v": "v_proj", "o": "o_proj", "lq1": "lambda_q1", "lk1": "lambda_k1",
                "lq2": "lambda_q2", "lk2": "lambda_k2"}
        base.update(names or {})
        # the kernels' geometry: 2 H query heads, G kv heads, key rows of both maps, value rows of vdim
        super().__init__(prefix, hidden_size, MAPS * num_heads, num_kv_heads, MAPS * head_dim, position=position,
                         qkv_bias=False, out_bias=False, window=window,
                         scale=scale if scale is not None else 1.0 / math.sqrt(head_dim), names=base,
                         weight_suffix=weight_suffix, v_head_dim=v_head_dim, cache_window=cache_window)
        self.heads, self.kv_heads, self.map_dim = int(num_heads), int(num_kv_heads), int(head_dim)
        self.diff, self.norm_eps, self.qk_norm, self.own_kv = float(diff), float(norm_eps), bool(qk_norm), bool(own_kv)
        self.w_fused = self.q_norm_w = self.k_norm_w = None
        self.lam = 0.0

    def _vector(self, which: str) -> str:
        return f"{self.prefix}.{self.names[which]}"

    def weight_specs(self) -> List[WeightSpec]:
        D, H, G, d, vd = self.hidden_size, self.heads, self.kv_heads, self.map_dim, self.v_head_dim
        specs = [WeightSpec(self._n("q", "weight"), (H * MAPS * d, D)), WeightSpec(self._n("o", "weight"), (D, H * vd))]
        if self.own_kv:
            specs += [WeightSpec(self._n("k", "weight"), (G * MAPS * d, D)), WeightSpec(self._n("v", "weight"), (G * vd, D))]
        if self.qk_norm:
            specs.append(WeightSpec(self._n("q", "norm"), (d,), init=("one_plus_normal", 0.1)))
            if self.own_kv:
                specs.append(WeightSpec(self._n("k", "norm"), (d,), init=("one_plus_normal", 0.1)))
        specs += [WeightSpec(self._vector(v), (d,), init=("normal", 0.1)) for v in ("lq1", "lk1", "lq2", "lk2")]
        return specs + self.position.weight_specs()

    def bind(self, tensors, dtype, device) -> None:
        ws = [tensors[self._n(p, "weight")] for p in (("q", "k", "v") if self.own_kv else ("q",))]
        wdt = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
        self.w_fused = torch.cat([w.to(wdt) for w in ws], dim=0).contiguous()
        self.w_o = tensors[self._n("o", "weight")]
        if self.qk_norm:
            self.q_norm_w = tensors[self._n("q", "norm")].float().contiguous()
            if self.own_kv:
                self.k_norm_w = tensors[self._n("k", "norm")].float().contiguous()
        v = {name: tensors[self._vector(name)].double().cpu() for name in ("lq1", "lk1", "lq2", "lk2")}
        self.lam = float(torch.exp((v["lq1"] * v["lk1"]).sum()) - torch.exp((v["lq2"] * v["lk2"]).sum())) + self.diff
        self.position.bind(tensors, dtype, device)

    def forward(self, x, residual, ctx, cache: CacheView) -> None:
        if isinstance(x, LazyNorm):
            x = x.materialize()
        if cache.writes and not self.own_kv:
            raise ops.KernelError(f"{self.prefix}: a mixer without keys and values of its own must read another run's cache")
        T = x.shape[0]
        H, G, d, vd = self.heads, self.kv_heads, self.map_dim, self.v_head_dim
        writes = cache.writes
        w = self.w_fused if (writes or not self.own_kv) else self.w_fused[: H * MAPS * d]
        fused = L.linear(x, w, None, L.STORE)                       # [T, q | k | v]
        table = self.position.rotary_table()
        inv_freq, rotary_dim, interleaved = table if table is not None else (None, 0, False)
        q = torch.empty((T, H * MAPS * MAPS * d), dtype=x.dtype, device=x.device)
        k0 = H * MAPS * d
        ops.head_prepare(fused, 0, k0, H * MAPS, G * MAPS if writes else 0, d, ctx.positions,
                         ctx.slot_mapping[cache.group] if writes else None, q, cache.k, cache.v, q_maps=MAPS,
                         values="columns" if writes else None, v_off=k0 + G * MAPS * d if writes else -1,
                         v_width=G * vd if writes else 0, q_norm_w=self.q_norm_w, k_norm_w=self.k_norm_w,
                         eps=self.norm_eps, inv_freq=inv_freq, rotary_dim=rotary_dim, interleaved=interleaved)
        maps = torch.empty((T, H * MAPS * vd), dtype=torch.float32, device=x.device)
        self.attend(q, cache, ctx, maps)
        heads = torch.empty((T, H * vd), dtype=x.dtype, device=x.device)
        ops.diff_combine(maps, heads, H, vd, self.lam, self.norm_eps, 1.0 - self.diff)
        L.linear(heads, self.w_o, None, L.RESIDUAL, residual=residual)


register_part("mixer", "differential_attention", DifferentialAttentionMixer)
