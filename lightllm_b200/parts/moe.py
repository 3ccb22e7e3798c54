"""Feed-forward layers made of routed experts."""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Tuple

import torch

from ..config import register_part
from ..csrc import ops
from ..weights import WeightSpec
from . import linear as L
from .base import FeedForward, LazyNorm
from .mlp import ACTIVATIONS


class RoutedExperts(FeedForward):
    """``h += sum over the chosen experts e of w_e * W_down_e (act(W_gate_e x) * (W_up_e x))``.

    Routing (float32): logits ``z = W_r x``, scores ``sigmoid(z)`` (or a softmax over the experts with
    ``score="softmax"``), the ``top`` experts with the largest ``score + correction`` (``correction``: a per-expert
    tensor that takes part in the choice only, or none), weights = the chosen experts' scores, divided by their sum
    (+ ``renorm_eps``) with ``renormalize``, times ``route_scale``.

    ``groups = (count, keep)``: the router's outputs form ``count`` equal groups of neighbours, a group's score is its
    largest choice score, and only outputs of the ``keep`` best groups can be chosen.  ``identity`` = n: the router has
    ``num_experts + n`` outputs and the last n are identity experts without tensors, whose output is the input x itself
    (times the weight); they take part in scores, groups and the choice like any other.  ``activation``: ``silu``, or
    ``clamped_swish`` with ``alpha``, ``limit``, ``up_shift`` (see :class:`~.mlp.GatedMLP`).  ``shared`` = ``{"intermediate_size",
    "activation", "alpha", "limit", "up_shift", "gate"}``: one more expert of the same form (tensors under ``shared_prefix``)
    that every token takes; with ``gate`` its output is multiplied by ``sigmoid(w_sg . x)``, one number a token (the row
    ``<shared_prefix><gate name>`` [1, D]), computed in float beside the router's logits.

    Three ways to run the experts, all with launches whose shapes follow from the step's token count alone, so that steps
    replay from CUDA graphs:

    * **every expert on every row** (few rows, float32, odd sizes): gate and up of all experts are the rows of one matrix
      (interleaved pair by pair, the gated activation in the contraction's epilogue), the activations of expert e are
      multiplied by w_e (zero for the experts a token did not choose) and the down matrices, side by side along the inner
      dimension, add the weighted sum into the stream: ``sum_e w_e W_down_e a_e = [W_down_0 .. W_down_E-1] [w_0 a_0; ..;
      w_E-1 a_E-1]``.  A decode step reads every expert's weights once, as it would anyway from about ``E / top`` rows on.
    * **pair by pair** (bfloat16, fewer (token, expert) pairs than experts: a decode step of a few rows): every pair streams
      its own expert's weights through a CUDA-core kernel and the experts nobody chose are not read.
    * **grouped** (bfloat16 on the tensor cores, from ``GROUPED_MIN_ROWS`` rows on or where it needs less arithmetic): the
      (token, expert) pairs are sorted by expert on the device, every expert's rows padded to whole tiles of 128, the rows
      gathered, and two grouped contractions (each row tile takes its expert's weights) make the experts' outputs in
      float, which are then added into the stream token by token with the routing weights, in the order of the choice.
      The padded row count is bounded by ``T * top + 128 * E`` on the host, so nothing is read back from the device."""

    graph_safe = True
    accepts_lazy_norm = False
    GROUPED = True               # False: every expert on every row, always (for comparisons)
    # From this many rows on the grouped contractions are taken whatever the arithmetic says: measured at the 0.5B sizes
    # with 8 experts of which 2 are chosen, a decode step of 64 rows takes 1.10 ms grouped against 1.19 ms with every
    # expert on every row (the few-row contraction streams 4 times the weights at a quarter of the memory bandwidth),
    # one of 8 rows 0.98 against 0.91.
    GROUPED_MIN_ROWS = 48

    def __init__(self, prefix: str, hidden_size: int, intermediate_size: int, num_experts: int, top: int,
                 route_scale: float = 1.0, score: str = "sigmoid", renormalize: bool = False, correction: bool = False,
                 activation: str = "silu", names: Optional[Dict[str, str]] = None, weight_suffix: str = ".weight",
                 expert_prefix: str = "experts.", renorm_eps: float = 0.0, groups: Optional[Tuple[int, int]] = None,
                 identity: int = 0, alpha: float = 1.0, limit: Optional[float] = None, up_shift: float = 0.0,
                 shared: Optional[Dict] = None, shared_prefix: str = "shared."):
        outputs = num_experts + int(identity)
        if num_experts < 0 or identity < 0 or not 0 < top <= outputs:
            raise ValueError(f"top {top} of {num_experts} experts and {identity} identity experts")
        if score not in ("sigmoid", "softmax"):
            raise ValueError(f"score must be 'sigmoid' or 'softmax', got {score!r}")
        if activation not in ("silu", "clamped_swish"):
            raise ValueError(f"routed experts implement the SiLU and the clamped swish gate, not {activation!r}")
        if activation == "clamped_swish" and (limit is None or not limit > 0):
            raise ValueError("the clamped gate needs a positive 'limit'")
        if groups is not None:
            count, keep = int(groups[0]), int(groups[1])
            if count < 1 or outputs % count or not 1 <= keep <= count or keep * (outputs // count) < top:
                raise ValueError(f"{outputs} router outputs in {count} groups of which {keep} are kept cannot give {top} choices")
            groups = (count, keep) if count > 1 and keep < count else None          # one group, or all kept: no limit
        self.prefix, self.hidden_size, self.intermediate_size = prefix, hidden_size, intermediate_size
        self.num_experts, self.top, self.route_scale = num_experts, top, float(route_scale)
        self.identity, self.groups, self.renorm_eps = int(identity), groups, float(renorm_eps)
        self.score, self.renormalize, self.has_correction = score, bool(renormalize), bool(correction)
        # the contractions' GLU epilogue: None is SiLU
        self.glu = None if activation == "silu" else (ACTIVATIONS[activation], float(alpha), float(limit), float(up_shift))
        self.names = {"gate": "gate_proj", "up": "up_proj", "down": "down_proj", "router": "router",
                      "correction": "correction", "shared_gate": "gate"}
        self.names.update(names or {})
        self.weight_suffix, self.expert_prefix, self.shared_prefix = weight_suffix, expert_prefix, shared_prefix
        self.shared = None
        if shared is not None:
            act = shared.get("activation", activation)
            if act not in ("silu", "clamped_swish"):
                raise ValueError(f"the shared expert implements the SiLU and the clamped swish gate, not {act!r}")
            if act == "clamped_swish" and not (shared.get("limit") or 0) > 0:
                raise ValueError("the shared expert's clamped gate needs a positive 'limit'")
            self.shared = {"size": int(shared["intermediate_size"]), "gate": bool(shared.get("gate", False)),
                           "glu": None if act == "silu" else (ACTIVATIONS[act], float(shared.get("alpha", alpha)),
                                                               float(shared["limit"]), float(shared.get("up_shift", up_shift)))}
        self.w_router = self.correction = self.w_gate_up = self.w_down = self.w_down_rows = None
        self.w_shared_gate_up = self.w_shared_down = None

    @property
    def outputs(self) -> int:
        """Outputs of the router: the experts and the identity experts."""
        return self.num_experts + self.identity

    def _e(self, e: int, which: str) -> str:
        return f"{self.prefix}.{self.expert_prefix}{e}.{self.names[which]}{self.weight_suffix}"

    def _s(self, which: str) -> str:
        return f"{self.prefix}.{self.shared_prefix}{self.names[which]}{self.weight_suffix}"

    def weight_specs(self) -> List[WeightSpec]:
        D, I = self.hidden_size, self.intermediate_size
        specs = [WeightSpec(f"{self.prefix}.{self.names['router']}{self.weight_suffix}", (self.outputs, D), init=("normal", 0.1))]
        if self.has_correction:
            specs.append(WeightSpec(f"{self.prefix}.{self.names['correction']}", (self.outputs,), init=("normal", 0.1)))
        for e in range(self.num_experts):
            specs += [WeightSpec(self._e(e, "gate"), (I, D)), WeightSpec(self._e(e, "up"), (I, D)),
                      WeightSpec(self._e(e, "down"), (D, I))]
        if self.shared is not None:
            S = self.shared["size"]
            specs += [WeightSpec(self._s("gate"), (S, D)), WeightSpec(self._s("up"), (S, D)), WeightSpec(self._s("down"), (D, S))]
            if self.shared["gate"]:
                specs.append(WeightSpec(self._s("shared_gate"), (1, D), init=("normal", 0.1)))
        return specs

    def bind(self, tensors, dtype, device) -> None:
        E, I, D = self.num_experts, self.intermediate_size, self.hidden_size
        self.w_router = tensors[f"{self.prefix}.{self.names['router']}{self.weight_suffix}"].float().contiguous()
        if self.shared is not None and self.shared["gate"]:          # the gate's row rides behind the router's rows
            self.w_router = torch.cat([self.w_router, tensors[self._s("shared_gate")].float().view(1, D)]).contiguous()
        if self.has_correction:
            self.correction = tensors[f"{self.prefix}.{self.names['correction']}"].float().contiguous()
        if self.shared is not None:
            g, u = tensors[self._s("gate")], tensors[self._s("up")]
            wdt = torch.float32 if torch.float32 in (g.dtype, u.dtype) else g.dtype
            self.w_shared_gate_up = torch.stack([g.to(wdt), u.to(wdt)], dim=1).reshape(2 * self.shared["size"], D).contiguous()
            self.w_shared_down = tensors[self._s("down")]
            L.reserve_fused_scratch(device, 2 * self.shared["size"])
        if E == 0:
            return
        gates, ups = [tensors[self._e(e, "gate")] for e in range(E)], [tensors[self._e(e, "up")] for e in range(E)]
        downs = [tensors[self._e(e, "down")] for e in range(E)]
        wide = any(w.dtype == torch.float32 for w in gates + ups + downs)
        wdt = torch.float32 if wide else gates[0].dtype
        # rows: expert by expert, (gate_j, up_j) adjacent, so that the epilogue writes act(gate) * up in expert order
        self.w_gate_up = torch.stack([torch.stack([g.to(wdt), u.to(wdt)], dim=1).reshape(2 * I, D)
                                      for g, u in zip(gates, ups)]).reshape(E * 2 * I, D).contiguous()
        self.w_down = torch.cat([w.to(wdt) for w in downs], dim=1).contiguous()          # [D, E * I]
        if wdt == torch.bfloat16 and dtype == torch.bfloat16 and self.top < self.outputs and D % 8 == 0 and I % 8 == 0:
            self.w_down_rows = torch.cat(downs, dim=0).contiguous()                     # [E * D, I]: expert by expert
            self._iota = torch.arange(max(E, self.top), dtype=torch.int32, device=device)          # each pair's own row, pair by pair
        L.reserve_fused_scratch(device, E * 2 * I)

    def route(self, x):
        """(ids [T, top] int32, -1 for an identity expert; weights [T, top]; dense weights [T, experts]; the summed weights
        of a token's identity experts [T] or None; the shared expert's gate [T, 1] or None) of the rows of x."""
        T = x.shape[0]
        ids = torch.empty((T, self.top), dtype=torch.int32, device=x.device)
        weights = torch.empty((T, self.top), dtype=torch.float32, device=x.device)
        dense = torch.empty((T, max(self.num_experts, 1)), dtype=torch.float32, device=x.device)
        idw = torch.empty(T, dtype=torch.float32, device=x.device) if self.identity else None
        gated = self.shared is not None and self.shared["gate"]
        gate = torch.empty((T, 1), dtype=torch.float32, device=x.device) if gated else None
        count, keep = self.groups or (0, 0)
        ops.moe_route(x, self.w_router, self.correction, self.top, self.route_scale, ids, weights, dense,
                      softmax=self.score == "softmax", renormalize=self.renormalize, renorm_eps=self.renorm_eps,
                      real=self.num_experts, groups=count, keep=keep, identity_weight=idw,
                      gate_rows=1 if gated else 0, gate_out=gate)
        return ids, weights, dense, idw, gate

    def _forward_shared(self, x, residual, gate) -> None:
        """The expert every token takes: ``residual += gate * W_down act`` (the gate, one number a token, multiplies the
        activations, which commutes with the down projection)."""
        sh = self.shared
        act = L.linear(x, self.w_shared_gate_up, None, L.SWIGLU, glu=sh["glu"])
        if gate is not None:
            ops.moe_scale(act, gate, 1, sh["size"])
        L.linear(act, self.w_shared_down, None, L.RESIDUAL, residual=residual)

    def grouped_pays(self, rows: int) -> bool:
        """Whether the grouped contractions need less arithmetic than every expert on every row: ``rows * top`` pairs plus
        half a tile of padding an expert, against ``rows * experts``.  ``LLB_MOE_GROUPED=always|never`` in the environment
        overrides the rule (for comparisons)."""
        if not (self.GROUPED and self.w_down_rows is not None and ops.has_tcgen05()):
            return False
        forced = os.environ.get("LLB_MOE_GROUPED", "")
        if forced in ("always", "never"):
            return forced == "always"
        return rows >= self.GROUPED_MIN_ROWS or rows * self.top + 64 * self.num_experts < rows * self.num_experts

    def _forward_pairs(self, x, residual, routed) -> None:
        T = x.shape[0]
        ids, weights, _, idw, _ = routed
        pairs = T * self.top
        act = torch.empty((pairs, self.intermediate_size), dtype=x.dtype, device=x.device)
        y = torch.empty((pairs, self.hidden_size), dtype=torch.float32, device=x.device)
        ops.moe_pairs(x, ids, self.w_gate_up, self.w_down_rows, act, y, glu=self.glu)
        ops.moe_combine(y, self._iota[:pairs], weights, residual, x if idw is not None else None, idw)

    def _forward_grouped(self, x, residual, routed) -> None:
        T, E, I, D = x.shape[0], self.num_experts, self.intermediate_size, self.hidden_size
        ids, weights, _, idw, _ = routed
        tiles = ops.moe_sorted_tiles(T * self.top, E)
        rows = tiles * ops.MOE_TILE_ROWS
        slot = torch.empty(T * self.top, dtype=torch.int32, device=x.device)
        tile_group = torch.empty(tiles, dtype=torch.int32, device=x.device)
        ops.moe_sort(ids, E, slot, tile_group)
        xs = torch.empty((rows, D), dtype=x.dtype, device=x.device)          # padding rows keep what the memory held:
        ops.moe_gather(x, slot, self.top, xs)                               # a row's result depends on that row alone
        act = torch.empty((rows, I), dtype=x.dtype, device=x.device)
        ops.gemm_tcgen05_grouped(xs, self.w_gate_up, act, ops.EPI_SWIGLU, E, tile_group, glu=self.glu)
        y = torch.empty((rows, D), dtype=torch.float32, device=x.device)
        ops.gemm_tcgen05_grouped(act, self.w_down_rows, y, ops.EPI_STORE_F32, E, tile_group)
        ops.moe_combine(y, slot, weights, residual, x if idw is not None else None, idw)

    def forward(self, x, residual, ctx=None) -> None:
        if isinstance(x, LazyNorm):
            x = x.materialize()
        routed = self.route(x)
        if self.shared is not None:
            self._forward_shared(x, residual, routed[4])
        idw = routed[3]
        if self.num_experts == 0:
            ops.moe_combine(None, None, None, residual, x, idw)
            return
        if x.dtype == torch.bfloat16 and self.w_down_rows is not None and self.GROUPED and \
                x.shape[0] * self.top < self.num_experts and os.environ.get("LLB_MOE_GROUPED", "") != "never":
            self._forward_pairs(x, residual, routed)
            return
        if x.dtype == torch.bfloat16 and self.grouped_pays(x.shape[0]):
            self._forward_grouped(x, residual, routed)
            return
        act = L.linear(x, self.w_gate_up, None, L.SWIGLU, glu=self.glu)           # [T, E * I]
        ops.moe_scale(act, routed[2], self.num_experts, self.intermediate_size)
        L.linear(act, self.w_down, None, L.RESIDUAL, residual=residual)
        if idw is not None:
            ops.moe_combine(None, None, None, residual, x, idw)


register_part("ffn", "routed_experts", RoutedExperts)
