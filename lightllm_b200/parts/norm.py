"""RMSNorm of the float32 residual stream."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config import register_part
from ..csrc import ops
from ..weights import WeightSpec
from .base import Norm


class RMSNorm(Norm):
    """``y = x / sqrt(mean(x^2) + eps) * weight`` with the statistics in float32
    (src/ops/norm.cu:19-23,48-54).  ``weight_name`` is appended to ``prefix`` with a dot (an empty one makes the prefix
    itself the weight's name).  ``one_plus``: the checkpoint stores the weight around zero and the norm multiplies by
    ``1 + w``; the sum is made once, in float32, when the model is bound."""

    graph_safe = True

    def __init__(self, prefix: str, hidden_size: int, eps: float, weight_name: str = "weight", one_plus: bool = False):
        self.name = (f"{prefix}.{weight_name}" if weight_name else prefix) if prefix else weight_name
        self.hidden_size = hidden_size
        self.eps = float(eps)
        self.one_plus = bool(one_plus)
        self.weight = None
        self.out_dtype = torch.float32

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.name, (self.hidden_size,), init=("normal", 0.1) if self.one_plus else ("one_plus_normal", 0.01))]

    def bind(self, tensors: Dict[str, torch.Tensor], dtype, device) -> None:
        self.weight = tensors[self.name]
        if self.one_plus:
            self.weight = (1.0 + self.weight.float()).contiguous()
        self.out_dtype = dtype

    def rms_parameters(self):
        """(weight, eps) for kernels that fold this norm into their prologue."""
        return self.weight, self.eps

    def forward(self, residual, ctx=None, dtype=None):
        """``dtype``: the output's dtype when it is not the compute dtype (float32 for a reader that filters the normed
        stream before anything rounds it)."""
        out = torch.empty(residual.shape, dtype=dtype or self.out_dtype, device=residual.device)
        ops.rmsnorm(residual, self.weight, self.eps, out)
        return out

    def forward_rows(self, residual, rows, ctx=None):
        out = torch.empty((rows.numel(), self.hidden_size), dtype=self.out_dtype, device=residual.device)
        ops.rmsnorm(residual, self.weight, self.eps, out, rows=rows)
        return out


class LayerNorm(Norm):
    """``y = (x - mean) / sqrt(var + eps) * weight + bias`` with ``var`` the mean of the squared deviations, all in
    float32.  ``weight_name`` / ``bias_name`` are appended to ``prefix`` with a dot; an empty ``weight_name`` makes the
    prefix itself the weight's name; ``bias_name=None`` is a layer norm without a bias.  As a norm on a branch's output (``h += LN(branch)``) the sum is one kernel and
    stays float32 (:meth:`add_into`)."""

    graph_safe = True
    copies_stream = True          # add_into can leave the updated stream in bfloat16 as well

    def __init__(self, prefix: str, hidden_size: int, eps: float, weight_name: str = "weight",
                 bias_name: Optional[str] = "bias"):
        join = lambda tail: f"{prefix}.{tail}" if prefix and tail else (prefix or tail)
        self.name, self.bias_name = join(weight_name), (None if bias_name is None else join(bias_name))
        self.hidden_size = hidden_size
        self.eps = float(eps)
        self.weight = self.bias = None
        self.out_dtype = torch.float32

    def weight_specs(self) -> List[WeightSpec]:
        specs = [WeightSpec(self.name, (self.hidden_size,), init=("one_plus_normal", 0.1))]
        if self.bias_name is not None:
            specs.append(WeightSpec(self.bias_name, (self.hidden_size,), init=("normal", 0.1)))
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor], dtype, device) -> None:
        self.weight = tensors[self.name]
        self.bias = tensors[self.bias_name] if self.bias_name is not None else None
        if self.bias is not None and self.weight.dtype != self.bias.dtype:
            self.weight, self.bias = self.weight.float(), self.bias.float()
        self.out_dtype = dtype

    def forward(self, residual, ctx=None):
        out = torch.empty(residual.shape, dtype=self.out_dtype, device=residual.device)
        ops.layernorm(residual, self.weight, self.bias, self.eps, out)
        return out

    def forward_rows(self, residual, rows, ctx=None):
        out = torch.empty((rows.numel(), self.hidden_size), dtype=self.out_dtype, device=residual.device)
        ops.layernorm(residual, self.weight, self.bias, self.eps, out, rows=rows)
        return out

    def add_into(self, branch, residual, ctx=None, copy=None) -> None:
        """``residual += LN(branch)``, both float32: the normed branch is never rounded to the compute dtype.
        ``copy`` (bfloat16) receives the updated stream as well, for the projections of the next branch."""
        ops.layernorm(branch, self.weight, self.bias, self.eps, residual, accumulate=True, copy=copy)


register_part("norm", "rmsnorm", RMSNorm)
register_part("norm", "layernorm", LayerNorm)
