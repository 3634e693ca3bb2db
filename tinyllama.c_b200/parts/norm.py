"""RMSNorm over the 32-bit residual stream.

o = x * 1/sqrt(mean(x^2) + eps) * w  (CodeClaper/tinyllama.c cpu_op.c:44-64, applied per
row at cpu_op.c:526-533).  The reference fixes eps at 1e-6 (def.h:10); here it is a
parameter.  Statistics are 32-bit; the output takes the activation type.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import ops
from .base import Part, WeightSpec, register_norm, to_vec


@register_norm("rmsnorm")
class RMSNorm(Part):
    def __init__(self, width: int, eps: float, weight_name: str):
        self.width, self.eps, self.weight_name = int(width), float(eps), weight_name
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.weight_name, (self.width,), "ones")]

    def bind(self, tensors: Dict[str, torch.Tensor], dtype, device) -> None:
        self.weight = to_vec(tensors[self.weight_name], device)

    def forward(self, x32: torch.Tensor, out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        ops.rmsnorm(x32, self.weight, self.eps, out, rows)
        return out
