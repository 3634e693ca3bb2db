"""Dense gated feed-forward (SwiGLU).

d = W_down (silu(W_gate x) * (W_up x))  (CodeClaper/tinyllama.c falcon_h1.c:382-395).
The gate and up projections are stacked into one product.  The multiplier on the gate's
pre-activation, the one on the output, and the biases have no counterpart in the
reference.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .. import ops
from .base import Part, WeightSpec, act_empty, register_feed_forward, scratch_buf
from .linear import StackedLinear


@register_feed_forward("swiglu")
class SwiGLU(Part):
    def __init__(self, hidden: int, intermediate: int, prefix: str, bias: bool = False, gate_scale: float = 1.0,
                 down_scale: float = 1.0):
        self.hidden, self.F = int(hidden), int(intermediate)
        b = (lambda n: prefix + n + ".bias") if bias else (lambda n: None)
        self.gate_up = StackedLinear(hidden)
        self.gate_up.add(prefix + "gate_proj.weight", self.F, b("gate_proj"), 1.0, gate_scale)
        self.gate_up.add(prefix + "up_proj.weight", self.F, b("up_proj"))
        self.down = StackedLinear(self.F)
        self.down.add(prefix + "down_proj.weight", hidden, b("down_proj"), 1.0, down_scale)

    def weight_specs(self) -> List[WeightSpec]:
        return self.gate_up.weight_specs() + self.down.weight_specs()

    def bind(self, tensors: Dict[str, torch.Tensor], dtype, device) -> None:
        self.gate_up.bind(tensors, dtype, device)
        self.down.bind(tensors, dtype, device)
        # Rows regrouped as 8 gate rows followed by their 8 up rows, so that the product's epilogue
        # has a feature's gate and up side by side and writes silu(gate) * up directly.
        self.interleaved = self.F % 8 == 0
        if self.interleaved:
            F = self.F
            idx = torch.arange(2 * F, device=self.gate_up.weight.device).reshape(2, F // 8, 8).permute(1, 0, 2).reshape(-1)
            self.gate_up.weight = self.gate_up.weight[idx].contiguous()
            if self.gate_up.colscale is not None:
                self.gate_up.colscale = self.gate_up.colscale[idx].contiguous()
            if self.gate_up.colbias is not None:
                self.gate_up.colbias = self.gate_up.colbias[idx].contiguous()

    def forward(self, normed: torch.Tensor, residual: torch.Tensor) -> None:
        T = normed.shape[0]
        act = scratch_buf("swiglu.act", (T, self.F), normed.dtype, normed.device)
        if self.interleaved:
            ops.linear_swiglu(normed, self.gate_up.weight, act, self.gate_up.colscale, self.gate_up.colbias)
        else:
            gu = scratch_buf("swiglu.gate_up", (T, 2 * self.F), torch.float32, normed.device)
            self.gate_up.forward(normed, gu)
            ops.swiglu(gu, act)
        self.down.forward(act, residual, accumulate=True)

