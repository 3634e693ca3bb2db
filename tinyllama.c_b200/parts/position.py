"""Position encodings of the attention mixer.

Rotary, split-half ("NEOX") form: for pair i of the first r dims of a head,
theta_i = 1/base^(2i/r), angle = position * theta_i, (a, b) = (x[i], x[i + r/2]) ->
(a cos - b sin, a sin + b cos); dims past r are copied (CodeClaper/tinyllama.c
cpu_op.c:637-651).  The reference recomputes powf/cosf/sinf per element; here the
inverse frequencies are a table built once in 64-bit and rounded to 32-bit, and the
angle is the 32-bit product with the integer position.  A rotation is described to the
mixer by its table: the kernels that store keys and values (and single-token attention)
rotate by themselves.  "none" rotates nothing.  Any other encoding of positions in q and k
is a Position part with a transform() of its own (see parts/base.py).
"""
from __future__ import annotations

from typing import Optional

import torch

from .base import Position, register_position


@register_position("rope_neox")
class RotaryNeox(Position):
    def __init__(self, head_dim: int, theta: float, rope_dim: Optional[int] = None):
        self.head_dim = int(head_dim)
        self.rope_dim = int(rope_dim) if rope_dim else self.head_dim      # falcon_h1.c:265
        if self.rope_dim % 2 or self.rope_dim > self.head_dim:
            raise ValueError(f"rotary width {self.rope_dim} must be even and at most head_dim {self.head_dim}")
        self.theta = float(theta)
        self.inv_freq: Optional[torch.Tensor] = None

    def bind(self, tensors, dtype, device) -> None:
        i = torch.arange(self.rope_dim // 2, dtype=torch.float64)
        inv = 1.0 / torch.pow(torch.tensor(self.theta, dtype=torch.float64), 2.0 * i / self.rope_dim)
        self.inv_freq = inv.to(torch.float32).to(device).contiguous()

    def rotation_table(self) -> torch.Tensor:
        """The inverse frequencies (float32 [rope_dim/2]) for the kernels, which rotate by themselves."""
        return self.inv_freq


@register_position("none")
class NoPosition(RotaryNeox):
    """No position encoding: queries and keys are stored as projected."""

    def __init__(self, head_dim: int):
        super().__init__(head_dim, 10000.0, head_dim)

    def bind(self, tensors, dtype, device) -> None:
        self.inv_freq = torch.zeros(0, dtype=torch.float32, device=device)
