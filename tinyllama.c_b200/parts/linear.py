"""A projection y = (x W^T) * colscale + colbias, with the weights of several projections
stacked row-wise so that one matrix product serves them all.

The reference multiplies by one weight tensor per graph node (falcon_h1.c:315-317,
342-343, 383-386) and adds an optional bias as a separate node (falcon_h1.c:319-330).
Here the stacked rows, every constant multiplier and the bias are prepared once at
load time: y[:, n] = acc[n] * colscale[n] + colbias[n], where a scalar that multiplies
the input or the output and a per-row multiplier vector all fold into colscale, and
the bias times the output multiplier into colbias.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from .. import ops
from .base import WeightSpec


def matrix_dtype(stored: torch.dtype, run: torch.dtype) -> torch.dtype:
    """float32 runs use float32 weights; bfloat16 runs keep bfloat16 weights in bfloat16 and
    leave a matrix that was stored in 32-bit as it is."""
    if run == torch.float32 or stored == torch.float32:
        return torch.float32
    return torch.bfloat16


class StackedLinear:
    """Rows of several named weights (and optional biases) stacked into one projection."""

    def __init__(self, in_features: int):
        self.in_features = int(in_features)
        self.segments: List[dict] = []
        self.weight: Optional[torch.Tensor] = None
        self.colscale: Optional[torch.Tensor] = None
        self.colbias: Optional[torch.Tensor] = None

    def add(self, weight_name: str, rows: int, bias_name: Optional[str] = None, in_scale: float = 1.0,
            out_scale=1.0) -> int:
        """Adds `rows` output rows; returns their first column in the stacked output.
        y = ((x * in_scale) W^T + bias) * out_scale, out_scale a number or one value per row."""
        off = self.out_features
        self.segments.append(dict(w=weight_name, b=bias_name, rows=int(rows), in_scale=float(in_scale),
                                  out_scale=out_scale, off=off))
        return off

    @property
    def out_features(self) -> int:
        return sum(s["rows"] for s in self.segments)

    def weight_specs(self) -> List[WeightSpec]:
        specs = []
        for s in self.segments:
            specs.append(WeightSpec(s["w"], (s["rows"], self.in_features), "normal"))
            if s["b"]:
                specs.append(WeightSpec(s["b"], (s["rows"],), "normal"))
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor], dtype: torch.dtype, device) -> None:
        mats = [tensors[s["w"]] for s in self.segments]
        mdt = torch.bfloat16
        for m in mats:
            if matrix_dtype(m.dtype, dtype) == torch.float32:
                mdt = torch.float32
        if len(mats) == 1:
            self.weight = mats[0].to(device=device, dtype=mdt).contiguous()
        else:
            self.weight = torch.cat([m.to(device=device, dtype=mdt) for m in mats], dim=0).contiguous()
        scale = torch.ones(self.out_features, dtype=torch.float64)
        bias = torch.zeros(self.out_features, dtype=torch.float64)
        any_scale = any_bias = False
        for s in self.segments:
            sl = slice(s["off"], s["off"] + s["rows"])
            osc = s["out_scale"]
            osc = torch.as_tensor(osc, dtype=torch.float64) if not isinstance(osc, (int, float)) \
                else torch.full((s["rows"],), float(osc), dtype=torch.float64)
            scale[sl] = osc * s["in_scale"]
            if s["b"]:
                bias[sl] = tensors[s["b"]].to(torch.float64) * osc
                any_bias = True
            if bool((scale[sl] != 1.0).any()):
                any_scale = True
        self.colscale = scale.to(torch.float32).to(device) if any_scale else None
        self.colbias = bias.to(torch.float32).to(device) if any_bias else None

    def forward(self, x: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> torch.Tensor:
        # a part of a product fused along K keeps its weight as a column range of the fused matrix; used on
        # its own (a mixer outside its block) it multiplies by a dense copy
        w = self.weight if self.weight.is_contiguous() else self.weight.contiguous()
        ops.linear(x, w, out, self.colscale, self.colbias, accumulate)
        return out

    @staticmethod
    def fuse_bound(parts: Sequence["StackedLinear"]) -> Optional["StackedLinear"]:
        """One projection over the rows of several bound projections of the same input.  The
        parts then share the fused storage (their weights become row ranges of it).  None if
        the parts cannot share one product (different input widths or element types)."""
        if len(parts) < 2 or len({p.in_features for p in parts}) != 1 or len({p.weight.dtype for p in parts}) != 1:
            return None
        fused = StackedLinear(parts[0].in_features)
        dev = parts[0].weight.device
        fused.weight = torch.cat([p.weight for p in parts], dim=0).contiguous()
        ones = lambda n: torch.ones(n, dtype=torch.float32, device=dev)
        zeros = lambda n: torch.zeros(n, dtype=torch.float32, device=dev)
        if any(p.colscale is not None for p in parts):
            fused.colscale = torch.cat([p.colscale if p.colscale is not None else ones(p.out_features) for p in parts])
        if any(p.colbias is not None for p in parts):
            fused.colbias = torch.cat([p.colbias if p.colbias is not None else zeros(p.out_features) for p in parts])
        off = 0
        for p in parts:
            for seg in p.segments:
                fused.segments.append(dict(seg, off=off + seg["off"]))
            p.weight = fused.weight[off:off + p.out_features]          # the part's rows inside the fused storage
            off += p.out_features
        return fused

    @staticmethod
    def fuse_bound_inputs(parts: Sequence["StackedLinear"], can_scale: Sequence[bool]):
        """One projection for several bound projections whose outputs are added together: their inputs lie
        side by side in one activation buffer and their weights side by side along K, so the sum forms
        in one accumulator.  The epilogue has one scale per output column, so the parts' scales must
        agree up to one number each, by which the part's input has to be multiplied instead
        (can_scale[i]: whoever fills part i's columns of the buffer can do that).  One part may be unable
        to: its scale becomes the epilogue's.  Biases add.  Returns (projection, factor per part), or
        None if the parts cannot share a product.  The parts' own weights become column ranges of the
        fused matrix."""
        if len(parts) < 2 or len({p.out_features for p in parts}) != 1 or len({p.weight.dtype for p in parts}) != 1:
            return None
        if any(p.in_features % 8 for p in parts):            # every part's columns start on a 16-byte boundary
            return None
        fixed = [i for i, ok in enumerate(can_scale) if not ok]
        if len(fixed) > 1:
            return None
        base = fixed[0] if fixed else 0
        dev, n = parts[0].weight.device, parts[0].out_features
        vec = lambda p: p.colscale if p.colscale is not None else torch.ones(n, dtype=torch.float32, device=dev)
        if bool((vec(parts[base]) == 0).any()):
            return None
        factors = []
        for i, p in enumerate(parts):
            r = vec(p).double() / vec(parts[base]).double()
            if float((r - r[0]).abs().max()) > 1e-6 * abs(float(r[0])):
                return None
            factors.append(1.0 if i == base else float(r[0]))
        fused = StackedLinear(sum(p.in_features for p in parts))
        fused.weight = torch.cat([p.weight for p in parts], dim=1).contiguous()
        fused.colscale = parts[base].colscale
        if any(p.colbias is not None for p in parts):
            fused.colbias = torch.stack([p.colbias for p in parts if p.colbias is not None]).double().sum(0).float()
        fused.segments = [dict(seg) for seg in parts[base].segments]      # the rows of the output (any part's)
        off = 0
        for p in parts:
            p.weight = fused.weight[:, off:off + p.in_features]          # the part's columns inside the fused storage
            off += p.in_features
        return fused, factors
