"""Mamba2 (selective state-space) mixer with a per-sequence conv window and state.

CodeClaper/tinyllama.c: in_proj of width d_ssm + conv_dim + n_heads laid out
z | x | B | C | dt (falcon_h1.c:342-343; cpu_op.c:849, 865, 925-929); causal depthwise
convolution + SiLU over x|B|C with a window of d_conv-1 raw samples (cpu_op.c:836-889);
dt = softplus(dt + dt_bias), dA = exp(dt * A) with A = -exp(A_log) (cpu_op.c:933-934,
806-808); S = S*dA + B*(x*dt), y = S.C + x*D (cpu_op.c:939-951); gate by silu(z) and
grouped RMSNorm (cpu_op.c:950-958); out_proj (falcon_h1.c:367-368).  The reference keeps
one window and one state per layer for its single sequence (falcon_h1.c:136-147); here
they are fixed-size per-sequence cache entries.  The five multipliers on the in_proj
slices, the in/out multipliers, the projection biases and norm-before-gate have no
counterpart in the reference.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence

import torch

from ... import ops
from ..base import ChunkRequest, LayerCache, Part, StateRequest, StepInfo, WeightSpec, act_empty, register_mixer, scratch_buf, to_vec
from ..linear import StackedLinear


@register_mixer("mamba2")
class Mamba2Mixer(Part):
    single_token_launches = 3      # convolution, scan, gated norm: what a one-token step launches in mix()

    def __init__(self, hidden: int, d_ssm: int, n_heads: int, d_head: int, n_groups: int, d_state: int, d_conv: int,
                 prefix: str, eps: float, conv_bias: bool = True, proj_bias: bool = False, rms_norm: bool = True,
                 norm_before_gate: bool = False, slice_scales: Sequence[float] = (1.0,) * 5, in_scale: float = 1.0,
                 out_scale: float = 1.0, cache_key: str = "mamba", scan_chunk: int = ops.SSD_CHUNK):
        if n_heads * d_head != d_ssm or n_heads % n_groups or d_ssm % n_groups:
            raise ValueError("mamba2: n_heads*d_head must equal d_ssm and both be multiples of n_groups")
        if not (1 <= int(d_state) <= ops.MAX_STATE_SIZE):
            raise ValueError(f"mamba2: state size {d_state} is outside what the kernels are built for "
                             f"(1..{ops.MAX_STATE_SIZE})")
        if not (1 <= int(d_conv) <= ops.MAX_CONV_TAPS):
            raise ValueError(f"mamba2: {d_conv} convolution taps are outside what the kernels are built for "
                             f"(1..{ops.MAX_CONV_TAPS})")
        if int(n_heads) > ops.MAX_HEADS:
            raise ValueError(f"mamba2: {n_heads} heads exceed the kernels' limit of {ops.MAX_HEADS}")
        self.hidden, self.Di, self.Hs, self.P = int(hidden), int(d_ssm), int(n_heads), int(d_head)
        self.G, self.N, self.K = int(n_groups), int(d_state), int(d_conv)
        self.Cd = self.Di + 2 * self.G * self.N                      # falcon_h1.c:124
        self.eps, self.rms_norm, self.norm_before_gate = float(eps), bool(rms_norm), bool(norm_before_gate)
        self.prefix, self.cache_key = prefix, cache_key
        # rows of a chunk of the parallel scan of prompts: the result does not depend on it (the state is
        # linear in its initial value); the tensor-core form takes chunks of ops.SSD_CHUNK rows only
        self.scan_chunk = int(scan_chunk)
        if self.scan_chunk < 1:
            raise ValueError(f"mamba2: a scan chunk of {scan_chunk} rows")
        self.conv_bias = bool(conv_bias)
        mz, mx, mb, mc, mdt = [float(v) for v in slice_scales]
        rows = [mz] * self.Di + [mx] * self.Di + [mb] * (self.G * self.N) + [mc] * (self.G * self.N) + [mdt] * self.Hs
        self.in_proj = StackedLinear(hidden)
        self.in_proj.add(prefix + "in_proj.weight", self.Di + self.Cd + self.Hs,
                         prefix + "in_proj.bias" if proj_bias else None, in_scale, rows)
        self.out_proj = StackedLinear(self.Di)
        self.out_proj.add(prefix + "out_proj.weight", hidden, prefix + "out_proj.bias" if proj_bias else None,
                          1.0, out_scale)
        self.conv_w = self.conv_b = self.A = self.D = self.dt_bias = self.norm_w = None
        self.dtype = None

    # ---- declarations ------------------------------------------------------------------
    def weight_specs(self) -> List[WeightSpec]:
        p = self.prefix
        specs = self.in_proj.weight_specs() + self.out_proj.weight_specs()
        specs.append(WeightSpec(p + "conv1d.weight", (self.Cd, 1, self.K), "conv"))
        if self.conv_bias:
            specs.append(WeightSpec(p + "conv1d.bias", (self.Cd,), "normal"))
        specs += [WeightSpec(p + "A_log", (self.Hs,), "a_log"), WeightSpec(p + "D", (self.Hs,), "d_skip"),
                  WeightSpec(p + "dt_bias", (self.Hs,), "dt_bias")]
        if self.rms_norm:
            specs.append(WeightSpec(p + "norm.weight", (self.Di,), "ones"))
        return specs

    def cache_requests(self) -> list:
        return [StateRequest(self.cache_key + ".conv", (self.K - 1, self.Cd)),
                StateRequest(self.cache_key + ".ssm", (self.Hs, self.P, self.N))]

    # The row-by-row scan of a sequence takes 1 to 2 us a row and layer, more in a batch (a 128-token prompt of the
    # 1.5B sizes: 9.5 ms against 4.8 ms as one chunk in matrix form; 32 prompts of 128 tokens: 55 ms against 14.8;
    # 64 of 20 tokens: 20.4 against 11.8).  So the step's chunk table is asked for as soon as a sequence brings
    # more than CHUNKS_FROM_ROWS rows, and used when a sequence has more than 32 rows or the step has at least
    # 128: a few short sequences are quicker row by row (one prompt of 30 tokens: 4.0 ms against 4.5, the chunked
    # form's extra launches).
    CHUNKS_FROM_ROWS = 8
    CHUNKS_WORTH_ROWS, CHUNKS_WORTH_STEP = 32, 128

    def step_requests(self) -> list:
        return [ChunkRequest(self.scan_chunk, min(self.scan_chunk, self.CHUNKS_FROM_ROWS))]

    def bind(self, tensors: Dict[str, torch.Tensor], dtype, device) -> None:
        p = self.prefix
        self.dtype = dtype
        self.in_proj.bind(tensors, dtype, device)
        self.out_proj.bind(tensors, dtype, device)
        self.conv_w = to_vec(tensors[p + "conv1d.weight"].reshape(self.Cd, self.K), device)
        self.conv_b = to_vec(tensors[p + "conv1d.bias"], device) if self.conv_bias else None
        self.A = (-torch.exp(tensors[p + "A_log"].to(torch.float32))).to(device).contiguous()    # cpu_op.c:806-808
        self.D = to_vec(tensors[p + "D"], device)
        self.dt_bias = to_vec(tensors[p + "dt_bias"], device)
        self.norm_w = to_vec(tensors[p + "norm.weight"], device) if self.rms_norm else None

    # ---- one step --------------------------------------------------------------------------
    def input_projection(self) -> StackedLinear:
        return self.in_proj

    def forward(self, normed: torch.Tensor, step: StepInfo, cache: LayerCache, residual: torch.Tensor) -> None:
        proj = act_empty((step.n_rows, self.in_proj.out_features), normed, torch.float32)
        self.in_proj.forward(normed, proj)
        self.forward_projected(proj, step, cache, residual)

    def forward_projected(self, proj: torch.Tensor, step: StepInfo, cache: LayerCache, residual: torch.Tensor) -> None:
        """proj: this mixer's input projection, float32 [T, z|x|B|C|dt] (rows may be strided)."""
        self.output(self.mix(proj, step, cache), residual)

    def output_projection(self) -> StackedLinear:
        return self.out_proj

    mix_takes_scale = True         # mix() can multiply its result by a number on the way out
    mix_takes_join = True          # mix() calls `join` once, before its last kernel

    def mix(self, proj: torch.Tensor, step: StepInfo, cache: LayerCache, out: Optional[torch.Tensor] = None,
            out_scale: float = 1.0, join: Optional[Callable[[], None]] = None) -> torch.Tensor:
        """Everything between the input projection and the output projection: [T, d_ssm] times
        out_scale, written to `out` (rows may be strided) where one is given.  (A block that runs
        several output projections as one product moves a part of this one's multiplier here.)
        `join`, where given, is called once on the current stream before the last kernel: a block that runs
        other mixers on other streams waits for them there, where this stream waits for another one anyway
        (the scan's second stream), so that the kernel after this mixer follows its last one directly."""
        if not cache.writes:
            raise ValueError("mamba2: a recurrent mixer cannot run on another layer's cache without storing "
                             "(its window and state would advance twice in one step)")
        T, f32 = step.n_rows, torch.float32
        conv_state = cache.state[self.cache_key + ".conv"]
        ssm_state = cache.state[self.cache_key + ".ssm"]
        new = lambda tag, shape, dtype: scratch_buf(f"mamba2.{self.cache_key}.{tag}", shape, dtype, proj.device)   # (two mixers of a layer have two keys)
        # prompts cut into chunks of a bfloat16 run: the scan in matrix form, whose operands x|B|C the convolution
        # writes in bfloat16 at once; everything else scans 32-bit values
        chunks = step.chunks.get(self.scan_chunk)
        if chunks is not None and step.max_new <= self.CHUNKS_WORTH_ROWS and step.n_rows < self.CHUNKS_WORTH_STEP:
            chunks = None
        matrix_form = chunks is not None and self.dtype == torch.bfloat16 and self.scan_chunk <= ops.SSD_CHUNK \
            and ops.ssd_ok(self.Hs, self.P, self.N, self.G)
        xbc = new("xbc", (T, self.Cd), torch.bfloat16 if matrix_form else f32)
        dt, dA = new("dt", (T, self.Hs), f32), new("dA", (T, self.Hs), f32)
        ops.mamba_conv(proj, self.Di, self.Di + self.Cd, self.conv_w, self.conv_b, self.dt_bias, self.A, conv_state,
                       step.cu_seqlens, step.row_seq, step.slots, step.start_pos, xbc, dt, dA,
                       step.max_new == 1, self.dtype == torch.bfloat16,
                       len(step.host_start) == step.n_seqs and not any(step.host_start))
        y = new("y", (T, self.Di), f32)
        # in matrix form the outputs may come as two summands, the one that needs no state computed beside the walk
        # over the chunks; the gated norm adds them
        y_part = new("y_part", (T, self.Di), f32) if matrix_form else None
        in_two = ops.ssm_scan(xbc, dt, dA, self.D, ssm_state, step.cu_seqlens, step.slots, step.start_pos, y, self.Hs,
                              self.P, self.N, self.G, chunks, self.A if matrix_form else None, y_part)
        gated = out if out is not None else new("gated", (T, self.Di), self.dtype)
        if join is not None:
            join()
        ops.gated_rmsnorm(y, proj[:, :self.Di], self.norm_w, self.eps, self.G, self.norm_before_gate, gated,
                          out_scale, y_part if in_two else None)
        return gated

    def output(self, gated: torch.Tensor, residual: torch.Tensor) -> None:
        """Adds the output projection of `gated` into the residual stream."""
        self.out_proj.forward(gated, residual, accumulate=True)
