"""Grouped-query attention mixer over the paged key/value cache.

CodeClaper/tinyllama.c: q/k/v projections with optional biases (falcon_h1.c:315-330),
rotation of q and k (falcon_h1.c:332-333), K/V write-through and causal attention with
kv head h/(H/KV), scale 1/sqrt(head_dim) and an optional window (cpu_op.c:964-1064;
graph.c:1275), output projection (falcon_h1.c:338).  The multipliers on the input, the
keys and the output have no counterpart there; they fold into the projections.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from ... import ops
from ..base import KVRequest, LayerCache, Part, PartSpec, StepInfo, WeightSpec, act_empty, register_mixer, scratch_buf
from ..linear import StackedLinear


@register_mixer("attention")
class AttentionMixer(Part):
    def __init__(self, hidden: int, n_heads: int, n_kv_heads: int, head_dim: int, prefix: str,
                 position: PartSpec, bias: bool = False, window: Optional[int] = None, in_scale: float = 1.0,
                 out_scale: float = 1.0, key_scale: float = 1.0, cache_key: str = "kv"):
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} heads are not a multiple of {n_kv_heads} key/value heads")
        if not (1 <= int(head_dim) <= ops.MAX_HEAD_DIM):
            raise ValueError(f"attention: head size {head_dim} is outside what the kernels are built for "
                             f"(1..{ops.MAX_HEAD_DIM})")
        if int(n_heads) > ops.MAX_HEADS:
            raise ValueError(f"attention: {n_heads} heads exceed the kernels' limit of {ops.MAX_HEADS}")
        self.hidden, self.H, self.KV, self.hd = int(hidden), int(n_heads), int(n_kv_heads), int(head_dim)
        self.window = int(window) if window else None
        self.cache_key = cache_key
        self.position = position.build()
        b = (lambda n: prefix + n + ".bias") if bias else (lambda n: None)
        self.qkv = StackedLinear(hidden)
        self.q_off = self.qkv.add(prefix + "q_proj.weight", self.H * self.hd, b("q_proj"), in_scale)
        self.k_off = self.qkv.add(prefix + "k_proj.weight", self.KV * self.hd, b("k_proj"), in_scale, key_scale)
        self.v_off = self.qkv.add(prefix + "v_proj.weight", self.KV * self.hd, b("v_proj"), in_scale)
        self.o = StackedLinear(self.H * self.hd)
        self.o.add(prefix + "o_proj.weight", hidden, b("o_proj"), 1.0, out_scale)
        self.dtype = None

    @property
    def single_token_launches(self) -> int:
        """Kernels that mix() launches in a one-token step: one where the fused kernel serves (a
        bfloat16 cache, a head size it is built for, a position part with a rotation table), else
        rotation + split keys + merge."""
        fused = self.dtype == torch.bfloat16 and self.position.rotation_table() is not None \
            and ops.library().tlc_attention_decode_fused_ok(self.H, self.KV, self.hd) \
            and not ops.DISABLE_FUSED_DECODE_ATTENTION
        return 1 if fused else 3

    def weight_specs(self) -> List[WeightSpec]:
        return self.qkv.weight_specs() + self.o.weight_specs() + self.position.weight_specs()

    def cache_requests(self) -> list:
        return [KVRequest(self.cache_key, self.KV, self.hd, self.window)]

    def bind(self, tensors: Dict[str, torch.Tensor], dtype, device) -> None:
        self.dtype = dtype
        self.qkv.bind(tensors, dtype, device)
        self.o.bind(tensors, dtype, device)
        self.position.bind(tensors, dtype, device)
        self._no_rotation = torch.zeros(0, dtype=torch.float32, device=device)
        # arrival counters of the one-kernel attention of single-token steps: this mixer's own, so that no other
        # mixer, model or stream ever shares them; made here, outside any stream capture
        self._arrivals = ops.new_arrival_counters(device) if torch.device(device).type == "cuda" else None

    def input_projection(self) -> StackedLinear:
        """What this mixer computes from the normed input before anything else (a block may stack
        the input projections of its mixers into one product)."""
        return self.qkv

    def forward(self, normed: torch.Tensor, step: StepInfo, cache: LayerCache, residual: torch.Tensor) -> None:
        qkv = act_empty((step.n_rows, self.qkv.out_features), normed, torch.float32)
        self.qkv.forward(normed, qkv)
        self.forward_projected(qkv, step, cache, residual)

    def forward_projected(self, qkv: torch.Tensor, step: StepInfo, cache: LayerCache, residual: torch.Tensor) -> None:
        """qkv: this mixer's input projection, float32 [T, q|k|v] (rows may be strided)."""
        self.output(self.mix(qkv, step, cache), residual)

    def output_projection(self) -> StackedLinear:
        """What turns mix()'s result into this mixer's share of the residual stream (a block may run
        the output projections of its mixers as one product over their results side by side)."""
        return self.o

    mix_takes_max_blocks = True    # mix() can bound how many SMs its prompt kernel holds

    def mix(self, qkv: torch.Tensor, step: StepInfo, cache: LayerCache, out: Optional[torch.Tensor] = None,
            max_blocks: int = 0) -> torch.Tensor:
        """Everything between the input projection and the output projection: [T, H*hd], written
        to `out` (rows may be strided) where one is given.  max_blocks > 0: the attention kernel of a prompt
        holds at most that many SMs (a block that runs another mixer beside this one leaves it the rest)."""
        T = step.n_rows
        kv = cache.kv[self.cache_key]
        table = self.position.rotation_table()
        if table is None:
            # not a rotation: the part changes q and k in place; what is stored below is its result
            self.position.transform(qkv, self.q_off, self.k_off, step, self.H, self.KV, self.hd)
            table = self._no_rotation
        if step.max_new == 1 and ops.attention_decode_fused_ok(qkv, self.dtype, self.H, self.KV, self.hd):
            # one token per sequence: rotation, store and attention in one kernel
            att = out if out is not None else scratch_buf(f"attention.{self.cache_key}.out", (T, self.H * self.hd), self.dtype, qkv.device)
            ops.attention_decode_fused(qkv, self.q_off, self.k_off, self.v_off, kv.k_pages, kv.v_pages, table,
                                       cache.writes, kv.block_table, step.positions, step.row_seq, step.slots, att,
                                       self.H, self.KV, self.hd, 1.0 / math.sqrt(self.hd), self.window or 0,
                                       step.max_context, self._arrivals)
            return att
        q = scratch_buf(f"attention.{self.cache_key}.q", (T, self.H * self.hd), self.dtype, qkv.device)
        ops.rope_kv_store(qkv, self.q_off, self.k_off, self.v_off, q, kv.k_pages, kv.v_pages, table, step.positions,
                          step.row_seq, step.slots, kv.block_table, self.H, self.KV, self.hd, cache.writes)
        att = out if out is not None else scratch_buf(f"attention.{self.cache_key}.out", (T, self.H * self.hd), self.dtype, qkv.device)
        ops.attention(q, kv.k_pages, kv.v_pages, kv.block_table, step.positions, step.row_seq, step.slots, att,
                      self.H, self.KV, self.hd, 1.0 / math.sqrt(self.hd), self.window or 0,
                      step.max_context if step.max_new == 1 else 0, step.cu_seqlens, step.start_pos, step.max_context,
                      max_blocks)
        return att

    def output(self, att: torch.Tensor, residual: torch.Tensor) -> None:
        """Adds the output projection of `att` into the residual stream."""
        self.o.forward(att, residual, accumulate=True)
