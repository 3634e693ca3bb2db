"""A layer: norm -> mixers in parallel on the same normed input -> residual; norm ->
feed-forward -> residual.

CodeClaper/tinyllama.c falcon_h1.c:311-395: n = norm(x); x = (x + attn(n)) + ssm(n);
x = x + ffn(norm(x)).  The residual stream is 32-bit; each mixer and the feed-forward add
their output into it in the order they are listed.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional

import torch

from .base import LayerCache, LayerSpec, Part, StepInfo, WeightSpec, act_empty, scratch_buf
from .linear import StackedLinear


# Mixers that are independent of one another between their input and output projections run side by side on
# streams of their own.  One-token steps are chains of short kernels; in a prompt the walk over a sequence's chunks
# keeps a block on two SMs in three for most of its time, and the attention kernel's blocks, one to an SM, take the
# rest (2,048 tokens: 9.71 -> 9.31 ms).  TLC_PARALLEL_PROMPT_MIXERS=0 keeps prompts on one stream.
PARALLEL_MIXERS = bool(int(os.environ.get("TLC_PARALLEL_MIXERS", "1")))
_MAIN_MIXER = int(os.environ["TLC_MAIN_MIXER"]) if "TLC_MAIN_MIXER" in os.environ else None
FUSE_OUTPUTS = bool(int(os.environ.get("TLC_FUSE_OUTPUTS", "1")))
PARALLEL_PROMPT_MIXERS = bool(int(os.environ.get("TLC_PARALLEL_PROMPT_MIXERS", "1")))
# In a prompt the mixers' long kernels want an SM for each of their blocks.  One of a side stream that is resident
# first keeps the current stream's blocks waiting until its own have finished; a side mixer that can
# (mix_takes_max_blocks) may be told to hold at most this many SMs and to work through its tiles with them.
# 0: no bound, the default.  Measured at the 1.5B sizes (2,048 tokens; the walk over the chunks has 96 blocks,
# attention 128): with 48 the walk ends 12 us earlier (86 -> 143.5 us after the layer's start instead of 155.7),
# attention takes 53 us instead of 30, and the part of the scan that runs beside both finds no room and ends
# as late as the walk did before: 7.51 ms a step either way.  The three kernels fill the SMs between them.
PROMPT_SIDE_BLOCKS = int(os.environ.get("TLC_PROMPT_SIDE_BLOCKS", "0"))


_streams = {}


def _current_stream(device) -> "torch.cuda.Stream":
    """The current stream of the device as a torch object.  torch.cuda.current_stream() takes some 10 us of Python
    a call and a block asks once a layer, so the object is kept by the stream's handle (which torch's raw query
    gives in a fraction of that) and made anew only when the handle is a new one."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    raw = getattr(torch._C, "_cuda_getCurrentRawStream", None)
    if raw is None:
        return torch.cuda.current_stream(index)
    handle = raw(index)
    hit = _streams.get((index, handle))
    if hit is None:
        if len(_streams) > 64:
            _streams.clear()
        hit = _streams[(index, handle)] = torch.cuda.current_stream(index)
    return hit


class Block(Part):
    def __init__(self, spec: LayerSpec, act_dtype_of=None):
        self.spec = spec
        self.mixer_norm = spec.mixer_norm.build()
        self.mixers = [m.build() for m in spec.mixers]
        self.ffn_norm = spec.ffn_norm.build() if spec.ffn_norm is not None else None
        self.ffn = spec.ffn.build() if spec.ffn is not None else None
        self.dtype: Optional[torch.dtype] = None

    def parts(self) -> List[Part]:
        return [p for p in [self.mixer_norm, *self.mixers, self.ffn_norm, self.ffn] if p is not None]

    def weight_specs(self) -> List[WeightSpec]:
        return [s for p in self.parts() for s in p.weight_specs()]

    def cache_requests(self) -> list:
        return [r for m in self.mixers for r in m.cache_requests()]

    def step_requests(self) -> list:
        return [r for p in self.parts() for r in p.step_requests()]

    def bind(self, tensors: Dict[str, torch.Tensor], dtype, device) -> None:
        self.dtype = dtype
        for p in self.parts():
            p.bind(tensors, dtype, device)
        # Mixers that run in parallel on the same normed input and say what they first project it to
        # share one product: their input projections are stacked.  Any other mixer gets the normed
        # input as a tensor.
        self.fused_in, self.fused_offsets = None, []
        if len(self.mixers) > 1 and all(hasattr(m, "input_projection") and hasattr(m, "forward_projected")
                                        for m in self.mixers):
            projs = [m.input_projection() for m in self.mixers]
            self.fused_in = StackedLinear.fuse_bound(projs)
            off = 0
            for pr in projs:
                self.fused_offsets.append((off, pr.out_features))
                off += pr.out_features
        # Likewise their output projections, whose results are added into the residual stream: the mixers
        # write side by side into one buffer, and one product over the weights side by side along K forms
        # the sum in its accumulator.
        self.fused_out, self.out_offsets, self.out_scales = None, [], []
        if self.fused_in is not None and FUSE_OUTPUTS and all(hasattr(m, "output_projection") and hasattr(m, "mix")
                                                              for m in self.mixers):
            outs = [m.output_projection() for m in self.mixers]
            fused = StackedLinear.fuse_bound_inputs(outs, [bool(getattr(m, "mix_takes_scale", False)) for m in self.mixers])
            if fused is not None:
                self.fused_out, self.out_scales = fused
                off = 0
                for pr in outs:
                    self.out_offsets.append((off, pr.in_features))
                    off += pr.in_features

    def _mix_in_parallel(self, parts, step: StepInfo, cache: LayerCache, x32: torch.Tensor) -> None:
        """One mixer runs on the current stream, every other on a side stream that starts after the
        shared input projection.  Output projections add into the residual stream one after the
        other on the current stream, in the mixers' order, each after its mixer has finished.  (Under stream capture the
        side streams become parallel branches of the graph.)"""
        main = _current_stream(x32.device)
        if not hasattr(self, "_side"):
            self._side = [torch.cuda.Stream(device=x32.device) for _ in self.mixers[1:]]
            # events are made once: a record overwrites the event's last state, and every wait of this block follows
            # its record in program order
            self._fork = torch.cuda.Event()
            self._done = [torch.cuda.Event() for _ in self.mixers]
        # the mixer with the longest chain of kernels stays on the current stream, where every
        # kernel follows its predecessor by a programmatic edge
        lengths = [int(getattr(m, "single_token_launches", 1)) for m in self.mixers]
        here = _MAIN_MIXER if _MAIN_MIXER is not None else lengths.index(max(lengths))
        fork = self._fork
        fork.record(main)
        acts, done = [None] * len(self.mixers), [None] * len(self.mixers)
        joint, views = self._joint_activations(x32)
        sides = iter(self._side)
        for i, (m, part) in enumerate(zip(self.mixers, parts)):
            if i == here:
                continue
            side = next(sides)
            side.wait_event(fork)
            torch.cuda.set_stream(side)              # (the context manager asks for the current stream again: 10 us)
            try:
                bound = PROMPT_SIDE_BLOCKS if step.max_new > 1 and getattr(m, "mix_takes_max_blocks", False) else 0
                acts[i] = self._mix(i, part, step, cache, views[i], max_blocks=bound)
                done[i] = self._done[i]
                done[i].record(side)
            finally:
                torch.cuda.set_stream(main)
        # The wait for the side streams breaks the chain of programmatic launches on this stream.  A mixer that
        # offers to (mix_takes_join) places it before its own last kernel; otherwise it comes after the mixer.
        joined = []

        def join():
            if not joined:
                joined.append(True)
                for ev in done:
                    if ev is not None:
                        main.wait_event(ev)

        early = getattr(self.mixers[here], "mix_takes_join", False)
        acts[here] = self._mix(here, parts[here], step, cache, views[here], join if early else None)
        join()
        for i, m in enumerate(self.mixers):          # outputs in the mixers' order, whatever ran where
            if joint is None:
                m.output(acts[i], x32)
        if joint is not None:
            self.fused_out.forward(joint, x32, accumulate=True)

    def _mix(self, i: int, part: torch.Tensor, step: StepInfo, cache: LayerCache, view: Optional[torch.Tensor], join=None,
             max_blocks: int = 0):
        """Mixer i between its projections; into its columns of the joint buffer, scaled, where there is one."""
        m = self.mixers[i]
        more = {} if join is None else {"join": join}
        if max_blocks:
            more["max_blocks"] = max_blocks
        if view is None:
            return m.mix(part, step, cache, **more)
        if self.out_scales[i] != 1.0:
            return m.mix(part, step, cache, view, self.out_scales[i], **more)
        return m.mix(part, step, cache, view, **more)

    def _joint_activations(self, x32: torch.Tensor):
        """The buffer that the mixers fill side by side for the shared output projection, and each
        mixer's columns of it; (None, Nones) without a shared output projection."""
        if self.fused_out is None:
            return None, [None] * len(self.mixers)
        joint = scratch_buf("block.joint", (x32.shape[0], self.fused_out.in_features), self.dtype, x32.device)
        return joint, [joint[:, off:off + n] for off, n in self.out_offsets]

    def forward(self, x32: torch.Tensor, step: StepInfo, cache: LayerCache) -> None:
        """Updates the float32 residual stream x32 [T, D] in place."""
        if self.mixers:
            normed = scratch_buf("block.normed", x32.shape, self.dtype, x32.device)
            self.mixer_norm.forward(x32, normed)
            if self.fused_in is not None:
                proj = scratch_buf("block.proj", (x32.shape[0], self.fused_in.out_features), torch.float32, x32.device)
                self.fused_in.forward(normed, proj)
                parts = [proj[:, off:off + n] for off, n in self.fused_offsets]
                if (step.max_new == 1 or PARALLEL_PROMPT_MIXERS) and x32.is_cuda and PARALLEL_MIXERS and all(hasattr(m, "mix") for m in self.mixers):
                    self._mix_in_parallel(parts, step, cache, x32)
                elif self.fused_out is not None:
                    joint, views = self._joint_activations(x32)
                    for i, (part, view) in enumerate(zip(parts, views)):
                        self._mix(i, part, step, cache, view)
                    self.fused_out.forward(joint, x32, accumulate=True)
                else:
                    for m, part in zip(self.mixers, parts):
                        m.forward_projected(part, step, cache, x32)
            else:
                for m in self.mixers:
                    m.forward(normed, step, cache, x32)
        if self.ffn is not None:
            normed = scratch_buf("block.ffn_normed", x32.shape, self.dtype, x32.device)
            self.ffn_norm.forward(x32, normed)
            self.ffn.forward(normed, x32)
