"""What a part of a layer is: its weights, its cache needs, its forward call.

CodeClaper/tinyllama.c composes a model from graph builders (graph.h:51-78) that an
architecture file calls in order (falcon_h1.c:256-417), and lets an op own recurrent
state through ``graph_state`` (graph.c:343-357).  Here the same roles are classes: a
part is built from sizes and constants only (it never sees the model's name), declares
its tensors as ``WeightSpec`` and its per-sequence storage as ``KVRequest`` /
``StateRequest``, and is looked up by kind in a registry, so that a configuration can
choose a different mixer or feed-forward for every layer.

Interfaces
----------
Norm          forward(x32 [R, D] float32, out [R, D], rows=None)
Position      rotation_table() -> inverse frequencies (the kernels rotate q and k themselves), or None and
              transform(qkv, q_off, k_off, step, n_heads, n_kv, head_dim): changes the q and k columns of
              the 32-bit projection in place; storing keys and values is the mixer's business
Mixer         forward(normed [T, D], step, cache, residual [T, D] float32)  adds its output into residual
FeedForward   forward(normed [T, D], residual [T, D] float32)               adds its output into residual
All of them   weight_specs() -> [WeightSpec], bind(tensors, dtype, device)
Mixers also   cache_requests() -> [KVRequest | StateRequest], step_requests() -> [ChunkRequest]
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch


# ---- weights ----------------------------------------------------------------------------
@dataclass(frozen=True)
class WeightSpec:
    """One named tensor of a part.  ``init`` tells the random-weights mode how to draw it:
    normal | ones | zeros | a_log | dt_bias | d_skip."""
    name: str
    shape: Tuple[int, ...]
    init: str = "normal"


# ---- cache needs --------------------------------------------------------------------------
@dataclass(frozen=True)
class KVRequest:
    """Keys and values for every position of a sequence (or the last ``window`` of them)."""
    key: str
    kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateRequest:
    """A fixed-size tensor per sequence, zero for a sequence at position 0."""
    key: str
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass(frozen=True)
class ChunkRequest:
    """A table, built by the step function for every step, that cuts each sequence's new rows into
    chunks of at most ``rows`` rows (a recurrent mixer scans chunks in parallel and carries the state
    between them).  The mixer finds it as ``step.chunks[rows]``: None when no sequence of the step brings
    more than ``from_rows`` rows (a chunk's length unless given: a mixer whose chunked form already pays for
    shorter sequences says from how many rows), else (first row of every chunk [n+1], sequence of every chunk
    [n], first chunk of every sequence [B+1]), int32 on the device."""
    rows: int
    from_rows: Optional[int] = None


# ---- what a step gives every part ------------------------------------------------------------
@dataclass
class StepInfo:
    """The packed batch of one step, on the device (all int32).

    Row t of the packed activations belongs to sequence ``row_seq[t]`` of this step, whose
    cache slot is ``slots[b]``; its absolute position is ``positions[t]``; sequence b owns
    rows ``cu_seqlens[b] : cu_seqlens[b+1]`` and began this step at ``start_pos[b]``."""
    n_rows: int
    n_seqs: int
    tokens: torch.Tensor
    positions: torch.Tensor
    row_seq: torch.Tensor
    cu_seqlens: torch.Tensor
    slots: torch.Tensor
    start_pos: torch.Tensor
    max_new: int = 0            # longest run of new tokens among the sequences
    max_context: int = 0        # longest sequence after this step
    # host copies for parts that plan on the host
    host_lens: Tuple[int, ...] = ()
    host_start: Tuple[int, ...] = ()
    host_slots: Tuple[int, ...] = ()
    # one table per chunk length that a part asked for with a ChunkRequest (see there)
    chunks: Dict[int, Optional[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]]] = field(default_factory=dict)
    # the step's temporaries (see scratch_buf)
    scratch: Dict = field(default_factory=dict)


@dataclass
class KVView:
    """One layer's pages of a key/value group: [n_pages, kv_heads, 64, head_dim] each, and the
    group's block table [n_slots, max_pages] (page index of every 64 positions of a slot)."""
    k_pages: torch.Tensor
    v_pages: torch.Tensor
    block_table: torch.Tensor
    window: Optional[int] = None


@dataclass
class LayerCache:
    """What one entry of the layer schedule sees of the cache."""
    kv: Dict[str, KVView] = field(default_factory=dict)
    state: Dict[str, torch.Tensor] = field(default_factory=dict)     # [n_slots, *shape]
    writes: bool = True      # False: the layer reads another layer's cache and must not store into it


class Part:
    """Base of norms, position encodings, mixers and feed-forwards."""

    def weight_specs(self) -> List[WeightSpec]:
        return []

    def bind(self, tensors: Dict[str, torch.Tensor], dtype: torch.dtype, device: torch.device) -> None:
        pass

    def cache_requests(self) -> list:
        return []

    def step_requests(self) -> list:
        """What the step function must prepare for this part in every step (ChunkRequest)."""
        return []


class Position(Part):
    """Base of position encodings of an attention mixer.  A part answers one of two ways:

    * ``rotation_table()`` returns inverse frequencies (float32 [r/2], r <= head_dim; an empty tensor
      rotates nothing): q and k are rotated split-half by angle = position * frequency inside the
      kernels that store keys and values, and single-token attention does all of it in one kernel;
    * it returns None and ``transform(qkv, q_off, k_off, step, n_heads, n_kv, head_dim)`` changes the q
      columns [q_off, q_off + n_heads*head_dim) and the k columns of the 32-bit projection ``qkv``
      [T, *] in place, in whatever way it likes (``step.positions`` holds the rows' positions); the
      mixer then stores keys and values and attends.  A part that leaves q and k alone does nothing."""

    def rotation_table(self) -> Optional[torch.Tensor]:
        return None

    def transform(self, qkv: torch.Tensor, q_off: int, k_off: int, step: "StepInfo", n_heads: int, n_kv: int,
                  head_dim: int) -> None:
        pass


# ---- registries -------------------------------------------------------------------------------
_REGISTRIES: Dict[str, Dict[str, Callable[..., Part]]] = {
    "norm": {}, "position": {}, "mixer": {}, "feed_forward": {}}


def _register(kind: str, name: str):
    def deco(cls):
        _REGISTRIES[kind][name] = cls
        return cls
    return deco


def register_norm(name: str):
    return _register("norm", name)


def register_position(name: str):
    return _register("position", name)


def register_mixer(name: str):
    return _register("mixer", name)


def register_feed_forward(name: str):
    return _register("feed_forward", name)


@dataclass(frozen=True)
class PartSpec:
    """A part chosen by a configuration: registry kind, registered name, constructor arguments."""
    kind: str
    name: str
    params: Dict[str, Any] = field(default_factory=dict)

    def build(self) -> Part:
        reg = _REGISTRIES.get(self.kind)
        if reg is None or self.name not in reg:
            known = sorted(reg) if reg is not None else sorted(_REGISTRIES)
            raise KeyError(f"no {self.kind} named '{self.name}' is registered; known: {known}")
        return reg[self.name](**self.params)


@dataclass(frozen=True)
class LayerSpec:
    """One layer as data: pre-mixer norm, mixers that run in parallel on the normed input and
    add into the residual stream, pre-feed-forward norm, feed-forward."""
    mixer_norm: PartSpec
    mixers: Tuple[PartSpec, ...]
    ffn_norm: Optional[PartSpec]
    ffn: Optional[PartSpec]


@dataclass(frozen=True)
class LayerRun:
    """One entry of the order in which layers run.  ``layer`` indexes the model's layers and
    may repeat (the weights are shared; every entry has a cache of its own, so a sequence's
    state is the same whether its tokens come at once or one by one).  ``cache`` names another
    entry of the run order (by its index) whose cache this entry reads instead, without
    storing into it."""
    layer: int
    cache: Optional[int] = None

    @property
    def writes(self) -> bool:
        return self.cache is None


def to_vec(t: torch.Tensor, device) -> torch.Tensor:
    """Small per-channel tensors are used as float32 by every kernel (an exact widening)."""
    return t.to(device=device, dtype=torch.float32).contiguous()


def act_empty(shape, like: torch.Tensor, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """Uninitialised activation buffer on `like`'s device (its type unless `dtype` is given)."""
    return torch.empty(shape, dtype=dtype or like.dtype, device=like.device)


# A step's temporaries.  Every layer needs the same dozen buffers (normed rows, projections, the scan's outputs,
# ...) and an allocation costs some 3 us of host time, which is what short prompts are made of.  While a model
# runs a step (Model.forward enters `step_scratch`), `scratch_buf` hands out one buffer per (tag, shape, type)
# and the next layer gets the same one.  That is safe for the reason the allocator's own reuse is: a buffer's
# next writer is launched on the model's stream after everything that read it (kernels of side streams are
# waited for before the layer's output projection), and a kernel writes only after its wait on its predecessor.
# Two buffers that are alive at the same time carry different tags.  The buffers go when the step's StepInfo
# goes (a captured step keeps its StepInfo, and so its buffers, for as long as the graph lives).
_scratch: Optional[dict] = None


class step_scratch:
    """Context manager: temporaries asked for inside come from (and stay in) `step.scratch`."""

    def __init__(self, step: "StepInfo"):
        self.store = step.scratch

    def __enter__(self):
        global _scratch
        self.before, _scratch = _scratch, self.store
        return self

    def __exit__(self, *exc):
        global _scratch
        _scratch = self.before
        return False


def scratch_buf(tag: str, shape, dtype: torch.dtype, device) -> torch.Tensor:
    """An uninitialised buffer for a temporary of the running step; the same one for the same (tag, shape, type)
    until the step ends.  Outside a step it is a plain allocation."""
    if _scratch is None:
        return torch.empty(shape, dtype=dtype, device=device)
    key = (tag, tuple(shape), dtype)
    t = _scratch.get(key)
    if t is None:
        t = _scratch[key] = torch.empty(shape, dtype=dtype, device=device)
    return t
