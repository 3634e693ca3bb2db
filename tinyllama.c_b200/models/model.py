"""A model: embedding, layers, the order they run in, final norm, output head.

CodeClaper/tinyllama.c's architecture file builds one static node list per model
(falcon_h1.c:256-417) and the executor walks it (graph.c:1278-1302), evaluating the
output head for the last row only (graph.c:1282-1283).  Here the walk is over
``schedule``, a list of (layer, cache) pairs that is data of the model, and the head
runs on the rows whose logits are wanted.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from .. import ops
from ..parts.base import (ChunkRequest, LayerCache, LayerRun, LayerSpec, Part, PartSpec, StateRequest, StepInfo, WeightSpec,
                          step_scratch)
from ..parts.block import Block
from ..parts.linear import StackedLinear, matrix_dtype


class Model:
    def __init__(self, config, layer_specs: Sequence[LayerSpec], schedule: Optional[Sequence[LayerRun]],
                 final_norm: PartSpec, embed_name: str, head_name: Optional[str], vocab: int, hidden: int,
                 embed_scale: float = 1.0, head_scale: float = 1.0):
        self.config = config
        self.vocab, self.hidden = int(vocab), int(hidden)
        self.layers: List[Block] = [Block(s) for s in layer_specs]
        self.schedule: List[LayerRun] = list(schedule) if schedule is not None \
            else [LayerRun(i) for i in range(len(self.layers))]
        for r, run in enumerate(self.schedule):
            if not (0 <= run.layer < len(self.layers)):
                raise ValueError(f"run-order entry {r} names layer {run.layer}, which does not exist")
            if run.cache is not None and not (0 <= run.cache < len(self.schedule) and self.schedule[run.cache].cache is None):
                raise ValueError(f"run-order entry {r} reads the cache of entry {run.cache}, which has none of its own")
            if run.cache is not None and any(isinstance(q, StateRequest) for q in self.layers[run.layer].cache_requests()):
                raise ValueError(f"run-order entry {r} reads the cache of entry {run.cache} but layer {run.layer} has a "
                                 f"mixer with state of its own: only keys and values can be read without storing")
        # chunk lengths that parts want the step function to cut sequences into (one table each, every step)
        # as (rows, from how many rows of a sequence the table is wanted): the smallest threshold asked for a length
        asked: Dict[int, int] = {}
        for layer in self.layers:
            for q in layer.step_requests():
                if isinstance(q, ChunkRequest):
                    start = q.rows if q.from_rows is None else min(q.rows, q.from_rows)
                    asked[q.rows] = min(asked.get(q.rows, start), start)
        self.chunk_rows = tuple(sorted(asked))
        self.chunk_from = dict(asked)               # chunk length -> rows a sequence must exceed for the table to be made
        self.final_norm = final_norm.build()
        self.embed_name, self.head_name = embed_name, head_name            # head_name None: tied (core.c:1246-1249)
        self.embed_scale = float(embed_scale)
        self.head = StackedLinear(hidden)
        self.head.add(head_name or embed_name, vocab, None, 1.0, head_scale)
        self.embed_table: Optional[torch.Tensor] = None
        self.dtype: Optional[torch.dtype] = None
        self.device: Optional[torch.device] = None

    # ---- declarations ----------------------------------------------------------------------
    def weight_specs(self) -> List[WeightSpec]:
        specs = [WeightSpec(self.embed_name, (self.vocab, self.hidden), "normal")]
        if self.head_name:
            specs.append(WeightSpec(self.head_name, (self.vocab, self.hidden), "normal"))
        for layer in self.layers:
            specs += layer.weight_specs()
        specs += self.final_norm.weight_specs()
        seen, out = set(), []
        for s in specs:
            if s.name not in seen:
                seen.add(s.name)
                out.append(s)
        return out

    def cache_requests(self) -> Dict[int, list]:
        """Cache needs per entry of the run order that owns a cache (key: its index)."""
        return {r: self.layers[run.layer].cache_requests() for r, run in enumerate(self.schedule) if run.cache is None}

    def bind(self, tensors: Dict[str, torch.Tensor], dtype: torch.dtype, device) -> None:
        self.dtype, self.device = dtype, torch.device(device)
        for layer in self.layers:
            layer.bind(tensors, dtype, device)
        self.final_norm.bind(tensors, dtype, device)
        emb = tensors[self.embed_name]
        self.embed_table = emb.to(device=device, dtype=matrix_dtype(emb.dtype, dtype)).contiguous()
        if self.head_name is None:
            self.head.bind({self.embed_name: self.embed_table}, dtype, device)     # shares the table's storage
        else:
            self.head.bind(tensors, dtype, device)

    # ---- forward ------------------------------------------------------------------------------
    def forward(self, step: StepInfo, cache, want_rows: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """Runs the step's rows through every scheduled layer; returns float32 logits
        [n_wanted, vocab] for the packed rows in want_rows (None: no logits).

        The embedding is the step's first kernel and is launched with a full dependency on everything
        before it on the stream: kernels of this step may therefore fetch, ahead of their own dependency
        wait, what earlier steps left in the cache (never what a kernel of this step writes)."""
        x = torch.empty((step.n_rows, self.hidden), dtype=torch.float32, device=self.device)
        ops.embed(step.tokens, self.embed_table, self.embed_scale, x)
        with step_scratch(step):                       # the layers share the step's temporaries
            for r, run in enumerate(self.schedule):
                self.layers[run.layer].forward(x, step, cache.layer_view(r if run.cache is None else run.cache, run.writes))
        if want_rows is None or want_rows.numel() == 0:
            return None
        n = want_rows.numel()
        normed = torch.empty((n, self.hidden), dtype=self.dtype, device=self.device)
        self.final_norm.forward(x, normed, want_rows)
        logits = torch.empty((n, self.vocab), dtype=torch.float32, device=self.device)
        self.head.forward(normed, logits)
        return logits
