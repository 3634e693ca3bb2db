"""One-token steps replayed from a CUDA graph.

A decode step of a small batch is a few hundred short kernels; launched one by one from
the host they leave the GPU idle most of the time.  The reference has no such problem to
solve (one process-wide lock, default stream, graph.c:1340-1350).  Here the step for a
given number of sequences is captured once -- embedding, every layer, final norm, head
and the sampler -- over fixed device buffers; a later step copies its few integers
(tokens, positions, slots) into those buffers with one host-to-device copy and replays the
graph.  Kernels read lengths and pages from device memory, so a replay is valid for any
contents of the buffers.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Sequence

import torch

from .. import ops
from ..parts.base import StepInfo
from ..sampling.params import SamplingParams




class DecodeGraph:
    """The captured one-token step of `n` sequences."""

    def __init__(self, model, cache, params: SamplingParams, n: int, max_context: int):
        """max_context: no sequence may be longer than this after a replayed step (it sizes the
        grid of the attention kernel, which is fixed in the graph)."""
        self.model, self.cache, self.params, self.n = model, cache, params, int(n)
        self.max_context = int(max_context)
        dev = model.device
        B = self.n
        # one int32 buffer: tokens | positions | slots | start_pos   (variable per step)
        self.ibuf = torch.zeros(4 * B, dtype=torch.int32, device=dev)
        self.ihost = torch.zeros(4 * B, dtype=torch.int32).pin_memory()
        ar = torch.arange(B + 1, dtype=torch.int32, device=dev)
        self.info = StepInfo(n_rows=B, n_seqs=B, tokens=self.ibuf[0:B], positions=self.ibuf[B:2 * B],
                             row_seq=ar[:B].contiguous(), cu_seqlens=ar, slots=self.ibuf[2 * B:3 * B],
                             start_pos=self.ibuf[3 * B:4 * B], max_new=1, max_context=self.max_context)
        self.want = ar[:B].contiguous()
        self.uniforms = torch.zeros(B, dtype=torch.float32, device=dev)
        self.uhost = torch.zeros(B, dtype=torch.float32).pin_memory()
        nh = params.repeat_last_n if params.has_penalties else 0
        self.history = torch.full((B, max(nh, 1)), -1, dtype=torch.int32, device=dev) if nh else None
        self.hhost = torch.full((B, max(nh, 1)), -1, dtype=torch.int32).pin_memory() if nh else None
        self.work = torch.empty(B * model.vocab, dtype=torch.float32, device=dev) \
            if not (params.is_greedy and not params.has_penalties) else None
        self.out = torch.zeros(B, dtype=torch.int32, device=dev)
        self.argmax_work = ops.new_argmax_work(B, dev) if dev.type == "cuda" else None
        self.out_host = torch.zeros(B, dtype=torch.int32).pin_memory()
        self.logits: Optional[torch.Tensor] = None
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.launches = 0

    def _body(self) -> None:
        p = self.params
        self.logits = self.model.forward(self.info, self.cache, self.want)
        if p.is_greedy and not p.has_penalties:
            ops.argmax(self.logits, self.out, self.argmax_work)
        else:
            ops.sample(self.logits, self.work, self.history, self.uniforms, p.temperature, p.top_k, p.top_p, p.min_p,
                       p.repeat_penalty, p.frequency_penalty, p.presence_penalty, self.out)

    def capture(self) -> None:
        """Runs the step once eagerly on throw-away inputs that touch no live sequence's cache
        (slot and page 0 may be live, so the run is on a scratch copy of nothing: it reads and
        writes only what the buffers name, and the buffers name the sequences of the first real
        step), then captures it."""
        before = ops.launch_count()
        stream = torch.cuda.Stream(device=self.model.device)
        stream.wait_stream(torch.cuda.current_stream())
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            with torch.cuda.graph(self.graph, stream=stream):
                self._body()
        torch.cuda.current_stream().wait_stream(stream)
        self.launches = ops.launch_count() - before

    def run(self, slots: Sequence[int], tokens: Sequence[int], positions: Sequence[int],
            uniforms: Optional[Sequence[float]] = None, histories: Optional[Sequence[Sequence[int]]] = None) -> List[int]:
        B = self.n
        if max(positions) + 1 > self.max_context:
            raise ValueError(f"a sequence of {max(positions) + 1} positions does not fit this graph's {self.max_context}")
        h = self.ihost
        h[0:B] = torch.tensor(tokens, dtype=torch.int32)
        h[B:2 * B] = torch.tensor(positions, dtype=torch.int32)
        h[2 * B:3 * B] = torch.tensor(slots, dtype=torch.int32)
        h[3 * B:4 * B] = h[B:2 * B]
        self.ibuf.copy_(h, non_blocking=True)
        if self.work is not None and uniforms is not None:
            self.uhost.copy_(torch.tensor(uniforms, dtype=torch.float32))
            self.uniforms.copy_(self.uhost, non_blocking=True)
        if self.history is not None and histories is not None:
            n = self.history.shape[1]
            hh = self.hhost.numpy()                  # (a row at a time through torch costs 8 us a row: 0.5 ms at batch 64)
            hh.fill(-1)
            for r, hist in enumerate(histories):
                tail = hist[-n:] if isinstance(hist, (list, tuple)) else list(hist)[-n:]
                if tail:
                    hh[r, :len(tail)] = tail
            self.history.copy_(self.hhost, non_blocking=True)
        if self.graph is None:
            self.capture()          # the capture itself does not execute; the replay below does
        self.graph.replay()
        ops.count_launches(self.launches)
        self.out_host.copy_(self.out, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return self.out_host.tolist()

    @property
    def h2d_bytes(self) -> int:
        n = self.ibuf.numel() * 4
        if self.work is not None:
            n += self.uniforms.numel() * 4
        if self.history is not None:
            n += self.history.numel() * 4
        return n

    @property
    def d2h_bytes(self) -> int:
        return self.out.numel() * 4
