"""Picks the next token of every sequence of a batch on the GPU.

The reference's sample_token works on one logits row on the host with a thread-local
xorshift generator (sampler.c:11-24, 107-257).  Here a batch of rows is handled by one
kernel launch; the uniform number of a draw is a hash of (seed, sequence id, step), so a
sequence's tokens do not depend on which other sequences share its batch.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from .. import ops
from .params import SamplingParams

_M = (1 << 64) - 1


def uniform(seed: int, sequence: int, step: int) -> float:
    """A number in [0, 1) with 24 random bits, a pure function of its arguments (splitmix64)."""
    x = (seed * 0x9E3779B97F4A7C15 + sequence * 0xBF58476D1CE4E5B9 + step * 0x94D049BB133111EB + 0x2545F4914F6CDD1D) & _M
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _M
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _M
    x ^= x >> 31
    return (x >> 40) / float(1 << 24)


class Sampler:
    def __init__(self, params: SamplingParams, device):
        self.params = params
        self.device = torch.device(device)
        self._work: Optional[torch.Tensor] = None

    def sample(self, logits: torch.Tensor, histories: Optional[Sequence[Sequence[int]]] = None,
               sequence_ids: Optional[Sequence[int]] = None, steps: Optional[Sequence[int]] = None) -> torch.Tensor:
        """logits [R, V] float32 on the device -> int32 token ids [R] on the device.
        histories: the tokens of each row's sequence so far (for the penalties);
        sequence_ids / steps: what the draw of each row is keyed by."""
        p = self.params
        R, V = logits.shape
        out = torch.empty(R, dtype=torch.int32, device=logits.device)
        if p.is_greedy and not p.has_penalties:
            ops.argmax(logits, out)
            return out
        hist = None
        if p.has_penalties and histories is not None:
            n = p.repeat_last_n
            rows = []
            for h in histories:
                h = list(h)[-n:]
                rows.append(h + [-1] * (n - len(h)))
            hist = torch.tensor(rows, dtype=torch.int32).to(logits.device)
        seqs = list(sequence_ids) if sequence_ids is not None else list(range(R))
        stps = list(steps) if steps is not None else [0] * R
        u = torch.tensor([uniform(p.seed, s, t) for s, t in zip(seqs, stps)], dtype=torch.float32).to(logits.device)
        if self._work is None or self._work.numel() < R * V:
            self._work = torch.empty(R * V, dtype=torch.float32, device=logits.device)
        ops.sample(logits, self._work, hist, u, p.temperature, p.top_k, p.top_p, p.min_p, p.repeat_penalty,
                   p.frequency_penalty, p.presence_penalty, out)
        return out
