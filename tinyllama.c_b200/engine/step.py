"""The step function: run the tokens a step brings, as one batch, from the cache.

CodeClaper/tinyllama.c's step is graph_execute(session, tokens, n): it appends n tokens
of the one sequence at the session's position, in chunks of n_ubatch, and returns the
logits of the last row (graph.c:1360-1421, 1282-1283).  Here a step carries several
sequences: each brings its next tokens (a whole prompt, a chunk of one, or a single
token), all are packed back to back into one batch without padding, every part reads
what came before from the sequence's cache slot, and logits come back for the rows that
were asked for.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import ops
from ..cache import Cache, CacheError
from ..models.model import Model
from ..parts.base import StepInfo


@dataclass
class StepEntry:
    """One sequence's share of a step: its slot, its next tokens, and the indices among
    these tokens whose logits are wanted."""
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()


class StepError(ValueError):
    pass


def chunk_table(lens: Sequence[int], rows: int, from_rows: Optional[int] = None):
    """Cuts sequences of `lens` new rows, packed back to back, into chunks of at most `rows` rows:
    (first packed row of every chunk + the total [n+1], sequence of every chunk [n], first chunk of every
    sequence [B+1]); None when no sequence has more than `from_rows` rows (a chunk's length unless given)."""
    if not any(n > (rows if from_rows is None else from_rows) for n in lens):
        return None
    seg_start, seg_seq, seq_seg_start, t0 = [], [], [0], 0
    for b, n in enumerate(lens):
        for off in range(0, n, rows):
            seg_start.append(t0 + off)
            seg_seq.append(b)
        seq_seg_start.append(len(seg_seq))
        t0 += n
    seg_start.append(t0)
    return seg_start, seg_seq, seq_seg_start


def pack(entries: Sequence[StepEntry], starts: Sequence[int], vocab: int, device,
         chunk_rows: Sequence[int] = (), chunk_from: Optional[dict] = None) -> Tuple[StepInfo, torch.Tensor, int]:
    """Host lists -> one int32 buffer (pinned for a GPU) -> one copy to the device -> StepInfo views.
    Returns (step, packed rows whose logits are wanted, their count).  chunk_rows: the chunk lengths
    that parts of the model asked for (ChunkRequest); the step gets one table for each.  chunk_from: for a chunk
    length, the number of rows a sequence must exceed for its table to be made (the length itself unless given).

    The GPU waits while this runs (a prompt step starts with it), so rows are filled as arrays, not one by one."""
    B = len(entries)
    lens = [len(e.tokens) for e in entries]
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    T = cu[-1]
    want_rows: List[int] = []
    for b, e in enumerate(entries):
        for w in e.want:
            if not (0 <= int(w) < lens[b]):
                raise StepError(f"wanted index {w} is outside this step's {lens[b]} tokens")
            want_rows.append(cu[b] + int(w))
    W = len(want_rows)
    tables = {int(r): chunk_table(lens, int(r), (chunk_from or {}).get(int(r))) for r in sorted(set(chunk_rows))}
    tail: List[int] = cu + [e.slot for e in entries] + [int(s) for s in starts] + want_rows
    for tab in tables.values():
        if tab is not None:
            tail += tab[0] + tab[1] + tab[2]
    on_gpu = torch.device(device).type == "cuda"
    host = torch.empty(3 * T + len(tail), dtype=torch.int32, pin_memory=on_gpu)
    flat = host.numpy()
    for b, (e, start) in enumerate(zip(entries, starts)):
        n, o = lens[b], cu[b]
        try:
            ids = np.asarray(e.tokens, dtype=np.int64).reshape(-1)
        except (TypeError, ValueError, OverflowError):
            ids = np.asarray([int(t) for t in e.tokens], dtype=np.int64)
        bad = np.flatnonzero((ids < 0) | (ids >= vocab))
        if bad.size:
            raise StepError(f"token id {int(ids[bad[0]])} is outside the vocabulary 0..{vocab - 1}")
        flat[o:o + n] = ids
        flat[T + o:T + o + n] = np.arange(start, start + n, dtype=np.int64)
        flat[2 * T + o:2 * T + o + n] = b
    flat[3 * T:] = tail
    dev = host.to(device, non_blocking=True) if on_gpu else host
    o = 0

    def take(n):
        nonlocal o
        v = dev[o:o + n]
        o += n
        return v

    step = StepInfo(n_rows=T, n_seqs=B, tokens=take(T), positions=take(T), row_seq=take(T), cu_seqlens=take(B + 1),
                    slots=take(B), start_pos=take(B), max_new=max(lens) if lens else 0,
                    max_context=max((s + n for s, n in zip(starts, lens)), default=0),
                    host_lens=tuple(lens), host_start=tuple(starts), host_slots=tuple(e.slot for e in entries))
    want = take(W)
    for rows, tab in tables.items():
        step.chunks[rows] = None if tab is None else (take(len(tab[0])), take(len(tab[1])), take(len(tab[2])))
    return step, want, W


def step(model: Model, cache: Cache, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
    """Runs one step; returns float32 logits [n_wanted, vocab] on the device in the order of
    the entries and of their ``want`` lists (None when nothing is wanted).

    The slots of the entries must be held (Cache.acquire) and distinct.  Nothing is launched
    before every entry has been checked and its pages reserved."""
    entries = [e for e in entries]
    if not entries:
        return None
    if len({e.slot for e in entries}) != len(entries):
        raise StepError("a step names the same sequence slot twice")
    for e in entries:
        if len(e.tokens) == 0:
            raise StepError("a step entry brings no tokens")
    starts = [cache.reserve(e.slot, len(e.tokens)) for e in entries]
    info, want_rows, n_want = pack(entries, starts, model.vocab, model.device, model.chunk_rows,
                                   getattr(model, "chunk_from", None))
    cache.upload_tables()
    logits = model.forward(info, cache, want_rows if n_want else None)
    for e in entries:
        cache.commit(e.slot, len(e.tokens))
    ops.check_errors()        # a kernel that gave up on a bounded wait (this or an earlier step); does not synchronise
    return logits
