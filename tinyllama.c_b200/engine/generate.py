"""The generation loop: batches of unequal prompts, stop tokens, sequences that end early.

CodeClaper/tinyllama.c: prefill the prompt, sample, then while the token is not the stop
token and the budget lasts: emit it, run it as a one-token step, sample again
(bench.c:201-241, chat.c:296-339); generation also ends when the context is full
(chat.c:332-335).  The stop token is not emitted.  Here the same loop runs over a batch:
the prompts of a batch go through one step together, then every live sequence advances
one token per step; a sequence that ends gives its slot back at once and the others go on;
requests beyond one batch run as further batches that reuse the slots.

The loop decides on the host and talks to the model through a small backend (acquire,
step, sample, release), so its decisions can be tested without a GPU.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

from ..sampling.params import SamplingParams


@dataclass
class GenerationResult:
    prompt: List[int]
    tokens: List[int] = field(default_factory=list)
    finish_reason: str = ""              # "stop" | "length" | "context"


class EngineBackend:
    """The real backend: the model, its cache and the GPU sampler."""

    def __init__(self, model, cache, params: SamplingParams, graphs: Optional[dict] = None, use_graphs: bool = True,
                 max_step_tokens: int = 8192):
        from ..sampling.sampler import Sampler
        self.model, self.cache, self.params = model, cache, params
        self.sampler = Sampler(params, model.device)
        self.graphs = graphs if graphs is not None else {}        # (params, batch size) -> DecodeGraph
        self.use_graphs = use_graphs and model.device.type == "cuda"
        self.max_step_tokens = max(1, int(max_step_tokens))      # the reference's n_ubatch (graph.c:1397-1412)
        self.stats = dict(prefill_s=0.0, prefill_tokens=0, decode_s=0.0, decode_steps=0, decode_tokens=0,
                          h2d_bytes=0, d2h_bytes=0)

    def acquire(self) -> int:
        return self.cache.acquire()

    def release(self, slot: int) -> None:
        self.cache.release(slot)

    def capacity(self):
        """(free sequence slots, free pages of 64 positions)."""
        free_pages = min((g.pool.n_free for g in self.cache.kv_groups), default=1 << 30)
        return self.cache.slots.n_free, free_pages

    def step_and_sample(self, entries, histories, sequence_ids, steps) -> List[int]:
        """entries: (slot, tokens) pairs; logits are taken at each entry's last token.
        Returns the next token of every entry (host integers)."""
        import time
        from ..sampling.sampler import uniform
        from .step import StepEntry, step
        t0 = time.perf_counter()
        decode = all(len(t) == 1 for _, t in entries)
        if decode and self.use_graphs:
            out = self._graph_step(entries, histories, sequence_ids, steps, uniform)
        else:
            out = self._prompt_steps(entries, histories, sequence_ids, steps)
        dt = time.perf_counter() - t0
        n = sum(len(t) for _, t in entries)
        if decode:
            self.stats["decode_s"] += dt
            self.stats["decode_steps"] += 1
            self.stats["decode_tokens"] += n
        else:
            self.stats["prefill_s"] += dt
            self.stats["prefill_tokens"] += n
        return out

    def _prompt_steps(self, entries, histories, sequence_ids, steps) -> List[int]:
        """Prompts in steps of at most max_step_tokens tokens: whole prompts while they fit, a
        longer one in pieces that continue from the cache; the next token of an entry is
        sampled in the step that brings its last piece."""
        from .step import StepEntry, step
        done = [0] * len(entries)
        out: List[Optional[int]] = [None] * len(entries)
        i = 0
        while i < len(entries):
            budget, batch, finished = self.max_step_tokens, [], []
            j = i
            while j < len(entries) and budget > 0:
                slot, toks = entries[j]
                piece = toks[done[j]:done[j] + budget]
                done[j] += len(piece)
                budget -= len(piece)
                last = done[j] == len(toks)
                batch.append(StepEntry(slot, piece, (len(piece) - 1,) if last else ()))
                if not last:
                    break
                finished.append(j)
                j += 1
            logits = step(self.model, self.cache, batch)
            if finished:
                toks = self.sampler.sample(logits, [histories[k] for k in finished], [sequence_ids[k] for k in finished],
                                           [steps[k] for k in finished]).cpu().tolist()
                for k, t in zip(finished, toks):
                    out[k] = t
            i = j
        return out

    MAX_GRAPHS = 24

    def _graph_step(self, entries, histories, sequence_ids, steps, uniform) -> List[int]:
        """A one-token step through the captured graph of this batch size."""
        from .. import ops
        from .decode_graph import DecodeGraph
        B = len(entries)
        slots = [s for s, _ in entries]
        positions = [self.cache.reserve(s, 1) for s in slots]
        bucket = context_bucket(max(positions) + 1)
        key = (self.params, B, bucket)
        g = self.graphs.get(key)
        if g is None:
            if len(self.graphs) >= self.MAX_GRAPHS:
                self.graphs.pop(next(iter(self.graphs)))
            g = self.graphs[key] = DecodeGraph(self.model, self.cache, self.params, B, bucket)
        self.cache.upload_tables()
        u = [uniform(self.params.seed, i, t) for i, t in zip(sequence_ids, steps)] if g.work is not None else None
        out = g.run(slots, [t[0] for _, t in entries], positions, u, histories)
        for s in slots:
            self.cache.commit(s, 1)
        ops.check_errors()
        self.stats["h2d_bytes"] += g.h2d_bytes
        self.stats["d2h_bytes"] += g.d2h_bytes
        return out


def context_bucket(n: int) -> int:
    """Sequence lengths share a captured graph up to the next power of two (at least 512)."""
    b = 512
    while b < n:
        b *= 2
    return b


def plan_batches(prompt_lens: Sequence[int], max_new_tokens: int, max_batch: int, free_slots: int,
                 free_pages: int, max_context: int) -> List[List[int]]:
    """Splits requests, in order, into batches that fit the cache: at most max_batch and
    free_slots sequences, and pages for every sequence grown to its longest possible length."""
    batches, cur, cur_pages = [], [], 0
    for i, n in enumerate(prompt_lens):
        need = (min(n + max_new_tokens, max_context) + 63) // 64
        if need > free_pages:
            raise ValueError(f"request {i} needs {need} cache pages, only {free_pages} exist")
        if cur and (len(cur) >= min(max_batch, free_slots) or cur_pages + need > free_pages):
            batches.append(cur)
            cur, cur_pages = [], 0
        cur.append(i)
        cur_pages += need
    if cur:
        batches.append(cur)
    return batches


def generate(backend, prompts: Sequence[Sequence[int]], max_new_tokens: int = 128,
             stop_ids: Sequence[int] = (), max_batch: int = 64, max_context: int = 1 << 30,
             ignore_eos: bool = False) -> List[GenerationResult]:
    """Generates up to max_new_tokens for every prompt; returns results in the prompts' order."""
    for i, p in enumerate(prompts):
        if len(p) == 0:
            raise ValueError(f"prompt {i} is empty")
        if len(p) >= max_context:
            raise ValueError(f"prompt {i} has {len(p)} tokens, the context holds {max_context}")
    results = [GenerationResult(list(p)) for p in prompts]
    if max_new_tokens <= 0:
        for r in results:
            r.finish_reason = "length"
        return results
    stop = set() if ignore_eos else {int(s) for s in stop_ids}
    free_slots, free_pages = backend.capacity()
    if free_slots < 1:
        raise ValueError("no free sequence slot")
    for batch in plan_batches([len(p) for p in prompts], max_new_tokens, max_batch, free_slots, free_pages,
                              max_context):
        live = {i: backend.acquire() for i in batch}                   # request -> slot
        pending = {i: list(prompts[i]) for i in batch}                 # tokens the next step brings
        n_step = 0
        while live:
            order = sorted(live)
            entries = [(live[i], pending[i]) for i in order]
            histories = [results[i].prompt + results[i].tokens for i in order]
            nxt = backend.step_and_sample(entries, histories, order, [n_step] * len(order))
            n_step += 1
            for i, tok in zip(order, nxt):
                r = results[i]
                if tok in stop:                                        # bench.c:218 -- not emitted
                    r.finish_reason = "stop"
                else:
                    r.tokens.append(int(tok))
                    if len(r.tokens) >= max_new_tokens:
                        r.finish_reason = "length"
                    elif len(r.prompt) + len(r.tokens) >= max_context:    # chat.c:332-335
                        r.finish_reason = "context"
                if r.finish_reason:
                    backend.release(live.pop(i))
                    pending.pop(i)
                else:
                    pending[i] = [int(tok)]
    return results
