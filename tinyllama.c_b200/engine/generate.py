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

from ..cache import CacheError
from ..sampling.params import SamplingParams


@dataclass
class GenerationResult:
    prompt: List[int]
    tokens: List[int] = field(default_factory=list)
    finish_reason: str = ""              # "stop" | "length" | "context"
    uncached: int = 0                    # emitted tokens at the end that the model has not run yet (0 or 1)


@dataclass
class Continuation:
    """A request that goes on in a slot the caller holds (a further turn of a conversation, chat.c:296:
    history is never recomputed).  `history`: the tokens the slot's cache holds, in order (they count
    towards the context limit and the penalty window); `draws`: how many tokens were sampled for this
    sequence before (the sampler's draws are keyed by it).  The slot stays held when generation ends."""
    slot: int
    history: Sequence[int] = ()
    draws: int = 0


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
            out = self.decode_step(entries, histories, sequence_ids, steps)
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
        from .. import ops
        ops.check_errors()     # the tokens above were read after the step ran: a wait that ran out in it shows here
        return out

    MAX_GRAPHS = 24
    # A captured step is for one batch size, and capturing one costs 20 to 45 ms: requests that end at different times
    # would otherwise walk through every size on the way down (48 requests that stop at random: 190 steps, most of
    # them captures, 5.7 ms a step).  So a step of B sequences runs in the graph of the next size of `padded_batch`,
    # filled up with rows of a spare slot at position 0 (a token whose results nobody reads; its rows change no other
    # row's), while the cache has a slot and a page to spare.
    PAD_BATCHES = True

    @staticmethod
    def padded_batch(n: int) -> int:
        """The batch size whose graph serves n sequences: n up to 4, then multiples of 4 up to 16, then of 8."""
        if n <= 4:
            return n
        return (n + 3) // 4 * 4 if n <= 16 else (n + 7) // 8 * 8

    def decode_step(self, entries, histories=None, sequence_ids=None, steps=None) -> List[int]:
        """A one-token step of every entry through the captured graph of this batch size and context
        bucket (captured at first use): reserves the positions, uploads the step's integers, replays,
        reads the sampled tokens back, commits.  Generation and the benchmark both step through here."""
        from .. import ops
        from ..sampling.sampler import uniform
        from .decode_graph import DecodeGraph
        if histories is None:
            histories = [()] * len(entries)
        if sequence_ids is None:
            sequence_ids = list(range(len(entries)))
        if steps is None:
            steps = [0] * len(entries)
        B = len(entries)
        slots = [s for s, _ in entries]
        positions = [self.cache.reserve(s, 1) for s in slots]
        bucket = context_bucket(max(positions) + 1)
        n_graph, spare = B, None
        if self.PAD_BATCHES and self.padded_batch(B) > B and self.cache.slots.n_free > 0:
            spare = self.cache.acquire()
            try:
                self.cache.reserve(spare, 1)               # a page for the row it stores at position 0
                n_graph = self.padded_batch(B)
            except CacheError:
                self.cache.release(spare)
                spare = None
        try:
            key = (self.params, n_graph, bucket)
            g = self.graphs.get(key)
            if g is None:
                if len(self.graphs) >= self.MAX_GRAPHS:
                    self.graphs.pop(next(iter(self.graphs)))
                g = self.graphs[key] = DecodeGraph(self.model, self.cache, self.params, n_graph, bucket)
            self.cache.upload_tables()
            fill = n_graph - B
            u = [uniform(self.params.seed, i, t) for i, t in zip(sequence_ids, steps)] + [0.5] * fill if g.work is not None else None
            out = g.run(slots + [spare] * fill, [t[0] for _, t in entries] + [0] * fill, positions + [0] * fill, u,
                        list(histories) + [()] * fill)[:B]
        finally:
            if spare is not None:
                self.cache.release(spare)                  # (the step has run: the tokens were read back)
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
             ignore_eos: bool = False, continuations: Optional[Sequence[Optional[Continuation]]] = None,
             on_token=None) -> List[GenerationResult]:
    """Generates up to max_new_tokens for every prompt; returns results in the prompts' order.

    continuations[i], where given, makes request i go on in a slot the caller holds (see Continuation);
    on_token(i, token) is called for every emitted token as soon as it is known."""
    conts = list(continuations) if continuations is not None else [None] * len(prompts)
    if len(conts) != len(prompts):
        raise ValueError("one continuation (or None) per prompt")
    past = [list(c.history) if c is not None else [] for c in conts]
    for i, p in enumerate(prompts):
        if len(p) == 0:
            raise ValueError(f"prompt {i} is empty")
        if len(past[i]) + len(p) >= max_context:
            raise ValueError(f"prompt {i} has {len(past[i]) + len(p)} tokens, the context holds {max_context}")
    results = [GenerationResult(list(p)) for p in prompts]
    if max_new_tokens <= 0:
        for r in results:
            r.finish_reason = "length"
        return results
    stop = set() if ignore_eos else {int(s) for s in stop_ids}
    free_slots, free_pages = backend.capacity()
    if free_slots < 1 and any(c is None for c in conts):
        raise ValueError("no free sequence slot")
    # a request that continues a held slot already owns the pages of its history
    lens = [len(past[i]) % 64 + len(p) if conts[i] is not None else len(p) for i, p in enumerate(prompts)]
    n_held = sum(c is not None for c in conts)
    for batch in plan_batches(lens, max_new_tokens, max_batch, free_slots + n_held, free_pages, max_context):
        live = {i: (conts[i].slot if conts[i] is not None else backend.acquire()) for i in batch}    # request -> slot
        pending = {i: list(prompts[i]) for i in batch}                 # tokens the next step brings
        seen = {i: past[i] + results[i].prompt for i in batch}         # every token of the request so far: grows by one a step
        n_step = 0
        while live:
            order = sorted(live)
            entries = [(live[i], pending[i]) for i in order]
            histories = [seen[i] for i in order]
            draws = [n_step + (conts[i].draws if conts[i] is not None else 0) for i in order]
            nxt = backend.step_and_sample(entries, histories, order, draws)
            n_step += 1
            for i, tok in zip(order, nxt):
                r = results[i]
                if tok in stop:                                        # bench.c:218 -- not emitted
                    r.finish_reason = "stop"
                else:
                    r.tokens.append(int(tok))
                    seen[i].append(int(tok))
                    if on_token is not None:
                        on_token(i, int(tok))
                    if len(r.tokens) >= max_new_tokens:
                        r.finish_reason = "length"
                    elif len(past[i]) + len(r.prompt) + len(r.tokens) >= max_context:    # chat.c:332-335
                        r.finish_reason = "context"
                    r.uncached = 1 if r.finish_reason else 0
                if r.finish_reason:
                    slot = live.pop(i)
                    if conts[i] is None:
                        backend.release(slot)
                    pending.pop(i)
                else:
                    pending[i] = [int(tok)]
    return results
