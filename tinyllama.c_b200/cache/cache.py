"""The cache: a slot per live sequence, paged keys and values per layer group, and
fixed-size per-sequence state.

CodeClaper/tinyllama.c allocates K and V as [kv_head][ctx][head_dim] float32 per layer,
only for layers that attend (graph.c:817-872), keeps recurrent buffers that ops register
one by one (graph.c:343-357; falcon_h1.c:136-147) and serves one sequence per session
(def.h:533-542).  Here:

* a *slot* belongs to one live sequence and records its length; slots are handed back
  when the sequence ends and reused by later ones;
* layers whose mixers ask for keys/values with the same (kv heads, head size, window) form
  a *group* with one page pool [layers, pages, kv heads, 64, head size] and one block
  table [slots, pages per slot]; a windowed group gives back pages that fell out of every
  future query's window;
* every fixed-size state request (same key and shape) forms a group [layers, slots, *shape];
  a sequence at position 0 is treated as all-zero by the kernels, so nothing is cleared
  on reuse.

Sizes come from the parts' requests, never from an architecture's name.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..parts.base import KVRequest, KVView, LayerCache, StateRequest
from .allocators import CacheError, IndexPool

PAGE = 64


def pages_for(n_tokens: int) -> int:
    return (int(n_tokens) + PAGE - 1) // PAGE


@dataclass
class _KVGroup:
    request: KVRequest
    layers: List[int]
    k: torch.Tensor                   # [n_layers, n_pages, KV, PAGE, hd]
    v: torch.Tensor
    table: torch.Tensor               # device [n_slots, max_pages] int32
    table_host: torch.Tensor          # pinned or plain CPU mirror
    pool: IndexPool
    pages_of: List[List[int]]         # per slot: page index per 64 positions (-1 = given back)
    dirty: set


@dataclass
class _StateGroup:
    request: StateRequest
    layers: List[int]
    data: torch.Tensor                # [n_layers, n_slots, *shape]


class Cache:
    def __init__(self, requests: Dict[int, list], max_tokens: int, max_seqs: int, dtype: torch.dtype, device,
                 max_pages_per_seq: Optional[int] = None):
        """requests: cache id (layer index) -> that layer's KVRequest / StateRequest list.
        max_tokens: positions that live sequences may hold together, each sequence rounded up
        to whole pages of 64; max_seqs: live sequences at any time."""
        self.device = torch.device(device)
        self.dtype = dtype
        self.n_pages = max(1, pages_for(max_tokens))
        self.max_seqs = max(1, int(max_seqs))
        self.max_pages_per_seq = int(max_pages_per_seq or self.n_pages)
        self.slots = IndexPool(self.max_seqs, "sequence slot")
        self.seq_len = [0] * self.max_seqs
        self.kv_groups: List[_KVGroup] = []
        self.state_groups: List[_StateGroup] = []
        self._kv_of: Dict[Tuple[int, str], Tuple[int, int]] = {}        # (cache id, key) -> (group, index in group)
        self._state_of: Dict[Tuple[int, str], Tuple[int, int]] = {}
        self._views: Dict[Tuple[int, bool], LayerCache] = {}
        pin = self.device.type == "cuda"
        for cid in sorted(requests):
            for req in requests[cid]:
                if isinstance(req, KVRequest):
                    sig = (req.kv_heads, req.head_dim, req.window)
                    gi = next((i for i, g in enumerate(self.kv_groups)
                               if (g.request.kv_heads, g.request.head_dim, g.request.window) == sig), None)
                    if gi is None:
                        self.kv_groups.append(_KVGroup(req, [], None, None, None, None,
                                                       IndexPool(self.n_pages, "cache page"),
                                                       [[] for _ in range(self.max_seqs)], set()))
                        gi = len(self.kv_groups) - 1
                    g = self.kv_groups[gi]
                    self._kv_of[(cid, req.key)] = (gi, len(g.layers))
                    g.layers.append(cid)
                elif isinstance(req, StateRequest):
                    sig = (req.key, tuple(req.shape), req.dtype)
                    gi = next((i for i, g in enumerate(self.state_groups)
                               if (g.request.key, tuple(g.request.shape), g.request.dtype) == sig), None)
                    if gi is None:
                        self.state_groups.append(_StateGroup(req, [], None))
                        gi = len(self.state_groups) - 1
                    g = self.state_groups[gi]
                    self._state_of[(cid, req.key)] = (gi, len(g.layers))
                    g.layers.append(cid)
                else:
                    raise CacheError(f"layer {cid}: unknown cache request {req!r}")
        for g in self.kv_groups:
            shape = (len(g.layers), self.n_pages, g.request.kv_heads, PAGE, g.request.head_dim)
            g.k = torch.zeros(shape, dtype=dtype, device=self.device)
            g.v = torch.zeros(shape, dtype=dtype, device=self.device)
            g.table = torch.zeros((self.max_seqs, self.max_pages_per_seq), dtype=torch.int32, device=self.device)
            g.table_host = torch.zeros((self.max_seqs, self.max_pages_per_seq), dtype=torch.int32,
                                       pin_memory=pin)
        for g in self.state_groups:
            g.data = torch.zeros((len(g.layers), self.max_seqs, *g.request.shape), dtype=g.request.dtype,
                                 device=self.device)

    # ---- sizes -----------------------------------------------------------------------------
    def bytes(self) -> int:
        n = 0
        for g in self.kv_groups:
            n += 2 * g.k.numel() * g.k.element_size()
        for g in self.state_groups:
            n += g.data.numel() * g.data.element_size()
        return n

    # ---- slots -----------------------------------------------------------------------------
    def acquire(self) -> int:
        """A free slot for a new sequence of length 0."""
        s = self.slots.alloc()
        self.seq_len[s] = 0
        return s

    def release(self, slot: int) -> None:
        """Gives back the slot and every page it holds."""
        self.slots.free(slot)                       # raises on a double free before anything changes
        for g in self.kv_groups:
            for p in g.pages_of[slot]:
                if p >= 0:
                    g.pool.free(p)
            g.pages_of[slot] = []
        self.seq_len[slot] = 0

    def length(self, slot: int) -> int:
        return self.seq_len[slot]

    def live_tokens(self) -> int:
        """Positions held now, each live sequence rounded up to whole pages."""
        return sum(pages_for(self.seq_len[s]) * PAGE for s in self.slots.held())

    # ---- per step ----------------------------------------------------------------------------
    def reserve(self, slot: int, n_new: int) -> int:
        """Makes room for n_new more positions of the slot's sequence; returns its start position."""
        if not self.slots._held[slot]:
            raise CacheError(f"sequence slot {slot} is not held")
        start = self.seq_len[slot]
        need = pages_for(start + n_new)
        if need > self.max_pages_per_seq:
            raise CacheError(f"a sequence of {start + n_new} positions needs {need} pages; "
                             f"the block table holds {self.max_pages_per_seq}")
        for g in self.kv_groups:
            have = g.pages_of[slot]
            if need > len(have):
                if need - len(have) > g.pool.n_free:
                    raise CacheError(f"cache is full: {need - len(have)} more pages needed for slot {slot}, "
                                     f"{g.pool.n_free} of {g.pool.n} free")
                first = len(have)
                fresh = [g.pool.alloc() for _ in range(first, need)]
                have.extend(fresh)
                g.table_host[slot, first:need] = torch.tensor(fresh, dtype=g.table_host.dtype)   # one write, not one a page
                g.dirty.add(slot)
        return start

    def commit(self, slot: int, n_new: int) -> None:
        """The step stored n_new positions; windowed groups give back pages no later query can see."""
        self.seq_len[slot] += n_new
        L = self.seq_len[slot]
        for g in self.kv_groups:
            w = g.request.window
            if w:
                first_needed = max(0, L + 1 - w) // PAGE       # the next query at position L sees keys >= L+1-w
                have = g.pages_of[slot]
                for i in range(min(first_needed, len(have))):
                    if have[i] >= 0:
                        g.pool.free(have[i])
                        have[i] = -1

    def upload_tables(self) -> None:
        """Copies block-table rows that changed since the last step to the device."""
        for g in self.kv_groups:
            for slot in sorted(g.dirty):
                g.table[slot].copy_(g.table_host[slot], non_blocking=True)
            g.dirty.clear()

    # ---- views ---------------------------------------------------------------------------------
    def layer_view(self, cache_id: int, writes: bool = True) -> LayerCache:
        view = self._views.get((cache_id, writes))
        if view is not None:
            return view
        view = self._views[(cache_id, writes)] = LayerCache(writes=writes)
        for (cid, key), (gi, li) in self._kv_of.items():
            if cid == cache_id:
                g = self.kv_groups[gi]
                view.kv[key] = KVView(g.k[li], g.v[li], g.table, g.request.window)
        for (cid, key), (gi, li) in self._state_of.items():
            if cid == cache_id:
                view.state[key] = self.state_groups[gi].data[li]
        return view

    def check(self) -> None:
        """Invariants: no slot or page lost, held twice or freed twice."""
        self.slots.check()
        for g in self.kv_groups:
            g.pool.check()
            held = [p for s in range(self.max_seqs) for p in g.pages_of[s] if p >= 0]
            if sorted(held) != g.pool.held():
                raise CacheError("pages held by sequences differ from the pool's record")
            for s in range(self.max_seqs):
                if g.pages_of[s] and not self.slots._held[s]:
                    raise CacheError(f"free slot {s} still holds pages")
