"""The cache's bookkeeping (no slot or page lost, held twice or freed twice) and the
generation loop's decisions, without a GPU."""
import random

import pytest
import torch

from tinyllama_c_b200.cache import Cache, CacheError, IndexPool
from tinyllama_c_b200.engine.generate import generate, plan_batches
from tinyllama_c_b200.parts import KVRequest, StateRequest


def make_cache(max_tokens=64 * 6, max_seqs=3, window=None):
    reqs = {0: [KVRequest("kv", 2, 8, None), StateRequest("s", (3,))],
            1: [KVRequest("kv", 2, 8, window), StateRequest("s", (3,)), StateRequest("t", (2, 2))]}
    return Cache(reqs, max_tokens, max_seqs, torch.float32, "cpu")


def test_index_pool():
    p = IndexPool(3, "thing")
    a, b, c = p.alloc(), p.alloc(), p.alloc()
    assert (a, b, c) == (0, 1, 2)
    with pytest.raises(CacheError, match="out of things"):
        p.alloc()
    p.free(1)
    with pytest.raises(CacheError, match="freed twice"):
        p.free(1)
    with pytest.raises(CacheError, match="does not exist"):
        p.free(7)
    assert p.alloc() == 1
    p.free(2), p.free(0)
    assert p.alloc() == 0                       # lowest free index first
    p.check()


def test_groups_follow_the_requests():
    c = make_cache(window=16)
    assert len(c.kv_groups) == 2                 # full keys and a window of them: storage of their own
    assert len(c.state_groups) == 2 and c.state_groups[0].data.shape == (2, 3, 3)
    c = make_cache()
    assert len(c.kv_groups) == 1 and c.kv_groups[0].k.shape == (2, 6, 2, 64, 8)
    v0, v1 = c.layer_view(0), c.layer_view(1)
    assert v0.kv["kv"].k_pages.data_ptr() != v1.kv["kv"].k_pages.data_ptr()
    assert set(v1.state) == {"s", "t"} and v1.state["t"].shape == (3, 2, 2)


def test_slots_and_pages_random_walk():
    rng = random.Random(0)
    c = make_cache(max_tokens=64 * 10, max_seqs=4, window=100)
    live = {}
    for _ in range(400):
        if live and rng.random() < 0.3:
            s = rng.choice(list(live))
            c.release(s)
            del live[s]
        elif len(live) < 4 and rng.random() < 0.5:
            s = c.acquire()
            assert s not in live and c.length(s) == 0
            live[s] = 0
        elif live:
            s = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 30, 70])
            try:
                start = c.reserve(s, n)
            except CacheError:
                continue
            assert start == live[s]
            c.commit(s, n)
            live[s] += n
        c.check()
        assert sorted(live) == c.slots.held()
    for s in list(live):
        c.release(s)
    c.check()
    assert all(g.pool.n_held == 0 for g in c.kv_groups)


def test_release_twice_and_reserve_errors():
    c = make_cache()
    s = c.acquire()
    c.reserve(s, 65)
    c.commit(s, 65)
    assert c.live_tokens() == 128
    c.release(s)
    with pytest.raises(CacheError, match="freed twice"):
        c.release(s)
    with pytest.raises(CacheError, match="not held"):
        c.reserve(s, 1)
    a, b = c.acquire(), c.acquire()
    c.reserve(a, 64 * 5)
    with pytest.raises(CacheError, match="cache is full"):
        c.reserve(b, 65)
    c.check()


def test_window_group_gives_pages_back():
    c = make_cache(max_tokens=64 * 8, window=70)
    s = c.acquire()
    c.reserve(s, 300)
    full, win = c.kv_groups
    assert full.pool.n_held == 5 and win.pool.n_held == 5      # a long prompt needs all its pages within the step
    c.commit(s, 300)
    assert full.pool.n_held == 5 and win.pool.n_held == 2      # positions 231.. remain visible: pages 3 and 4
    c.check()
    c.release(s)
    assert win.pool.n_held == 0


class FakeBackend:
    """Next token = (sum of the sequence so far) % 10; records what the loop asked for."""

    def __init__(self, slots=2, pages=100):
        self.free, self.pages, self.seqs, self.calls, self.released = list(range(slots)), pages, {}, [], []

    def capacity(self):
        return len(self.free), self.pages

    def acquire(self):
        s = self.free.pop(0)
        self.seqs[s] = []
        return s

    def release(self, s):
        assert s in self.seqs
        del self.seqs[s]
        self.free.append(s)
        self.released.append(s)

    def step_and_sample(self, entries, histories, ids, steps):
        self.calls.append([(s, list(t)) for s, t in entries])
        out = []
        for (s, t), h in zip(entries, histories):
            self.seqs[s] += list(t)
            assert self.seqs[s] == list(h)               # the loop's history is what the cache has seen
            out.append(sum(self.seqs[s]) % 10)
        return out


def test_loop_batches_stops_and_reuses_slots():
    be = FakeBackend(slots=2)
    prompts = [[1, 2], [3], [4, 4, 4], [9]]
    res = generate(be, prompts, max_new_tokens=4, stop_ids=[7], max_batch=8)
    # two batches of two, because there are two slots; every slot is given back
    assert [len(c) for c in be.calls if len(c[0][1]) > 1 or True][0] == 2
    assert sorted(be.released) == [0, 0, 1, 1] and not be.seqs
    # request 0: 3, 6, 2, 4 -> length; request 1: 3, 6, 2, 4; request 2: 2, 4, 8, 6; request 3: 9, 8, 6, 2
    assert res[0].tokens == [3, 6, 2, 4] and res[0].finish_reason == "length"
    assert res[2].tokens == [2, 4, 8, 6]
    # first call of a batch brings whole prompts, later calls one token each, only for live requests
    assert be.calls[0] == [(0, [1, 2]), (1, [3])]
    assert all(len(t) == 1 for call in be.calls[1:3] for _, t in call)


def test_loop_stop_token_is_not_emitted_and_others_go_on():
    be = FakeBackend(slots=3)
    res = generate(be, [[1, 2], [5], [2, 2]], max_new_tokens=5, stop_ids=[6])
    assert res[0].tokens == [3] and res[0].finish_reason == "stop"          # 3, then 6 stops
    assert res[1].tokens == [5, 0, 0, 0, 0] and res[1].finish_reason == "length"
    assert res[2].tokens == [4, 8] and res[2].finish_reason == "stop"       # 4, 8, then 16 % 10 = 6
    sizes = [len(c) for c in be.calls]
    assert sizes == sorted(sizes, reverse=True) and sizes[0] == 3 and sizes[-1] == 1
    res = generate(be, [[1, 2]], max_new_tokens=5, stop_ids=[6], ignore_eos=True)
    assert len(res[0].tokens) == 5


def test_loop_context_limit_and_errors():
    be = FakeBackend(slots=1)
    res = generate(be, [[1, 1, 1]], max_new_tokens=50, max_context=6)
    assert len(res[0].tokens) == 3 and res[0].finish_reason == "context"    # chat.c:332-335
    with pytest.raises(ValueError, match="empty"):
        generate(be, [[]])
    with pytest.raises(ValueError, match="context holds"):
        generate(be, [[1] * 6], max_context=6)


def test_plan_batches_respects_slots_and_pages():
    assert plan_batches([10, 10, 10], 10, max_batch=2, free_slots=8, free_pages=100, max_context=1000) == [[0, 1], [2]]
    assert plan_batches([100, 100, 10], 28, max_batch=8, free_slots=8, free_pages=4, max_context=1000) == [[0, 1], [2]]
    with pytest.raises(ValueError, match="needs"):
        plan_batches([1000], 10, 8, 8, 4, 2000)


def test_padded_batch_sizes_are_few_and_never_smaller():
    """The captured step that serves n sequences has at least n rows, at most 3 (up to 16) or 7 more, and the
    sizes that 1..256 sequences use are a short list: what bounds the number of captures of a run."""
    from tinyllama_c_b200.engine.generate import EngineBackend
    sizes = [EngineBackend.padded_batch(n) for n in range(1, 257)]
    assert all(p >= n and p - n <= (3 if n <= 16 else 7) for n, p in zip(range(1, 257), sizes))
    assert sizes == sorted(sizes) and sizes[:4] == [1, 2, 3, 4] and sizes[4] == 8
    assert all(EngineBackend.padded_batch(p) == p for p in sizes)            # a padded size pads no further
    assert len(set(sizes)) == 4 + 3 + 30                                     # 1..4; 8, 12, 16; 24, 32, .. 256


def test_context_buckets_are_powers_of_two_from_512():
    from tinyllama_c_b200.engine.generate import context_bucket
    assert [context_bucket(n) for n in (1, 512, 513, 1024, 1025, 40000)] == [512, 512, 1024, 1024, 2048, 65536]
    assert all(context_bucket(n) >= n and context_bucket(n) < 2 * max(n, 512) for n in range(1, 5000, 37))


# ---- the step's packing and its temporaries ------------------------------------------------------
def test_chunk_tables_follow_the_requests_thresholds():
    """A table is made when a sequence brings more rows than the request's threshold (a chunk's length unless the
    part says from how many rows its chunked form pays), and cuts every sequence into chunks of the chunk length."""
    from tinyllama_c_b200.engine.step import chunk_table, pack, StepEntry, StepError
    assert chunk_table([5, 128, 1], 128) is None                       # nothing longer than a chunk
    assert chunk_table([5, 128, 1], 128, 32) == ([0, 5, 133, 134], [0, 1, 2], [0, 1, 2, 3])
    assert chunk_table([5, 20], 128, 32) is None
    assert chunk_table([130, 3], 64) == ([0, 64, 128, 130, 133], [0, 0, 0, 1], [0, 3, 4])
    entries = [StepEntry(0, list(range(40)), (39,)), StepEntry(3, [7], (0,))]
    info, want, n = pack(entries, [0, 9], 100, "cpu", (128, 16), {128: 32})
    assert n == 2 and want.tolist() == [39, 40]
    assert info.tokens.tolist() == list(range(40)) + [7] and info.positions.tolist() == list(range(40)) + [9]
    assert info.row_seq.tolist() == [0] * 40 + [1] and info.cu_seqlens.tolist() == [0, 40, 41]
    assert info.slots.tolist() == [0, 3] and info.start_pos.tolist() == [0, 9] and info.max_new == 40 and info.max_context == 40
    seg_start, seg_seq, seq_seg_start = info.chunks[128]               # 40 rows > 32: one chunk a sequence
    assert seg_start.tolist() == [0, 40, 41] and seg_seq.tolist() == [0, 1] and seq_seg_start.tolist() == [0, 1, 2]
    assert [t.tolist() for t in info.chunks[16]] == [[0, 16, 32, 40, 41], [0, 0, 0, 1], [0, 3, 4]]
    info, _, _ = pack([StepEntry(0, list(range(30)), ())], [0], 100, "cpu", (128,), {128: 32})
    assert info.chunks[128] is None
    with pytest.raises(StepError, match="token id 100 is outside"):
        pack([StepEntry(0, [1, 100], ())], [0], 100, "cpu")
    with pytest.raises(StepError, match="wanted index 2"):
        pack([StepEntry(0, [1, 2], (2,))], [0], 100, "cpu")


def test_a_steps_temporaries_are_shared_inside_the_step_only():
    from tinyllama_c_b200.parts.base import StepInfo, scratch_buf, step_scratch
    z = torch.zeros(1, dtype=torch.int32)
    step = StepInfo(n_rows=1, n_seqs=1, tokens=z, positions=z, row_seq=z, cu_seqlens=z, slots=z, start_pos=z)
    outside = scratch_buf("a", (2, 3), torch.float32, "cpu")
    assert scratch_buf("a", (2, 3), torch.float32, "cpu") is not outside           # no step: plain allocations
    with step_scratch(step):
        a = scratch_buf("a", (2, 3), torch.float32, "cpu")
        assert scratch_buf("a", (2, 3), torch.float32, "cpu") is a                # the next layer gets the same buffer
        assert scratch_buf("b", (2, 3), torch.float32, "cpu") is not a            # another tag, shape or type: another
        assert scratch_buf("a", (2, 4), torch.float32, "cpu") is not a
        assert scratch_buf("a", (2, 3), torch.bfloat16, "cpu") is not a
        other = StepInfo(n_rows=1, n_seqs=1, tokens=z, positions=z, row_seq=z, cu_seqlens=z, slots=z, start_pos=z)
        with step_scratch(other):                                                  # a step inside a step has its own
            assert scratch_buf("a", (2, 3), torch.float32, "cpu") is not a
        assert scratch_buf("a", (2, 3), torch.float32, "cpu") is a
    assert len(step.scratch) == 4 and len(other.scratch) == 1
    assert scratch_buf("a", (2, 3), torch.float32, "cpu") is not a
