"""Schedules of steps that the whole / last-32 / unequal-batch cuts do not reach, against the plain
implementation in 32-bit and in bfloat16: a prompt in pieces that ask for no logits followed at once by
single-token steps (nothing on the host separates those steps); a step that mixes one request's prompt
piece with other requests' single tokens; generation that crosses a context bucket of the captured
decode step (a new capture, another attention grid, eviction of old captures)."""
import numpy as np
import pytest
import torch

import tinyllama_c_b200 as tlc
from tinyllama_c_b200.engine import StepEntry
from tinyllama_c_b200.engine.generate import EngineBackend

import configs
from helpers import make_model_dir, random_tokens, read_config, read_weights, release_all
from plain import falcon_h1_plain as plain
from test_gpu_model import check, expected

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("sched")
    out = {name: make_model_dir(root, configs.ALL[name], seed=60 + i, name=name) for i, name in enumerate("ABD")}
    out["long"] = make_model_dir(root, dict(configs.TINY_D, max_position_embeddings=2048), seed=70, name="long")
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "D"])
@pytest.mark.parametrize("piece", [40, 129])
def test_prompt_in_pieces_without_logits_then_single_tokens(folders, name, dtype, piece):
    """A 300-token prompt in pieces; only the last piece wants a row.  Then 8 one-token steps, one of
    which wants nothing.  No step before the last piece returns anything to the host, so the host never
    waits between them: what orders a step after the one before is the launch of its first kernel."""
    cfg = configs.ALL[name]
    toks = random_tokens(cfg["vocab_size"], 308, 5)
    want = expected(folders[name], toks, dtype)
    llm = tlc.LLM(folders[name], dtype=dtype, max_tokens=512, max_seqs=2)
    s = llm.cache.acquire()
    rows, at = [], []
    for i in range(0, 300, piece):
        chunk = toks[i:min(i + piece, 300)]
        last = i + piece >= 300
        out = llm.step([StepEntry(s, chunk, [len(chunk) - 1] if last else [])])
        assert (out is not None) == last
    rows.append(out.cpu().numpy())
    at.append(299)
    for k in range(300, 308):
        out = llm.step([StepEntry(s, [toks[k]], [] if k == 303 else [0])])
        if k != 303:
            rows.append(out.cpu().numpy())
            at.append(k)
    llm.cache.release(s)
    check(np.concatenate(rows), want[at], dtype, f"{name} prompt in pieces of {piece}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_one_layer_pieces_of_at_most_128_rows_then_a_token(tmp_path, dtype):
    """One layer: the writer of a sequence's state and window is only a handful of launches ahead of the
    kernel of the next step that fetches them before its dependency wait."""
    cfg = dict(configs.TINY_D, num_hidden_layers=1)
    d = make_model_dir(tmp_path, cfg, seed=8, name="one")
    toks = random_tokens(cfg["vocab_size"], 262, 9)
    want = expected(d, toks, dtype)
    llm = tlc.LLM(d, dtype=dtype, max_tokens=512, max_seqs=1)
    s = llm.cache.acquire()
    for a, b in ((0, 100), (100, 228), (228, 260)):                                # 100, 128 and 32 rows
        llm.step([StepEntry(s, toks[a:b], [])])
    llm.step([StepEntry(s, [toks[260]], [])])
    got = llm.step([StepEntry(s, [toks[261]], [0])]).cpu().numpy()
    check(got, want[261:262], dtype, "one layer, pieces then tokens")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "D"])
def test_a_step_that_mixes_a_prompt_piece_with_single_tokens(folders, name, dtype):
    cfg = configs.ALL[name]
    V = cfg["vocab_size"]
    toks = [random_tokens(V, n, 30 + n) for n in (140, 21, 12)]
    want = [expected(folders[name], t, dtype) for t in toks]
    llm = tlc.LLM(folders[name], dtype=dtype, max_tokens=512, max_seqs=3)
    slots = [llm.cache.acquire() for _ in toks]
    # request 0 brings its first 70 tokens; requests 1 and 2 all but their last token
    llm.step([StepEntry(slots[0], toks[0][:70], []), StepEntry(slots[1], toks[1][:-1], []),
              StepEntry(slots[2], toks[2][:-1], [])])
    # the mixed step: 70 more rows of request 0 between the single tokens of requests 1 and 2
    got = llm.step([StepEntry(slots[1], toks[1][-1:], [0]), StepEntry(slots[0], toks[0][70:], [0, 34, 69]),
                    StepEntry(slots[2], toks[2][-1:], [0])]).cpu().numpy()
    check(got[0:1], want[1][-1:], dtype, f"{name} mixed step, single token of request 1")
    check(got[1:4], want[0][[70, 104, 139]], dtype, f"{name} mixed step, prompt piece")
    check(got[4:5], want[2][-1:], dtype, f"{name} mixed step, single token of request 2")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_generation_crosses_a_context_bucket(folders, dtype, monkeypatch):
    """Prompts of 500 and 470 tokens and 40 new tokens: the longer sequence crosses 512 positions at its
    13th token, where the captured step of the 512 bucket no longer fits and the 1024 one is captured; with
    room for two captures only, the old ones are dropped on the way."""
    monkeypatch.setattr(EngineBackend, "MAX_GRAPHS", 2)
    cfg = read_config(folders["long"])
    V = cfg["vocab_size"]
    prompts = [random_tokens(V, n, 800 + n) for n in (500, 470)]
    llm = tlc.LLM(folders["long"], dtype=dtype, max_tokens=64 * 20, max_seqs=2)
    res = llm.generate(prompts, tlc.GREEDY, max_new_tokens=40, ignore_eos=True)
    buckets = sorted({k[2] for k in llm._graphs})
    assert len(llm._graphs) <= 2 and 1024 in buckets
    W = read_weights(folders["long"])
    rnd = plain.bf16_round if dtype == "bfloat16" else plain._same
    for p, r in zip(prompts, res):
        assert len(r.tokens) == 40
        ref = plain.forward(cfg, W, (p + r.tokens)[:-1], rnd=rnd)
        margin = (1e-4 if dtype == "float32" else 0.03) * np.abs(ref).max()
        for k, tok in enumerate(r.tokens):
            row = ref[len(p) - 1 + k]
            best = int(np.argmax(row))
            assert tok == best or row[best] - row[tok] <= margin, f"{dtype}: token {k} is {tok}, plain argmax {best}"
    # temperature and penalties through the same captures: the tokens are those of the same steps run one
    # by one without captured graphs (same kernels, same draws keyed by seed, request and step)
    params = tlc.SamplingParams(temperature=0.8, top_k=30, top_p=0.9, min_p=0.02, repeat_penalty=1.2,
                                frequency_penalty=0.1, presence_penalty=0.1, seed=3)
    a = llm.generate(prompts, params, max_new_tokens=40, ignore_eos=True)
    assert len(llm._graphs) <= 2
    eager = tlc.LLM(folders["long"], dtype=dtype, max_tokens=64 * 20, max_seqs=2, use_graphs=False)
    b = eager.generate(prompts, params, max_new_tokens=40, ignore_eos=True)
    if dtype == "float32":
        assert [r.tokens for r in a] == [r.tokens for r in b]
    else:
        same = sum(x == y for ra, rb in zip(a, b) for x, y in zip(ra.tokens, rb.tokens))
        assert same >= 40          # bfloat16: a rounding may tip one draw; the sequences then part ways
    assert llm.cache.slots.n_held == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_requests_that_end_at_different_times_share_captured_steps(folders, dtype):
    """Seven requests whose stop tokens end them one by one: the captured steps are those of batch sizes 8, 4, 3, 2, 1
    (seven, six and five sequences run in the graph of eight, filled up with rows of a spare slot), the tokens are
    the ones that steps without captured graphs give, and every slot and page is back at the end."""
    cfg = read_config(folders["long"])
    V = cfg["vocab_size"]
    prompts = [random_tokens(V, n, 900 + n) for n in (30, 9, 17, 40, 12, 25, 33)]
    eager = tlc.LLM(folders["long"], dtype=dtype, max_tokens=64 * 16, max_seqs=8, use_graphs=False)
    free = eager.generate(prompts, tlc.GREEDY, max_new_tokens=24, ignore_eos=True)
    # every request gets a stop token out of its own greedy continuation, at a different step
    stops = {free[i].tokens[3 * i + 2] for i in range(len(prompts))}
    want = eager.generate(prompts, tlc.GREEDY, max_new_tokens=24, stop_ids=sorted(stops))
    assert len({len(r.tokens) for r in want}) >= 4, "the requests should end at different steps"
    llm = tlc.LLM(folders["long"], dtype=dtype, max_tokens=64 * 16, max_seqs=8)
    pages = [g.pool.n_free for g in llm.cache.kv_groups]
    got = llm.generate(prompts, tlc.GREEDY, max_new_tokens=24, stop_ids=sorted(stops))
    assert [r.tokens for r in got] == [r.tokens for r in want]
    assert [r.finish_reason for r in got] == [r.finish_reason for r in want]
    sizes = sorted({k[1] for k in llm._graphs})
    assert set(sizes) <= {1, 2, 3, 4, 8} and 8 in sizes, sizes
    assert llm.cache.slots.n_held == 0 and [g.pool.n_free for g in llm.cache.kv_groups] == pages


def test_a_turn_continues_in_a_held_slot(folders):
    """generate() with a Continuation: a second turn in the slot of the first equals one request that
    brings both turns' tokens (history is not recomputed, chat.c:296)."""
    llm = tlc.LLM(folders["A"], dtype="float32", max_tokens=512, max_seqs=2)
    V = configs.TINY_A["vocab_size"]
    t1, t2 = random_tokens(V, 9, 1), random_tokens(V, 5, 2)
    slot = llm.cache.acquire()
    r1 = llm.generate([t1], tlc.GREEDY, max_new_tokens=4, ignore_eos=True, continuations=[tlc.Continuation(slot)])[0]
    assert r1.finish_reason == "length" and r1.uncached == 1 and llm.cache.slots.n_held == 1
    cached = t1 + r1.tokens[:-1]
    seen = []
    r2 = llm.generate([r1.tokens[-1:] + t2], tlc.GREEDY, max_new_tokens=5, ignore_eos=True,
                      continuations=[tlc.Continuation(slot, cached, 4)], on_token=lambda i, t: seen.append(t))[0]
    assert seen == r2.tokens
    llm.cache.release(slot)
    whole = llm.generate([t1 + r1.tokens + t2], tlc.GREEDY, max_new_tokens=5, ignore_eos=True)[0]
    assert whole.tokens == r2.tokens
    assert llm.cache.slots.n_held == 0


def test_a_bounded_wait_that_runs_out_is_reported_and_cleared(folders):
    """The error channel: a block waits (with a limit of a few thousand cycles) on a barrier nobody
    arrives at, gives up, records its code and returns; the next step raises; after that the library works."""
    from tinyllama_c_b200 import ops
    llm = tlc.LLM(folders["D"], dtype="bfloat16", max_tokens=512, max_seqs=1)
    ops.check_errors()
    ops.wait_limit_cycles(5000)
    try:
        ops.selftest_bounded_wait()
        torch.cuda.synchronize()
    finally:
        ops.wait_limit_cycles(0)
    s = llm.cache.acquire()
    with pytest.raises(ops.KernelError, match="code 9"):
        llm.step([StepEntry(s, [1, 2, 3], [2])])
    llm.cache.release(s)
    ops.check_errors()                                   # cleared by the raise
    s = llm.cache.acquire()
    toks = random_tokens(configs.TINY_D["vocab_size"], 150, 4)
    got = llm.step([StepEntry(s, toks, [149])]).cpu().numpy()
    check(got, expected(folders["D"], toks, "bfloat16")[149:150], "bfloat16", "after the cleared error")
