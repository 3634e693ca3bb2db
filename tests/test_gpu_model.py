"""The engine on the GPU against the plain implementation, in 32-bit and in bfloat16:
each request alone and whole; with the last 32 tokens one by one; in batches of unequal
lengths whose shorter requests end earlier, one batch after another so that slots are
reused; long decoding; the first tokens of a sequence; greedy generation through the entry
point; trace replay as a separate process."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import tinyllama_c_b200 as tlc
from tinyllama_c_b200.engine import StepEntry

import configs
from helpers import make_model_dir, plain_logits, random_tokens, read_config, read_weights, record, release_all
from plain import falcon_h1_plain as plain

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# float32 is compared with the exact plain implementation; what differs is accumulation order:
# at most 1e-4 (mean 2e-5) of the request's largest |logit|.
# bfloat16 is compared with the plain implementation's model of a bfloat16 engine (the same values
# rounded to bfloat16 at the same places).  What remains is 32-bit accumulation order, which now
# and then tips a rounding by 2^-8 of a value; the allowance is the rounding noise itself: the
# engine must agree with the bfloat16 model at least as closely as that model agrees with exact
# arithmetic on the same request (`Want.noise_max`, `Want.noise_mean`).  Where only a few rows are
# compared (a single decoded token), their mean error is held to the mean noise of the request's
# noisiest row instead of the request-wide mean: one row's mean is not an average over rows, and rows
# differ in noise by a factor of two or three.  A cache or batching fault moves logits by about their
# own size, fifty times more.
TOL = {"float32": 1e-4}
MEAN_TOL = {"float32": 2e-5}


class Want(np.ndarray):
    """Expected logits [T, V] that carry the request's allowance in absolute units."""

    def __new__(cls, arr, noise_max, noise_mean, noise_row_mean=None):
        o = np.asarray(arr).view(cls)
        o.noise_max, o.noise_mean = float(noise_max), float(noise_mean)
        o.noise_row_mean = float(noise_row_mean if noise_row_mean is not None else noise_mean)
        return o

    def __array_finalize__(self, obj):
        if obj is not None:
            self.noise_max = getattr(obj, "noise_max", None)
            self.noise_mean = getattr(obj, "noise_mean", None)
            self.noise_row_mean = getattr(obj, "noise_row_mean", None)


def expected(model_dir, toks, dtype) -> Want:
    exact = plain_logits(model_dir, toks, "float32")
    scale = np.abs(exact).max()
    if dtype == "float32":
        return Want(exact, TOL[dtype] * scale, MEAN_TOL[dtype] * scale)
    model = plain_logits(model_dir, toks, "bfloat16")
    noise = np.abs(model - exact)
    return Want(model, noise.max(), noise.mean(), noise.mean(axis=1).max())


def check(got, want, dtype, what):
    err = np.abs(got - np.asarray(want))
    mean_allowed = want.noise_mean if err.shape[0] >= 8 else want.noise_row_mean
    record(dtype, "max", err.max() / want.noise_max)
    record(dtype, "mean", err.mean() / mean_allowed)
    assert err.max() <= want.noise_max, f"{what}: max error {err.max():.3e}, allowed {want.noise_max:.3e}"
    assert err.mean() <= mean_allowed, f"{what}: mean error {err.mean():.3e}, allowed {mean_allowed:.3e}"


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("models")
    return {name: make_model_dir(root, cfg, seed=20 + i, name=name) for i, (name, cfg) in enumerate(configs.ALL.items())}


@pytest.fixture(scope="module")
def engines(folders):
    cache = {}

    def get(name, dtype):
        if (name, dtype) not in cache:
            cache[(name, dtype)] = tlc.LLM(folders[name], dtype=dtype, max_tokens=64 * 24, max_seqs=4)
        release_all(cache[(name, dtype)])
        return cache[(name, dtype)]
    return get


@pytest.fixture(scope="module")
def requests_of(folders):
    """(configuration, dtype) -> five requests of unequal lengths and the plain logits of each."""
    out = {}
    for name, cfg in configs.ALL.items():
        lens = [1, 40, 9, 150, 97]
        toks = [random_tokens(cfg["vocab_size"], n, 50 + i) for i, n in enumerate(lens)]
        for dtype in ("float32", "bfloat16"):
            out[(name, dtype)] = (toks, [expected(folders[name], t, dtype) for t in toks])
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_each_request_alone_and_whole(engines, requests_of, name, dtype):
    llm = engines(name, dtype)
    for toks, want in zip(*requests_of[(name, dtype)]):
        s = llm.cache.acquire()
        got = llm.step([StepEntry(s, toks, list(range(len(toks))))]).cpu().numpy()
        llm.cache.release(s)
        check(got, want, dtype, f"{name} whole request of {len(toks)}")
    llm.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_last_32_tokens_one_by_one(engines, requests_of, name, dtype):
    llm = engines(name, dtype)
    for toks, want in zip(*requests_of[(name, dtype)]):
        n = len(toks)
        head = max(1, n - 32)
        s = llm.cache.acquire()
        rows = [llm.step([StepEntry(s, toks[:head], list(range(head)))]).cpu().numpy()]
        for i in range(head, n):
            rows.append(llm.step([StepEntry(s, [toks[i]], [0])]).cpu().numpy())
        llm.cache.release(s)
        got = np.concatenate(rows, axis=0)
        check(got, want, dtype, f"{name} request of {n}, last {n - head} decoded")
        # the first decoded token and the prompt's last row are where a cache fault shows first
        check(got[head - 1:head + 1], want[head - 1:head + 1], dtype, f"{name} around the cut at {head}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_unequal_batches_with_slot_reuse(engines, requests_of, name, dtype):
    """Two batches one after the other on a cache of 4 slots; in each, prompts (all but the last
    k tokens) run in one step, then one token each; shorter requests end earlier."""
    llm = engines(name, dtype)
    toks, want = requests_of[(name, dtype)]
    for batch in ([0, 1, 2, 3], [4, 2, 1]):
        slots = {i: llm.cache.acquire() for i in batch}
        decode = {i: min(len(toks[i]) - 1, 3 + 5 * k) for k, i in enumerate(batch)}     # unequal decode lengths
        cut = {i: len(toks[i]) - decode[i] for i in batch}
        got = llm.step([StepEntry(slots[i], toks[i][:cut[i]], [0, cut[i] - 1]) for i in batch]).cpu().numpy()
        for r, i in enumerate(batch):
            check(got[2 * r:2 * r + 2], want[i][[0, cut[i] - 1]], dtype, f"{name} batch prefill of request {i}")
        live = []
        for i in batch:                                   # a request whose prompt was all of it ends here
            if cut[i] < len(toks[i]):
                live.append(i)
            else:
                llm.cache.release(slots[i])
        k = 0
        while live:
            ents = [StepEntry(slots[i], [toks[i][cut[i] + k]], [0]) for i in live]
            got = llm.step(ents).cpu().numpy()
            for r, i in enumerate(live):
                check(got[r:r + 1], want[i][cut[i] + k:cut[i] + k + 1], dtype,
                      f"{name} request {i} decode {k} in a batch of {len(live)}")
            k += 1
            for i in list(live):
                if cut[i] + k >= len(toks[i]):
                    llm.cache.release(slots[i])
                    live.remove(i)
        llm.cache.check()
    assert llm.cache.slots.n_held == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(engines, folders, dtype):
    """A 3-token prompt followed by 200 single-token steps (crosses three pages)."""
    llm = engines("A", dtype)
    toks = random_tokens(configs.TINY_A["vocab_size"], 203, 77)
    want = expected(folders["A"], toks, dtype)
    s = llm.cache.acquire()
    rows = [llm.step([StepEntry(s, toks[:3], [0, 1, 2])]).cpu().numpy()]
    for t in toks[3:]:
        rows.append(llm.step([StepEntry(s, [t], [0])]).cpu().numpy())
    llm.cache.release(s)
    check(np.concatenate(rows), want, dtype, "long decoding")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_first_tokens_of_a_sequence(engines, requests_of, name, dtype):
    """Token by token from the very first one: the conv window and the state start empty."""
    llm = engines(name, dtype)
    toks, want = requests_of[(name, dtype)][0][1][:8], requests_of[(name, dtype)][1][1][:8]
    s = llm.cache.acquire()
    rows = [llm.step([StepEntry(s, [t], [0])]).cpu().numpy() for t in toks]
    llm.cache.release(s)
    check(np.concatenate(rows), want, dtype, f"{name} first tokens")


@pytest.mark.parametrize("window", [None, 37])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_peaked_attention_over_a_far_key(tmp_path, dtype, window):
    """Queries and keys scaled so that scores are spread wide: a query's mass sits on a few
    keys, often far ones, and a wrong page or position shows as a large error.  With a window
    of 37 the mass often sits on a key near the window's edge: one key too many or too few shows
    too, and so does a page behind the window that was given back too early."""
    cfg = dict(configs.TINY_A, sliding_window=window)
    d = make_model_dir(tmp_path, cfg, seed=5, name="peaked")
    from safetensors.torch import load_file, save_file
    w = load_file(os.path.join(d, "model.safetensors"))
    for k in list(w):
        if k.endswith("q_proj.weight") or k.endswith("k_proj.weight"):
            w[k] = (w[k].float() * 4.0).to(w[k].dtype)
    save_file(w, os.path.join(d, "model.safetensors"))
    toks = random_tokens(cfg["vocab_size"], 230, 91)
    want = expected(d, toks, dtype)
    llm = tlc.LLM(d, dtype=dtype, max_tokens=512, max_seqs=2)
    s = llm.cache.acquire()
    rows = [llm.step([StepEntry(s, toks[:190], list(range(190)))]).cpu().numpy()]
    for t in toks[190:]:
        rows.append(llm.step([StepEntry(s, [t], [0])]).cpu().numpy())
    check(np.concatenate(rows), want, dtype, "peaked attention")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_entry_point(engines, folders, name, dtype):
    llm = engines(name, dtype)
    cfg = configs.ALL[name]
    prompts = [random_tokens(cfg["vocab_size"], n, 200 + n) for n in (3, 17, 1, 30, 8, 45)]
    res = llm.generate(prompts, tlc.GREEDY, max_new_tokens=10, ignore_eos=True, max_batch=4)
    assert llm.cache.slots.n_held == 0
    w = read_weights(folders[name])
    c = read_config(folders[name])
    rnd = plain.bf16_round if dtype == "bfloat16" else plain._same
    for p, r in zip(prompts, res):
        assert len(r.tokens) == 10 and r.finish_reason == "length"
        ref = plain.forward(c, w, (p + r.tokens)[:-1], rnd=rnd)
        for k, tok in enumerate(r.tokens):
            row = ref[len(p) - 1 + k]
            best = int(np.argmax(row))
            margin = 1e-4 * np.abs(ref).max() if dtype == "float32" else 0.03 * np.abs(ref).max()
            assert tok == best or row[best] - row[tok] <= margin, \
                f"{name} {dtype}: generated token {k} = {tok}, plain argmax {best}"
    # one request alone gives the same tokens as inside the batches (float32: exactly)
    alone = llm.generate([prompts[3]], tlc.GREEDY, max_new_tokens=10, ignore_eos=True)
    if dtype == "float32":
        assert alone[0].tokens == res[3].tokens


def test_generation_stops_and_samples_reproducibly(engines):
    llm = engines("A", "float32")
    prompts = [random_tokens(256, n, 300 + n) for n in (4, 12, 7)]
    params = tlc.SamplingParams(temperature=0.9, top_k=20, top_p=0.95, min_p=0.01, seed=7)
    a = llm.generate(prompts, params, max_new_tokens=12, ignore_eos=True)
    b = llm.generate(list(reversed(prompts)), params, max_new_tokens=12, ignore_eos=True)
    assert [r.tokens for r in a] == [r.tokens for r in llm.generate(prompts, params, max_new_tokens=12, ignore_eos=True)]
    assert len({tuple(r.tokens) for r in a}) > 1
    assert all(len(r.tokens) == 12 for r in b)
    # a stop token ends its sequence early and is not emitted; the others go on
    stop = a[1].tokens[4]
    c = llm.generate(prompts, params, max_new_tokens=12, stop_ids=[stop])
    first = a[1].tokens.index(stop)
    assert c[1].tokens == a[1].tokens[:first] and c[1].finish_reason == "stop"
    assert llm.cache.slots.n_held == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_as_a_program(folders, requests_of, tmp_path, dtype):
    toks, want = requests_of[("B", dtype)]
    out = str(tmp_path / "out")
    steps = [{"step": 0, "entries": [{"id": "r1", "tokens": toks[1][:30], "want": [0, 29]},
                                     {"id": "r2", "tokens": toks[2][:8], "want": [7]}], "end": []}]
    steps.append({"step": 1, "entries": [{"id": "r1", "tokens": [toks[1][30]], "want": [0]},
                                         {"id": "r2", "tokens": [toks[2][8]], "want": [0]}], "end": ["r2"]})
    steps.append({"step": 2, "entries": [{"id": "r1", "tokens": [toks[1][31]], "want": []}], "end": []})
    steps.append({"step": 3, "entries": [{"id": "r1", "tokens": [toks[1][32]], "want": [0]}], "end": ["r1"]})
    steps.append({"step": 4, "entries": [{"id": "r3", "tokens": toks[4], "want": [len(toks[4]) - 1]}], "end": ["r3"]})
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folders["B"], "--dtype", dtype,
                        "--out", out, "--max-tokens", "256"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(5)]
    V = configs.TINY_B["vocab_size"]
    rd = lambda i: np.fromfile(os.path.join(out, f"{i}.f32"), "<f4").reshape(-1, V)
    check(rd(0)[:2], want[1][[0, 29]], dtype, "trace step 0, first request")
    check(rd(0)[2:], want[2][7:8], dtype, "trace step 0, second request")
    check(rd(1)[:1], want[1][30:31], dtype, "trace step 1, first request")
    check(rd(1)[1:], want[2][8:9], dtype, "trace step 1, second request")
    assert not os.path.exists(os.path.join(out, "2.f32"))
    check(rd(3), want[1][32:33], dtype, "trace step 3")
    check(rd(4), want[4][-1:], dtype, "trace step 4")


def test_prompts_in_pieces_and_the_command_line(engines, folders, requests_of, tmp_path):
    """Prompts cut into steps of at most 48 tokens give the tokens of prompts run whole; the
    bench program generates the same tokens as the entry point."""
    llm = engines("D", "float32")
    cfg = configs.TINY_D
    prompts = [random_tokens(cfg["vocab_size"], n, 400 + n) for n in (130, 20, 61)]
    whole = llm.generate(prompts, tlc.GREEDY, max_new_tokens=6, ignore_eos=True)
    pieces = llm.generate(prompts, tlc.GREEDY, max_new_tokens=6, ignore_eos=True, max_step_tokens=48)
    assert [r.tokens for r in whole] == [r.tokens for r in pieces]
    assert llm.cache.slots.n_held == 0
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "bench"), "-m", folders["D"], "--dtype", "float32", "-t", "0",
                        "-n", "6", "-i", " ".join(map(str, prompts[1])), "--ignore-eos", "-ub", "16"],
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert p.stdout.strip().splitlines()[-1].split() == [str(t) for t in whole[1].tokens]
    chat = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "chat"), "-m", folders["D"], "--dtype", "float32", "-t", "0",
                           "-n", "6", "--ignore-eos"], input=" ".join(map(str, prompts[1])) + "\n/clear\n5 6 7\n/quit\n",
                          capture_output=True, text=True, timeout=600)
    assert chat.returncode == 0, chat.stderr[-2000:]
    assert chat.stdout.strip().splitlines()[0].split() == [str(t) for t in whole[1].tokens]
