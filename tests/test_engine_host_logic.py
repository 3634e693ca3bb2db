"""The engine's host logic (packing, block tables, slots, schedule) on a machine without a
GPU: the kernels are replaced by their plain PyTorch statements, everything else is the
product's code, and the result must equal the plain whole-sequence implementation."""
import numpy as np
import pytest
import torch

import tinyllama_c_b200 as tlc
from tinyllama_c_b200 import ops
from tinyllama_c_b200.engine import StepEntry, step
from tinyllama_c_b200.weights import load_model

import configs
from helpers import make_model_dir, plain_logits, random_tokens
from plain import ops_plain


@pytest.fixture()
def cpu_kernels(monkeypatch):
    ops_plain.install(monkeypatch, ops)


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_cuts_and_batches_equal_whole_sequences(tmp_path, cpu_kernels, name):
    cfg = configs.ALL[name]
    d = make_model_dir(tmp_path, cfg, seed=3)
    model = load_model(d, "float32", "cpu")
    cache = tlc.Cache(model.cache_requests(), max_tokens=64 * 8, max_seqs=3, dtype=torch.float32, device="cpu")
    lens = [70, 5, 33]
    prompts = [random_tokens(cfg["vocab_size"], n, 10 + i) for i, n in enumerate(lens)]
    want = [plain_logits(d, p) for p in prompts]
    scale = max(np.abs(w).max() for w in want)

    # whole, one request at a time
    for p, w in zip(prompts, want):
        s = cache.acquire()
        got = step(model, cache, [StepEntry(s, p, list(range(len(p))))]).numpy()
        cache.release(s)
        assert np.abs(got - w).max() < 2e-5 * scale
    # a batch of unequal lengths: all but the last 3 tokens in one step, then one token each
    slots = [cache.acquire() for _ in prompts]
    cut = [max(1, len(p) - 3) for p in prompts]
    got = step(model, cache, [StepEntry(s, p[:c], [c - 1]) for s, p, c in zip(slots, prompts, cut)]).numpy()
    for i, (w, c) in enumerate(zip(want, cut)):
        assert np.abs(got[i] - w[c - 1]).max() < 2e-5 * scale
    for k in range(3):
        ents, idx = [], []
        for i, (s, p, c) in enumerate(zip(slots, prompts, cut)):
            if c + k < len(p):
                ents.append(StepEntry(s, [p[c + k]], [0]))
                idx.append((i, c + k))
        got = step(model, cache, ents).numpy()
        for row, (i, pos) in enumerate(idx):
            assert np.abs(got[row] - want[i][pos]).max() < 2e-5 * scale
    for s in slots:
        cache.release(s)
    cache.check()
    assert cache.slots.n_held == 0 and all(g.pool.n_held == 0 for g in cache.kv_groups)


def _bound(in_features, out_features, scale, bias, seed):
    from tinyllama_c_b200.parts.linear import StackedLinear
    g = torch.Generator().manual_seed(seed)
    lin = StackedLinear(in_features)
    lin.add("w", out_features, "b" if bias else None, 1.0, scale)
    tensors = {"w": torch.randn(out_features, in_features, generator=g)}
    if bias:
        tensors["b"] = torch.randn(out_features, generator=g)
    lin.bind(tensors, torch.float32, "cpu")
    return lin


def test_output_projections_as_one_product(cpu_kernels):
    """Projections whose results are added share one product over their inputs side by side when their
    output scales agree up to a number each, which goes to whoever can scale its input; the sum, the
    biases and the scales come out as from the separate products."""
    from tinyllama_c_b200.parts.linear import StackedLinear
    g = torch.Generator().manual_seed(0)
    a, b = _bound(16, 24, 0.8, True, 1), _bound(40, 24, 0.9, False, 2)
    xa, xb = torch.randn(5, 16, generator=g), torch.randn(5, 40, generator=g)
    want = torch.ones(5, 24)
    a.forward(xa, want, accumulate=True)
    b.forward(xb, want, accumulate=True)
    fused, factors = StackedLinear.fuse_bound_inputs([a, b], [False, True])
    assert factors[0] == 1.0 and abs(factors[1] - 0.9 / 0.8) < 1e-6 and fused.in_features == 56
    got = torch.ones(5, 24)
    fused.forward(torch.cat([xa, xb * factors[1]], dim=1), got, accumulate=True)
    assert (got - want).abs().max() < 1e-5 * want.abs().max()
    # the parts still work on their own, from their columns of the fused matrix
    again = torch.ones(5, 24)
    a.forward(xa, again, accumulate=True)
    b.forward(xb, again, accumulate=True)
    assert torch.equal(again, want)
    # refused: nobody can take the second part's factor; widths off 16-byte boundaries; scales that differ by row
    assert StackedLinear.fuse_bound_inputs([_bound(16, 24, 0.8, False, 1), _bound(40, 24, 0.9, False, 2)], [False, False]) is None
    assert StackedLinear.fuse_bound_inputs([_bound(12, 24, 1.0, False, 1), _bound(40, 24, 1.0, False, 2)], [True, True]) is None
    rows = [1.0] * 12 + [2.0] * 12
    assert StackedLinear.fuse_bound_inputs([_bound(16, 24, 1.0, False, 1), _bound(40, 24, rows, False, 2)], [False, True]) is None
    assert StackedLinear.fuse_bound_inputs([_bound(16, 24, 1.0, False, 1), _bound(40, 32, 1.0, False, 2)], [True, True]) is None
