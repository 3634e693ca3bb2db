"""The plain implementation reproduces the logits that CodeClaper/tinyllama.c's own CPU engine
produced for tiny random Falcon-H1 models (recorded by tests/golden/make_golden.py)."""
import ast
import os

import numpy as np
import pytest

from plain import falcon_h1_plain as plain

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name", ["ref_a", "ref_b"])
def test_plain_equals_reference(name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    cfg = ast.literal_eval(str(z["config"]))
    W = {k[2:]: z[k] for k in z.files if k.startswith("w:")}
    tokens = z["tokens"].tolist()
    mine = plain.forward(cfg, W, tokens)
    scale = np.abs(mine).max()
    # the reference is 32-bit with its own summation order (measured 7e-6 at scale 10)
    assert np.abs(z["logits_by_token"] - mine).max() < 2e-6 * scale + 1e-6
    assert np.abs(z["logits_whole_last"] - mine[-1]).max() < 2e-6 * scale + 1e-6


def test_plain_float32_matches_float64():
    z = np.load(os.path.join(GOLDEN, "ref_a.npz"))
    cfg = ast.literal_eval(str(z["config"]))
    W = {k[2:]: z[k] for k in z.files if k.startswith("w:")}
    a = plain.forward(cfg, W, z["tokens"].tolist())
    b = plain.forward(cfg, W, z["tokens"].tolist(), dtype=np.float32)
    assert np.abs(a - b).max() < 1e-4


def test_plain_sampler_filters():
    logits = np.log(np.array([0.5, 0.2, 0.15, 0.1, 0.05]))
    ids, p = plain.filtered_distribution(logits, 1.0, top_k=3)
    assert list(ids) == [0, 1, 2] and abs(p.sum() - 1) < 1e-12
    ids, p = plain.filtered_distribution(logits, 1.0, top_p=0.7)
    assert list(ids) == [0, 1]                      # 0.5 < 0.7 <= 0.7
    ids, p = plain.filtered_distribution(logits, 1.0, min_p=0.25)
    assert list(ids) == [0, 1, 2]                   # 0.125 is the bar; 0.1 falls below
    pen = plain.apply_penalties([1.0, -1.0, 2.0], [0, 1, 0], repeat_penalty=2.0, frequency_penalty=0.5)
    assert np.allclose(pen, [1.0 / 2 - 2 * 0.5, -2.0 - 0.5, 2.0])
    assert plain.greedy([1.0, 3.0, 3.0]) == 1
