"""Shared helpers of the tests: model folders in temporary places, the plain forward."""
import json
import os

import numpy as np
import torch

import tinyllama_c_b200 as tlc
from plain import falcon_h1_plain as plain


def make_model_dir(tmp_path, cfg: dict, seed: int, dtype="bfloat16", std=0.25, name="model"):
    d = os.path.join(str(tmp_path), name)
    tlc.write_random_model(dict(cfg), d, seed=seed, dtype=dtype, std=std)
    return d


def read_weights(model_dir: str) -> dict:
    """Weights of a folder as float64 numpy arrays, read with the safetensors package (not the product's reader)."""
    from safetensors.torch import load_file
    return {k: v.to(torch.float64).numpy() for k, v in load_file(os.path.join(model_dir, "model.safetensors")).items()}


def read_config(model_dir: str) -> dict:
    with open(os.path.join(model_dir, "config.json")) as f:
        return json.load(f)


def plain_logits(model_dir: str, tokens, dtype: str = "float32") -> np.ndarray:
    """Logits of the plain implementation; for "bfloat16" with its model of a bfloat16 engine
    (inputs of matrix products and stored q/k/v rounded, everything else exact)."""
    rnd = plain.bf16_round if dtype == "bfloat16" else plain._same
    return plain.forward(read_config(model_dir), read_weights(model_dir), list(tokens), rnd=rnd)


def release_all(llm) -> None:
    """Gives back slots that an earlier, failed test left held."""
    for s in llm.cache.slots.held():
        llm.cache.release(s)


def random_tokens(vocab: int, n: int, seed: int):
    return np.random.default_rng(seed).integers(0, vocab, n).tolist()


STATS = {}      # (dtype, kind) -> largest error seen as a fraction of its allowance (printed after the run)


def record(dtype: str, kind: str, ratio: float) -> None:
    STATS[(dtype, kind)] = max(STATS.get((dtype, kind), 0.0), float(ratio))
