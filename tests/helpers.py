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


def plain_logits(model_dir: str, tokens) -> np.ndarray:
    return plain.forward(read_config(model_dir), read_weights(model_dir), list(tokens))


def random_tokens(vocab: int, n: int, seed: int):
    return np.random.default_rng(seed).integers(0, vocab, n).tolist()
