"""Parts defined here, outside the package, can be registered, built into a model and stepped:
a mixer with state of its own, a feed-forward with routing, another position encoding, and an
architecture that uses them -- one layer twice in the run order, one layer reading another's
cache.  None of this touches the package's files.  The toy parts compute with PyTorch (they
are test code); the package's own parts around them run its kernels, or their plain
statements when there is no GPU.
"""
import json
import os
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import tinyllama_c_b200 as tlc
from tinyllama_c_b200 import ops
from tinyllama_c_b200.config.base import ModelConfig
from tinyllama_c_b200.engine import StepEntry, step
from tinyllama_c_b200.models.model import Model
from tinyllama_c_b200.parts import (KVRequest, LayerRun, LayerSpec, Part, PartSpec, StateRequest, WeightSpec,
                                    register_feed_forward, register_mixer, register_position)
from tinyllama_c_b200.weights import load_model, write_random_model

from plain import ops_plain


@register_mixer("toy_decay")
class ToyDecayMixer(Part):
    """s_t = decay * s_{t-1} + W_in x_t (per sequence, state [width]); out = W_out s_t."""

    def __init__(self, hidden, width, prefix, decay=0.5):
        self.hidden, self.width, self.prefix, self.decay = hidden, width, prefix, decay

    def weight_specs(self):
        return [WeightSpec(self.prefix + "w_in", (self.width, self.hidden)),
                WeightSpec(self.prefix + "w_out", (self.hidden, self.width))]

    def cache_requests(self):
        return [StateRequest("toy.s", (self.width,))]

    def bind(self, tensors, dtype, device):
        self.w_in = tensors[self.prefix + "w_in"].to(device=device, dtype=torch.float32)
        self.w_out = tensors[self.prefix + "w_out"].to(device=device, dtype=torch.float32)

    def forward(self, normed, step_info, cache, residual):
        state = cache.state["toy.s"]
        u = normed.float() @ self.w_in.T
        for b in range(step_info.n_seqs):
            t0, t1 = step_info.host_lens and sum(step_info.host_lens[:b]), sum(step_info.host_lens[:b + 1])
            slot = step_info.host_slots[b]
            s = state[slot].clone() if step_info.host_start[b] > 0 else torch.zeros_like(state[slot])
            for t in range(t0, t1):
                s = self.decay * s + u[t]
                residual[t] += s @ self.w_out.T
            state[slot] = s


@register_feed_forward("toy_routed")
class ToyRoutedFFN(Part):
    """Two experts, the router picks one per token (argmax of 32-bit router logits)."""

    def __init__(self, hidden, prefix):
        self.hidden, self.prefix = hidden, prefix

    def weight_specs(self):
        return [WeightSpec(self.prefix + "router", (2, self.hidden)),
                WeightSpec(self.prefix + "experts", (2, self.hidden, self.hidden))]

    def bind(self, tensors, dtype, device):
        self.router = tensors[self.prefix + "router"].to(device=device, dtype=torch.float32)
        self.experts = tensors[self.prefix + "experts"].to(device=device, dtype=torch.float32)

    def forward(self, normed, residual):
        x = normed.float()
        choice = (x @ self.router.T).argmax(dim=1)
        for e in range(2):
            rows = (choice == e).nonzero().flatten()
            if rows.numel():
                residual[rows] += torch.tanh(x[rows] @ self.experts[e].T)


@register_position("toy_learned_offset")
class ToyScaledRotary(Part):
    """Another position encoding: the package's rotary table with positions counted in halves."""

    def __init__(self, head_dim, theta):
        from tinyllama_c_b200.parts.position import RotaryNeox
        self.inner = RotaryNeox(head_dim, theta)

    def bind(self, tensors, dtype, device):
        self.inner.bind(tensors, dtype, device)
        self.inner.inv_freq = (self.inner.inv_freq * 0.5).contiguous()

    def rotate_and_store(self, *a, **k):
        self.inner.rotate_and_store(*a, **k)


@dataclass(frozen=True)
class ToyConfig(ModelConfig):
    vocab_size: int
    hidden_size: int
    eps: float = 1e-5
    initializer_range: float = 0.3


def build_toy(cfg: ToyConfig) -> Model:
    D = cfg.hidden_size
    norm = lambda n: PartSpec("norm", "rmsnorm", dict(width=D, eps=cfg.eps, weight_name=n))
    att = lambda l, pos: PartSpec("mixer", "attention", dict(
        hidden=D, n_heads=2, n_kv_heads=1, head_dim=D // 2, prefix=f"l{l}.att.",
        position=PartSpec("position", pos, dict(head_dim=D // 2, **({} if pos == "none" else {"theta": 100.0})))))
    layers = [
        LayerSpec(norm("l0.n1"), (PartSpec("mixer", "toy_decay", dict(hidden=D, width=6, prefix="l0.toy.")),),
                  norm("l0.n2"), PartSpec("feed_forward", "toy_routed", dict(hidden=D, prefix="l0.moe."))),
        LayerSpec(norm("l1.n1"), (att(1, "toy_learned_offset"),), norm("l1.n2"),
                  PartSpec("feed_forward", "swiglu", dict(hidden=D, intermediate=2 * D, prefix="l1.ffn."))),
        LayerSpec(norm("l2.n1"), (att(2, "none"),), None, None),
    ]
    # layer 0 runs twice (one set of weights, a state per run); layer 2 reads the keys and values
    # that layer 1 (entry 1 of the run order) stored, without storing its own
    schedule = [LayerRun(0), LayerRun(1), LayerRun(0), LayerRun(2, cache=1)]
    return Model(cfg, layers, schedule, norm("final"), embed_name="emb", head_name=None, vocab=cfg.vocab_size, hidden=D)


tlc.register_architecture("ToyForCausalLM", ToyConfig, build_toy)
TOY = dict(architectures=["ToyForCausalLM"], vocab_size=50, hidden_size=16)


def run_cuts(model, device, dtype):
    cache = tlc.Cache(model.cache_requests(), 64 * 6, 3, dtype, device)
    assert sorted(cache._state_of) == [(0, "toy.s"), (2, "toy.s")]   # a state for each run of layer 0
    assert sorted(cache._kv_of) == [(1, "kv")]                       # layer 2 owns no pages: it reads layer 1's
    g = np.random.default_rng(0)
    toks = [g.integers(0, 50, n).tolist() for n in (9, 4)]
    # whole
    whole = []
    for t in toks:
        s = cache.acquire()
        whole.append(step(model, cache, [StepEntry(s, t, list(range(len(t))))]).cpu().numpy())
        cache.release(s)
    # batch: first tokens together, then one token each; the reused slots hold stale toy state
    slots = [cache.acquire() for _ in toks]
    got = [[] for _ in toks]
    first = step(model, cache, [StepEntry(s, t[:2], [0, 1]) for s, t in zip(slots, toks)]).cpu().numpy()
    got[0] += [first[0], first[1]]
    got[1] += [first[2], first[3]]
    for k in range(2, 9):
        live = [i for i, t in enumerate(toks) if k < len(t)]
        out = step(model, cache, [StepEntry(slots[i], [toks[i][k]], [0]) for i in live]).cpu().numpy()
        for r, i in enumerate(live):
            got[i].append(out[r])
    for i in range(2):
        assert np.abs(np.stack(got[i]) - whole[i]).max() < 2e-4 * np.abs(whole[i]).max()
    assert np.abs(whole[0]).max() > 1e-3


def test_toy_parts_on_the_cpu_stand_in(tmp_path, monkeypatch):
    ops_plain.install(monkeypatch, ops)
    d = write_random_model(dict(TOY), str(tmp_path / "toy"), seed=1, dtype="float32")
    assert json.load(open(os.path.join(d, "config.json")))["architectures"] == ["ToyForCausalLM"]
    run_cuts(load_model(d, "float32", "cpu"), "cpu", torch.float32)


@pytest.mark.gpu
def test_toy_parts_with_the_kernels(tmp_path):
    d = write_random_model(dict(TOY), str(tmp_path / "toy"), seed=1, dtype="float32")
    run_cuts(load_model(d, "float32", "cuda"), "cuda", torch.float32)
