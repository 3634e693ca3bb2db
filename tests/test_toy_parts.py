"""Parts defined here, outside the package, can be registered, built into a model and stepped:
a mixer with state of its own that asks the step function for chunks of 32 rows, a feed-forward
with routing, a position encoding that is another rotation and one that is no rotation at all,
and an architecture that uses them -- one layer twice in the run order, one layer reading
another's cache.  None of this touches the package's files.  The toy parts compute with PyTorch (they
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
from tinyllama_c_b200.parts import (ChunkRequest, KVRequest, LayerRun, LayerSpec, Part, PartSpec, Position, StateRequest,
                                    WeightSpec, register_feed_forward, register_mixer, register_position)
from tinyllama_c_b200.weights import load_model, write_random_model

from plain import ops_plain


@register_mixer("toy_decay")
class ToyDecayMixer(Part):
    """s_t = decay * s_{t-1} + W_in x_t (per sequence, state [width]); out = W_out s_t.  Long prompts are
    scanned chunk by chunk from the table of 32-row chunks that the step function builds on request."""
    CHUNK = 32

    def __init__(self, hidden, width, prefix, decay=0.5):
        self.hidden, self.width, self.prefix, self.decay = hidden, width, prefix, decay

    def weight_specs(self):
        return [WeightSpec(self.prefix + "w_in", (self.width, self.hidden)),
                WeightSpec(self.prefix + "w_out", (self.hidden, self.width))]

    def cache_requests(self):
        return [StateRequest("toy.s", (self.width,))]

    def step_requests(self):
        return [ChunkRequest(self.CHUNK)]

    def bind(self, tensors, dtype, device):
        self.w_in = tensors[self.prefix + "w_in"].to(device=device, dtype=torch.float32)
        self.w_out = tensors[self.prefix + "w_out"].to(device=device, dtype=torch.float32)

    def forward(self, normed, step_info, cache, residual):
        state = cache.state["toy.s"]
        u = normed.float() @ self.w_in.T
        table = step_info.chunks[self.CHUNK]               # the step function made it because this part asked
        longest = max(step_info.host_lens)
        assert (table is None) == (longest <= self.CHUNK)
        if table is None:
            bounds = np.concatenate([[0], np.cumsum(step_info.host_lens)])
            chunks = [(b, int(bounds[b]), int(bounds[b + 1])) for b in range(step_info.n_seqs)]
        else:
            seg_start, seg_seq, seq_seg_start = (t.cpu().tolist() for t in table)
            assert seq_seg_start[-1] == len(seg_seq) and seg_start[-1] == step_info.n_rows
            assert all(seg_start[c + 1] - seg_start[c] <= self.CHUNK for c in range(len(seg_seq)))
            chunks = [(seg_seq[c], seg_start[c], seg_start[c + 1]) for c in range(len(seg_seq))]
        carried = {}
        for b, t0, t1 in chunks:                           # chunks of a sequence come in order
            slot = step_info.host_slots[b]
            if b not in carried:
                carried[b] = state[slot].clone() if step_info.host_start[b] > 0 else torch.zeros_like(state[slot])
            s = carried[b]
            for t in range(t0, t1):
                s = self.decay * s + u[t]
                residual[t] += s @ self.w_out.T
            carried[b] = s
        for b, s in carried.items():
            state[step_info.host_slots[b]] = s


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


@register_position("toy_half_steps")
class ToyScaledRotary(Position):
    """Another rotation: positions counted in halves.  A rotation is described by its table."""

    def __init__(self, head_dim, theta):
        self.head_dim, self.theta = head_dim, theta

    def bind(self, tensors, dtype, device):
        i = torch.arange(self.head_dim // 2, dtype=torch.float64)
        self.table = (0.5 / self.theta ** (2.0 * i / self.head_dim)).to(torch.float32).to(device).contiguous()

    def rotation_table(self):
        return self.table


@register_position("toy_log_scale")
class ToyLogScale(Position):
    """No rotation at all: every query is scaled by 1 + log(1 + position) / 4 and every key gets a learned
    per-head offset.  It changes q and k of the 32-bit projection in place; the mixer stores and attends."""

    def __init__(self, head_dim, n_kv, prefix):
        self.head_dim, self.n_kv, self.prefix = head_dim, n_kv, prefix

    def weight_specs(self):
        return [WeightSpec(self.prefix + "key_offset", (self.n_kv, self.head_dim))]

    def bind(self, tensors, dtype, device):
        self.offset = tensors[self.prefix + "key_offset"].to(device=device, dtype=torch.float32).reshape(-1)

    def transform(self, qkv, q_off, k_off, step_info, n_heads, n_kv, head_dim):
        scale = 1.0 + torch.log1p(step_info.positions.to(torch.float32)) / 4.0
        qkv[:, q_off:q_off + n_heads * head_dim] *= scale[:, None]
        qkv[:, k_off:k_off + n_kv * head_dim] += self.offset


@dataclass(frozen=True)
class ToyConfig(ModelConfig):
    vocab_size: int
    hidden_size: int
    eps: float = 1e-5
    initializer_range: float = 0.3


def build_toy(cfg: ToyConfig) -> Model:
    D = cfg.hidden_size
    norm = lambda n: PartSpec("norm", "rmsnorm", dict(width=D, eps=cfg.eps, weight_name=n))
    pos_args = {"none": dict(head_dim=D // 2), "toy_half_steps": dict(head_dim=D // 2, theta=100.0),
                "toy_log_scale": dict(head_dim=D // 2, n_kv=1, prefix="l3.pos.")}
    att = lambda l, pos: PartSpec("mixer", "attention", dict(
        hidden=D, n_heads=2, n_kv_heads=1, head_dim=D // 2, prefix=f"l{l}.att.",
        position=PartSpec("position", pos, pos_args[pos])))
    layers = [
        LayerSpec(norm("l0.n1"), (PartSpec("mixer", "toy_decay", dict(hidden=D, width=6, prefix="l0.toy.")),),
                  norm("l0.n2"), PartSpec("feed_forward", "toy_routed", dict(hidden=D, prefix="l0.moe."))),
        LayerSpec(norm("l1.n1"), (att(1, "toy_half_steps"),), norm("l1.n2"),
                  PartSpec("feed_forward", "swiglu", dict(hidden=D, intermediate=2 * D, prefix="l1.ffn."))),
        LayerSpec(norm("l2.n1"), (att(2, "none"),), None, None),
        LayerSpec(norm("l3.n1"), (att(3, "toy_log_scale"),), None, None),
    ]
    # layer 0 runs twice (one set of weights, a state per run); layer 2 reads the keys and values
    # that layer 1 (entry 1 of the run order) stored, without storing its own
    schedule = [LayerRun(0), LayerRun(1), LayerRun(0), LayerRun(2, cache=1), LayerRun(3)]
    return Model(cfg, layers, schedule, norm("final"), embed_name="emb", head_name=None, vocab=cfg.vocab_size, hidden=D)


tlc.register_architecture("ToyForCausalLM", ToyConfig, build_toy)
TOY = dict(architectures=["ToyForCausalLM"], vocab_size=50, hidden_size=16)


def run_cuts(model, device, dtype):
    cache = tlc.Cache(model.cache_requests(), 64 * 6, 3, dtype, device)
    assert sorted(cache._state_of) == [(0, "toy.s"), (2, "toy.s")]   # a state for each run of layer 0
    assert sorted(cache._kv_of) == [(1, "kv"), (4, "kv")]            # layer 2 owns no pages: it reads layer 1's
    assert model.chunk_rows == (ToyDecayMixer.CHUNK,)                # the only chunk table a step has to build
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
    # a prompt of 75 rows is cut into chunks of 32, 32 and 11 rows for the toy mixer; the same tokens in
    # pieces of 40 + 35 (cut into 32 + 8 and 32 + 3) must give the same logits
    long = g.integers(0, 50, 75).tolist()
    s = cache.acquire()
    once = step(model, cache, [StepEntry(s, long, [39, 74])]).cpu().numpy()
    cache.release(s)
    s = cache.acquire()
    a = step(model, cache, [StepEntry(s, long[:40], [39])]).cpu().numpy()
    b = step(model, cache, [StepEntry(s, long[40:], [34])]).cpu().numpy()
    cache.release(s)
    assert np.abs(np.concatenate([a, b]) - once).max() < 2e-4 * np.abs(once).max()


def test_a_state_mixer_cannot_read_another_entry_s_cache():
    cfg = tlc.config.config_from_dict(dict(TOY))
    model = build_toy(cfg)
    with pytest.raises(ValueError, match="state of its own"):
        Model(cfg, [b.spec for b in model.layers], [LayerRun(0), LayerRun(0, cache=0)],
              PartSpec("norm", "rmsnorm", dict(width=16, eps=1e-5, weight_name="final")), embed_name="emb",
              head_name=None, vocab=50, hidden=16)


def test_toy_parts_on_the_cpu_stand_in(tmp_path, monkeypatch):
    ops_plain.install(monkeypatch, ops)
    d = write_random_model(dict(TOY), str(tmp_path / "toy"), seed=1, dtype="float32")
    assert json.load(open(os.path.join(d, "config.json")))["architectures"] == ["ToyForCausalLM"]
    run_cuts(load_model(d, "float32", "cpu"), "cpu", torch.float32)


@pytest.mark.gpu
def test_toy_parts_with_the_kernels(tmp_path):
    d = write_random_model(dict(TOY), str(tmp_path / "toy"), seed=1, dtype="float32")
    run_cuts(load_model(d, "float32", "cuda"), "cuda", torch.float32)
