"""Each part of a layer alone on the GPU against its plain function: norm, position encoding,
attention mixer, Mamba2 mixer, feed-forward and the block, in 32-bit and in bfloat16, at sizes
that no model of the other tests has.  A part gets its own cache (built from its own
cache_requests) and steps of unequal sequences: prompts in one step, then one token each."""
import numpy as np
import pytest
import torch

import tinyllama_c_b200 as tlc
from tinyllama_c_b200 import ops
from tinyllama_c_b200.cache import Cache
from tinyllama_c_b200.engine.step import StepEntry, pack
from tinyllama_c_b200.weights import load_model

from helpers import make_model_dir, read_weights
from plain import falcon_h1_plain as plain

pytestmark = pytest.mark.gpu

# two configurations that differ from each other and from the model tests' in every size and option
PARTS_1 = dict(
    architectures=["FalconH1ForCausalLM"], model_type="falcon_h1",
    vocab_size=64, hidden_size=80, num_hidden_layers=1, num_attention_heads=5, num_key_value_heads=1,
    head_dim=32, intermediate_size=104, rope_theta=50000.0, max_position_embeddings=256, rms_norm_eps=3e-6,
    tie_word_embeddings=True, attention_bias=True, mlp_bias=True, sliding_window=23,
    mamba_d_ssm=96, mamba_n_heads=3, mamba_d_head=32, mamba_n_groups=1, mamba_d_state=24, mamba_d_conv=3,
    mamba_chunk_size=8, mamba_conv_bias=False, mamba_proj_bias=True, mamba_rms_norm=True,
    mamba_norm_before_gate=True, key_multiplier=1.3, attention_in_multiplier=0.9, attention_out_multiplier=1.1,
    ssm_in_multiplier=0.8, ssm_out_multiplier=1.2, mlp_multipliers=[1.4, 0.7],
    ssm_multipliers=[0.9, 1.1, 1.2, 0.8, 1.3], eos_token_id=1)
PARTS_2 = dict(
    architectures=["FalconH1ForCausalLM"], model_type="falcon_h1",
    vocab_size=48, hidden_size=112, num_hidden_layers=1, num_attention_heads=6, num_key_value_heads=3,
    head_dim=16, intermediate_size=72, rope_theta=2000.0, max_position_embeddings=256, rms_norm_eps=1e-4,
    tie_word_embeddings=False, attention_bias=False, mlp_bias=False,
    mamba_d_ssm=80, mamba_n_heads=5, mamba_d_head=16, mamba_n_groups=5, mamba_d_state=8, mamba_d_conv=2,
    mamba_chunk_size=8, mamba_conv_bias=True, mamba_proj_bias=False, mamba_rms_norm=False,
    mamba_norm_before_gate=False, eos_token_id=1)
CONFIGS = {"one": PARTS_1, "two": PARTS_2}
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
# relative to the largest magnitude of the expected output: accumulation order in 32-bit; one or two
# roundings of a value to bfloat16 tipping the other way
TOL = {"float32": 2e-5, "bfloat16": 2e-2}
LENS, DECODED = [7, 1, 40], 3          # prompts of the three sequences, then DECODED steps of one token each


@pytest.fixture(scope="module")
def built(tmp_path_factory):
    root = tmp_path_factory.mktemp("parts")
    out = {}
    for i, (name, cfg) in enumerate(CONFIGS.items()):
        folder = make_model_dir(root, cfg, seed=70 + i, name=name)
        W = read_weights(folder)
        for dtype in DT:
            out[(name, dtype)] = (load_model(folder, dtype, "cuda"), W, cfg, plain.derived(cfg))
    return out


def rounder(dtype):
    return plain.bf16_round if dtype == "bfloat16" else plain._same


def inputs(width, dtype, seed, scale=1.0):
    """Rows for the three sequences (prompt + decoded tokens each), exactly representable in the run's type."""
    g = np.random.default_rng(seed)
    rows = [g.standard_normal((n + DECODED, width)) * scale for n in LENS]
    if dtype == "bfloat16":
        rows = [plain.bf16_round(r) for r in rows]
    return rows


def run_steps(part_forward, requests, rows, dtype, in_dtype=None, step_requests=()):
    """Feeds the sequences through part_forward(x [T, width], step, layer cache) -> [T, out]: all prompts in
    one step, then one token each; returns what came out per sequence, in order.  The cache has the run's
    type; x has in_dtype (default: the run's type)."""
    in_dtype = in_dtype or DT[dtype]
    cache = Cache({0: requests}, max_tokens=64 * 6, max_seqs=4, dtype=DT[dtype], device="cuda")
    slots = [cache.acquire() for _ in LENS]
    got = [[] for _ in LENS]
    done = [0] * len(LENS)
    for s in range(1 + DECODED):
        counts = LENS if s == 0 else [1] * len(LENS)
        entries = [StepEntry(slot, [0] * n, ()) for slot, n in zip(slots, counts)]
        starts = [cache.reserve(e.slot, len(e.tokens)) for e in entries]
        step, _, _ = pack(entries, starts, 1, "cuda", [q.rows for q in step_requests])
        cache.upload_tables()
        x = np.concatenate([rows[b][done[b]:done[b] + n] for b, n in enumerate(counts)])
        out = part_forward(torch.tensor(x, dtype=in_dtype, device="cuda"), step, cache.layer_view(0))
        torch.cuda.synchronize()
        out = out.float().cpu().numpy()
        o = 0
        for b, n in enumerate(counts):
            got[b].append(out[o:o + n])
            o += n
            done[b] += n
            cache.commit(slots[b], n)
    for slot in slots:
        cache.release(slot)
    cache.check()
    return [np.concatenate(g) for g in got]


def compare(got, want, dtype, what):
    for b, (g, w) in enumerate(zip(got, want)):
        err = np.abs(g - w).max()
        assert err <= TOL[dtype] * np.abs(w).max(), f"{what}, sequence {b}: error {err:.3e} of {np.abs(w).max():.3e}"


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("name", list(CONFIGS))
def test_norm_alone(built, name, dtype):
    model, W, cfg, d = built[(name, dtype)]
    norm = model.layers[0].mixer_norm
    x = np.random.default_rng(1).standard_normal((9, d["D"])) * 3
    out = torch.empty(9, d["D"], dtype=DT[dtype], device="cuda")
    norm.forward(torch.tensor(x, dtype=torch.float32, device="cuda"), out)
    want = plain.rms_norm(x.astype(np.float32).astype(np.float64), W["model.layers.0.input_layernorm.weight"], cfg["rms_norm_eps"])
    assert np.abs(out.float().cpu().numpy() - want).max() <= (1e-5 if dtype == "float32" else 6e-3) * np.abs(want).max()


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("name", list(CONFIGS))
def test_position_encoding_alone(built, name, dtype):
    """Rotation of q and k at each row's position, and the store of k and v at that position of the cache."""
    model, W, cfg, d = built[(name, dtype)]
    mixer = model.layers[0].mixers[0]
    H, KV, hd = d["H"], d["KV"], d["hd"]
    width = (H + 2 * KV) * hd
    rows = inputs(width, "float32", 2)

    def forward(x, step, lc):
        kv = lc.kv[mixer.cache_key]
        q = torch.empty(step.n_rows, H * hd, dtype=DT[dtype], device="cuda")
        ops.rope_kv_store(x, 0, H * hd, (H + KV) * hd, q, kv.k_pages, kv.v_pages, mixer.position.rotation_table(),
                          step.positions, step.row_seq, step.slots, kv.block_table, H, KV, hd, True)
        # read the rows' keys and values back from the pages
        pos, seq = step.positions.long(), step.row_seq.long()
        page = kv.block_table[step.slots.long()[seq], pos // 64].long()
        k = kv.k_pages[page, :, pos % 64, :].reshape(step.n_rows, KV * hd)
        v = kv.v_pages[page, :, pos % 64, :].reshape(step.n_rows, KV * hd)
        return torch.cat([q.float(), k.float(), v.float()], dim=1)

    got = run_steps(forward, mixer.cache_requests(), rows, dtype, torch.float32)
    want = []
    for r in rows:
        r = r.astype(np.float32).astype(np.float64)
        pos = np.arange(len(r))
        want.append(np.concatenate([plain.rope_neox(r[:, :H * hd], pos, H, hd, hd, cfg["rope_theta"]),
                                    plain.rope_neox(r[:, H * hd:(H + KV) * hd], pos, KV, hd, hd, cfg["rope_theta"]),
                                    r[:, (H + KV) * hd:]], axis=1))
    for g, w in zip(got, want):
        assert np.abs(g - w).max() <= (2e-5 if dtype == "float32" else 6e-3) * np.abs(w).max()


def _mixer_alone(built, name, dtype, index, plain_fn, in_mult, out_mult, what):
    model, W, cfg, d = built[(name, dtype)]
    mixer = model.layers[0].mixers[index]
    rows = inputs(d["D"], dtype, 3 + index)

    def forward(x, step, lc):
        residual = torch.zeros(step.n_rows, d["D"], dtype=torch.float32, device="cuda")
        mixer.forward(x, step, lc, residual)
        return residual

    got = run_steps(forward, mixer.cache_requests(), rows, dtype, step_requests=mixer.step_requests())
    want = [plain_fn(r * cfg.get(in_mult, 1.0), np.arange(len(r))) * cfg.get(out_mult, 1.0) for r in rows]
    compare(got, want, dtype, what)


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("name", list(CONFIGS))
def test_attention_mixer_alone(built, name, dtype):
    _, W, cfg, d = built[(name, dtype)]
    fn = lambda n, pos: plain.attention_mixer(n, W, "model.layers.0.", cfg, d, pos, rounder(dtype))
    _mixer_alone(built, name, dtype, 0, fn, "attention_in_multiplier", "attention_out_multiplier", "attention mixer")


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("name", list(CONFIGS))
def test_mamba2_mixer_alone(built, name, dtype):
    _, W, cfg, d = built[(name, dtype)]
    fn = lambda n, pos: plain.mamba2_mixer(n, W, "model.layers.0.", cfg, d, rounder(dtype))
    _mixer_alone(built, name, dtype, 1, fn, "ssm_in_multiplier", "ssm_out_multiplier", "Mamba2 mixer")


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("name", list(CONFIGS))
def test_feed_forward_alone(built, name, dtype):
    model, W, cfg, d = built[(name, dtype)]
    ffn = model.layers[0].ffn
    x = inputs(d["D"], dtype, 9)[2]
    residual = torch.zeros(len(x), d["D"], dtype=torch.float32, device="cuda")
    ffn.forward(torch.tensor(x, dtype=DT[dtype], device="cuda"), residual)
    want = plain.swiglu_mlp(x, W, "model.layers.0.", cfg, rounder(dtype))
    compare([residual.cpu().numpy()], [want], dtype, "feed-forward")


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("name", list(CONFIGS))
def test_block_alone(built, name, dtype):
    """Norm, both mixers side by side, residual, norm, feed-forward, residual: on the 32-bit residual stream."""
    model, W, cfg, d = built[(name, dtype)]
    block = model.layers[0]
    rows = inputs(d["D"], "float32", 11, scale=2.0)
    rows = [r.astype(np.float32).astype(np.float64) for r in rows]

    def forward(x32, step, lc):
        block.forward(x32, step, lc)
        return x32

    got = run_steps(forward, block.cache_requests(), rows, dtype, torch.float32)
    want = [plain.block(r, W, 0, cfg, d, np.arange(len(r)), rounder(dtype)) for r in rows]
    compare(got, want, dtype, "block")
