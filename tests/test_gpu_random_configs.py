"""Configurations drawn at random (fixed seeds) from the sizes and options the kernels claim to take:
head sizes in steps of 16, any number of heads and groups, widths that are no power of two, 2 to 5
convolution taps, windows, every bias and norm option, multipliers.  Three sequences of unequal
length start together (prompts in one step, then six tokens one by one) and are compared with the
plain implementation in 32-bit and in bfloat16."""
import numpy as np
import pytest

import tinyllama_c_b200 as tlc
from tinyllama_c_b200.engine import StepEntry

from helpers import make_model_dir, plain_logits, random_tokens

pytestmark = pytest.mark.gpu


def draw(rng):
    hd = int(rng.choice([16, 32, 48, 64, 80, 128]))
    kv, per = int(rng.choice([1, 2, 3])), int(rng.choice([1, 2, 4, 5, 8]))
    heads = int(rng.choice([2, 3, 4, 6]))
    groups = int(rng.choice([g for g in (1, 2, 3) if heads % g == 0]))
    p = int(rng.choice([8, 16, 24, 64]))
    return dict(
        architectures=["FalconH1ForCausalLM"], model_type="falcon_h1", vocab_size=int(rng.choice([100, 257, 512])),
        hidden_size=int(rng.choice([64, 72, 96, 136, 200])), num_hidden_layers=int(rng.choice([1, 2, 3])),
        num_attention_heads=kv * per, num_key_value_heads=kv, head_dim=hd,
        intermediate_size=int(rng.choice([40, 104, 136, 256])), rope_theta=float(rng.choice([1e4, 1e6, 1e11])),
        max_position_embeddings=1024, rms_norm_eps=float(rng.choice([1e-5, 1e-6])),
        tie_word_embeddings=bool(rng.integers(2)), attention_bias=bool(rng.integers(2)), mlp_bias=bool(rng.integers(2)),
        sliding_window=(int(rng.choice([20, 70, 130])) if rng.integers(3) == 0 else None),
        mamba_d_ssm=heads * p, mamba_n_heads=heads, mamba_d_head=p, mamba_n_groups=groups,
        mamba_d_state=int(rng.choice([8, 16, 40, 64, 128])), mamba_d_conv=int(rng.choice([2, 3, 4, 5])), mamba_chunk_size=8,
        mamba_conv_bias=bool(rng.integers(2)), mamba_proj_bias=bool(rng.integers(2)), mamba_rms_norm=bool(rng.integers(2)),
        mamba_norm_before_gate=bool(rng.integers(2)), key_multiplier=float(rng.choice([1.0, 0.7])),
        attention_in_multiplier=float(rng.choice([1.0, 1.2])), attention_out_multiplier=float(rng.choice([1.0, 0.8])),
        ssm_in_multiplier=float(rng.choice([1.0, 1.1])), ssm_out_multiplier=float(rng.choice([1.0, 0.9])),
        mlp_multipliers=[float(rng.choice([1.0, 0.6])), float(rng.choice([1.0, 1.3]))],
        ssm_multipliers=[float(x) for x in rng.choice([0.5, 1.0, 1.5], 5)], eos_token_id=1)


@pytest.mark.parametrize("seed", [11, 12, 13, 14, 15, 16])
def test_a_random_configuration(tmp_path, seed):
    rng = np.random.default_rng(seed)
    cfg = draw(rng)
    folder = make_model_dir(tmp_path, cfg, seed=seed, name="m")
    lens = [int(x) for x in rng.choice([1, 5, 33, 64, 65, 150, 300], 3)]
    toks = [random_tokens(cfg["vocab_size"], n + 6, 7 * seed + i) for i, n in enumerate(lens)]
    exact = [plain_logits(folder, t, "float32") for t in toks]
    for dtype in ("float32", "bfloat16"):
        llm = tlc.LLM(folder, dtype=dtype, max_tokens=64 * 24, max_seqs=4)
        slots = [llm.cache.acquire() for _ in lens]
        got = [[] for _ in lens]
        out = llm.step([StepEntry(s, t[:n], list(range(n))) for s, t, n in zip(slots, toks, lens)]).cpu().numpy()
        o = 0
        for b, n in enumerate(lens):
            got[b].append(out[o:o + n])
            o += n
        for k in range(6):
            out = llm.step([StepEntry(s, [t[n + k]], [0]) for s, t, n in zip(slots, toks, lens)]).cpu().numpy()
            for b in range(len(lens)):
                got[b].append(out[b:b + 1])
        for b in range(len(lens)):
            g = np.concatenate(got[b])
            if dtype == "float32":
                allowed = 1e-4 * np.abs(exact[b]).max()
                err = np.abs(g - exact[b]).max()
            else:
                # the engine must be as close to the plain model of a bfloat16 engine as that model is to exact arithmetic
                model = plain_logits(folder, toks[b], "bfloat16")
                allowed = np.abs(model - exact[b]).max()
                err = np.abs(g - model).max()
            assert err <= allowed, f"seed {seed} {dtype} sequence {b} (lengths {lens}): error {err:.3e}, allowed {allowed:.3e}; {cfg}"
