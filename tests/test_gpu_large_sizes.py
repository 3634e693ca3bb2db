"""One layer at the sizes of the 1.5B and 3B models with a small vocabulary against the plain
implementation, in 32-bit and in bfloat16; and the bfloat16 kernels at the full sizes of the 1.5B, 3B
and 7B models (vocabulary-sized head included) against the library's own 32-bit path.  These sizes take
the code paths that the tiny configurations do not: tcgen05 tiles, the tensor-core attention of prompts,
the chunked scan in matrix form, the weight-streaming products."""
import numpy as np
import pytest
import torch

import tinyllama_c_b200 as tlc
from tinyllama_c_b200.engine import StepEntry

from helpers import make_model_dir
from test_gpu_model import check, expected

pytestmark = pytest.mark.gpu

BASE = dict(architectures=["FalconH1ForCausalLM"], num_hidden_layers=1, num_key_value_heads=2, head_dim=128,
            rope_theta=1e11, max_position_embeddings=4096, rms_norm_eps=1e-5, mamba_n_groups=1, mamba_d_state=256,
            mamba_d_conv=4, mamba_conv_bias=True, mamba_rms_norm=True, key_multiplier=0.5, lm_head_multiplier=0.1,
            ssm_multipliers=[0.5, 0.5, 1.0, 1.0, 0.5], mlp_multipliers=[0.9, 0.5], embedding_multiplier=4.0)
SIZES = {
    "1.5B": dict(BASE, vocab_size=65536, hidden_size=2048, num_attention_heads=8, intermediate_size=4096,
                 mamba_d_ssm=3072, mamba_n_heads=48, mamba_d_head=64, tie_word_embeddings=True),
    "3B": dict(BASE, vocab_size=65536, hidden_size=2560, num_attention_heads=10, intermediate_size=8192,
               mamba_d_ssm=4096, mamba_n_heads=32, mamba_d_head=128, tie_word_embeddings=True),
    "7B": dict(BASE, vocab_size=130048, hidden_size=3072, num_attention_heads=12, intermediate_size=12288,
               mamba_d_ssm=3072, mamba_n_heads=24, mamba_d_head=128, tie_word_embeddings=False),
}


@pytest.mark.parametrize("name", ["1.5B", "3B", "7B"])
def test_bfloat16_follows_the_32_bit_path_at_model_sizes(name):
    cfg = SIZES[name]
    g = np.random.default_rng(5)
    prompts = [g.integers(0, cfg["vocab_size"], n).tolist() for n in (300, 37)]
    outs = {}
    for dtype in ("float32", "bfloat16"):
        # the same seed draws the same weights; the 32-bit model widens the bfloat16 values exactly
        model = tlc.random_model(cfg, seed=3, dtype="bfloat16", std=0.02, run_dtype=dtype)
        llm = tlc.LLM(model, max_tokens=1024, max_seqs=2)
        slots = [llm.cache.acquire() for _ in prompts]
        rows = [llm.step([StepEntry(s, p[:-3], [len(p) - 4]) for s, p in zip(slots, prompts)]).cpu().numpy()]
        for k in range(3, 0, -1):                      # three single-token steps of both sequences
            rows.append(llm.step([StepEntry(s, [p[-k]], [0]) for s, p in zip(slots, prompts)]).cpu().numpy())
        outs[dtype] = np.concatenate(rows)
        del llm, model
        torch.cuda.empty_cache()
    ref, got = outs["float32"], outs["bfloat16"]
    scale = np.abs(ref).max()
    assert scale > 1e-3
    err = np.abs(ref - got)
    # inputs of every product and q/k/v are rounded to bfloat16 (2^-9 each): a few per cent of the
    # logits' scale at the end of a layer; a wrong tile, page or chunk is of the order of the scale
    assert err.max() <= 0.06 * scale, f"{name}: max |bf16 - f32| = {err.max():.3e} at scale {scale:.3e}"
    assert err.mean() <= 0.01 * scale, f"{name}: mean |bf16 - f32| = {err.mean():.3e} at scale {scale:.3e}"
    top_ref, top_got = ref.argmax(1), got.argmax(1)
    margin = np.sort(ref, axis=1)
    clear = (margin[:, -1] - margin[:, -2]) > 0.05 * scale
    assert (top_ref[clear] == top_got[clear]).all()



@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["1.5B", "3B"])
def test_one_layer_at_model_sizes_against_the_plain_implementation(tmp_path, name, dtype):
    """head size 128, Mamba heads of 64 (1.5B) or 128 (3B) with a state of 256, the real widths; a vocabulary
    of 512 keeps the plain implementation quick.  A 300-token and a 37-token prompt together, then three
    single-token steps of both."""
    cfg = dict(SIZES[name], vocab_size=512, max_position_embeddings=512)
    d = make_model_dir(tmp_path, cfg, seed=11, std=0.02, name="layer")
    g = np.random.default_rng(6)
    prompts = [g.integers(0, cfg["vocab_size"], n).tolist() for n in (300, 37)]
    want = [expected(d, p, dtype) for p in prompts]
    llm = tlc.LLM(d, dtype=dtype, max_tokens=1024, max_seqs=2)
    slots = [llm.cache.acquire() for _ in prompts]
    got = llm.step([StepEntry(s, p[:-3], [0, len(p) - 4]) for s, p in zip(slots, prompts)]).cpu().numpy()
    for i, p in enumerate(prompts):
        check(got[2 * i:2 * i + 2], want[i][[0, len(p) - 4]], dtype, f"{name} layer, prompt {i}")
    for k in range(3, 0, -1):
        got = llm.step([StepEntry(s, [p[-k]], [0]) for s, p in zip(slots, prompts)]).cpu().numpy()
        for i, p in enumerate(prompts):
            check(got[i:i + 1], want[i][len(p) - k:len(p) - k + 1], dtype, f"{name} layer, token -{k} of prompt {i}")


@pytest.mark.parametrize("n_seqs", [24, 40])
def test_steps_of_17_to_64_sequences_at_model_sizes_against_the_plain_implementation(tmp_path, n_seqs):
    """One layer at the 1.5B sizes in bfloat16 with 24 and with 40 sequences: their short prompts in one step
    (some 300 to 500 rows: the tiled products), then two single-token steps of all of them together, which is where
    products of 17..64 rows run (weights on the wide side of the tensor-core instruction, a tile's K shared among
    the blocks of a cluster: the wide outputs with 24 rows, the narrow ones too with 40)."""
    cfg = dict(SIZES["1.5B"], vocab_size=512, max_position_embeddings=512)
    d = make_model_dir(tmp_path, cfg, seed=12, std=0.02, name="layer")
    g = np.random.default_rng(7)
    prompts = [g.integers(0, cfg["vocab_size"], int(n)).tolist() for n in g.integers(6, 20, n_seqs)]
    want = [expected(d, p, "bfloat16") for p in prompts]
    llm = tlc.LLM(d, dtype="bfloat16", max_tokens=64 * n_seqs, max_seqs=n_seqs)
    slots = [llm.cache.acquire() for _ in prompts]
    got = llm.step([StepEntry(s, p[:-2], [len(p) - 3]) for s, p in zip(slots, prompts)]).cpu().numpy()
    for i, p in enumerate(prompts):
        check(got[i:i + 1], want[i][len(p) - 3:len(p) - 2], "bfloat16", f"{n_seqs} sequences, prompt {i}")
    for k in (2, 1):
        got = llm.step([StepEntry(s, [p[-k]], [0]) for s, p in zip(slots, prompts)]).cpu().numpy()
        for i, p in enumerate(prompts):
            check(got[i:i + 1], want[i][len(p) - k:len(p) - k + 1], "bfloat16", f"{n_seqs} sequences, token -{k} of {i}")
