"""Configuration reading, the registry, weight checking and the random-weights mode."""
import json
import os

import pytest
import torch

import tinyllama_c_b200 as tlc
from tinyllama_c_b200.config import ConfigError, FalconH1Config, config_from_dict, load_config
from tinyllama_c_b200.weights import WeightError, build_model, load_file, load_model, save_file, write_random_model
from tinyllama_c_b200.weights.safetensors_io import SafetensorsError

import configs


def test_config_reads_every_key_and_derives_sizes():
    c = config_from_dict(dict(configs.TINY_B))
    assert isinstance(c, FalconH1Config)
    assert (c.hidden_size, c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (96, 6, 3, 24)
    assert (c.mamba_d_ssm, c.mamba_n_heads, c.mamba_d_head, c.mamba_n_groups, c.mamba_d_state, c.mamba_d_conv) == \
        (144, 6, 24, 2, 32, 3)
    assert c.mamba_conv_dim == 144 + 2 * 2 * 32 and c.mamba_proj_dim == 144 + c.mamba_conv_dim + 6
    assert c.ssm_multipliers == (0.5, 1.5, 0.8, 1.2, 0.7) and c.mlp_multipliers == (0.6, 1.3)
    assert c.rms_norm_eps == 1e-6 and c.rope_theta == 1e6 and not c.tie_word_embeddings
    assert c.stop_token_ids == (7, 9)
    assert config_from_dict(c.to_dict()) == c


def test_config_defaults():
    raw = dict(architectures=["FalconH1ForCausalLM"], vocab_size=100, hidden_size=64, intermediate_size=96,
               num_hidden_layers=1, num_attention_heads=4, mamba_n_heads=8, mamba_d_state=16)
    c = config_from_dict(raw)
    assert c.num_key_value_heads == 4 and c.head_dim == 16 and c.mamba_d_ssm == 128 and c.mamba_d_head == 16
    assert c.rope_theta == 10000.0 and c.sliding_window is None and c.stop_token_ids == ()


@pytest.mark.parametrize("change,needle", [
    (dict(num_key_value_heads=3), "multiple of"),
    (dict(mamba_d_head=10), "must equal mamba_d_ssm"),
    (dict(mamba_n_groups=3), "multiple of"),
    (dict(vocab_size="big"), "positive integer"),
    (dict(ssm_multipliers=[1, 2]), "list of 5"),
    (dict(hidden_act="gelu"), "hidden_act"),
    (dict(tie_word_embeddings="yes"), "true or false"),
])
def test_config_errors(change, needle):
    with pytest.raises(ConfigError, match=needle):
        config_from_dict(dict(configs.TINY_A, **change))


def test_config_missing_key_and_unknown_architecture(tmp_path):
    raw = dict(configs.TINY_A)
    del raw["mamba_d_state"], raw["vocab_size"]
    with pytest.raises(ConfigError, match="mamba_d_state") as e:
        config_from_dict(raw)
    assert "vocab_size" in str(e.value)
    with pytest.raises(ConfigError, match="unknown architecture 'LlamaForCausalLM'.*FalconH1ForCausalLM"):
        config_from_dict(dict(configs.TINY_A, architectures=["LlamaForCausalLM"]))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        load_config(str(tmp_path))
    with pytest.raises(ConfigError, match="no such file"):
        load_config(str(tmp_path / "nowhere"))


def test_random_model_folder_and_dtypes(tmp_path):
    d = write_random_model(dict(configs.TINY_A), str(tmp_path / "a"), seed=1)
    assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
    t = load_file(os.path.join(d, "model.safetensors"))
    assert t["model.embed_tokens.weight"].dtype == torch.bfloat16
    assert t["model.layers.0.mamba.A_log"].dtype == torch.float32            # per-head constants stay 32-bit
    assert "lm_head.weight" not in t                                          # tied
    # the same seed gives the same tensors; a tensor does not depend on which others exist
    d2 = write_random_model(dict(configs.TINY_A, num_hidden_layers=1), str(tmp_path / "b"), seed=1)
    t2 = load_file(os.path.join(d2, "model.safetensors"))
    assert all(torch.equal(t[k], t2[k]) for k in t2)
    d3 = write_random_model(dict(configs.TINY_A), str(tmp_path / "c"), seed=2)
    assert not torch.equal(t["model.embed_tokens.weight"], load_file(os.path.join(d3, "model.safetensors"))["model.embed_tokens.weight"])
    # the safetensors package reads what the writer wrote
    from safetensors.torch import load_file as ref_load
    r = ref_load(os.path.join(d, "model.safetensors"))
    assert set(r) == set(t) and all(torch.equal(r[k], t[k]) for k in t)


def test_load_keeps_bfloat16_and_32_bit_tensors(tmp_path):
    d = write_random_model(dict(configs.TINY_B), str(tmp_path / "m"), seed=3)
    m = load_model(d, "bfloat16", "cpu")
    att = m.layers[0].mixers[0]
    assert att.qkv.weight.dtype == torch.bfloat16 and att.qkv.weight.shape == ((6 + 3 + 3) * 24, 96)
    assert m.layers[0].mixers[1].A.dtype == torch.float32
    # a matrix stored in 32-bit stays so in a bfloat16 run
    t = dict(load_file(os.path.join(d, "model.safetensors")))
    t["lm_head.weight"] = t["lm_head.weight"].float()
    save_file(t, os.path.join(d, "model.safetensors"))
    m = load_model(d, "bfloat16", "cpu")
    assert m.head.weight.dtype == torch.float32 and m.embed_table.dtype == torch.bfloat16
    assert load_model(d, "float32", "cpu").embed_table.dtype == torch.float32


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = write_random_model(dict(configs.TINY_A), str(tmp_path / "m"), seed=4)
    path = os.path.join(d, "model.safetensors")
    t = dict(load_file(path))
    del t["model.layers.1.mamba.dt_bias"], t["model.final_layernorm.weight"]
    t["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(10, 64, dtype=torch.bfloat16)
    t["model.layers.0.extra.weight"] = torch.zeros(3)
    save_file(t, path)
    with pytest.raises(WeightError) as e:
        load_model(d, "float32", "cpu")
    msg = str(e.value)
    assert "missing tensors (2)" in msg and "model.layers.1.mamba.dt_bias" in msg and "model.final_layernorm.weight" in msg
    assert "unexpected tensors (1)" in msg and "model.layers.0.extra.weight" in msg
    assert "wrong shapes (1)" in msg and "expected [64, 64], found [10, 64]" in msg


def test_truncated_and_malformed_files(tmp_path):
    d = write_random_model(dict(configs.TINY_A), str(tmp_path / "m"), seed=5)
    path = os.path.join(d, "model.safetensors")
    raw = open(path, "rb").read()
    open(path, "wb").write(raw[: len(raw) // 2])
    with pytest.raises(WeightError, match="data range"):
        load_model(d, "float32", "cpu")
    open(path, "wb").write(b"\x05")
    with pytest.raises(WeightError, match="too short"):
        load_model(d, "float32", "cpu")
    os.remove(path)
    with pytest.raises(WeightError, match="neither model.safetensors"):
        load_model(d, "float32", "cpu")


def test_kernels_refuse_cpu_tensors():
    from tinyllama_c_b200 import ops
    with pytest.raises(ops.KernelError, match="no CPU path"):
        ops.swiglu(torch.zeros(2, 4), torch.zeros(2, 2))
