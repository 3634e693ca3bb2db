"""Tiny Falcon-H1 configurations of the test-suite.  A and B differ in every size and
option; C is B's shape with the Mamba norm on, norm before gate, and a sliding window."""

TINY_A = dict(
    architectures=["FalconH1ForCausalLM"], model_type="falcon_h1",
    vocab_size=256, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
    head_dim=16, intermediate_size=128, rope_theta=10000.0, max_position_embeddings=256, rms_norm_eps=1e-5,
    tie_word_embeddings=True, attention_bias=False, mlp_bias=False,
    mamba_d_ssm=64, mamba_n_heads=4, mamba_d_head=16, mamba_n_groups=1, mamba_d_state=16, mamba_d_conv=4,
    mamba_chunk_size=8, mamba_conv_bias=True, mamba_proj_bias=False, mamba_rms_norm=True,
    mamba_norm_before_gate=False, eos_token_id=11)

TINY_B = dict(
    architectures=["FalconH1ForCausalLM"], model_type="falcon_h1",
    vocab_size=384, hidden_size=96, num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=3,
    head_dim=24, intermediate_size=160, rope_theta=1000000.0, max_position_embeddings=512, rms_norm_eps=1e-6,
    tie_word_embeddings=False, attention_bias=True, mlp_bias=True,
    mamba_d_ssm=144, mamba_n_heads=6, mamba_d_head=24, mamba_n_groups=2, mamba_d_state=32, mamba_d_conv=3,
    mamba_chunk_size=16, mamba_conv_bias=False, mamba_proj_bias=True, mamba_rms_norm=False,
    mamba_norm_before_gate=True,
    embedding_multiplier=5.0, lm_head_multiplier=0.5, key_multiplier=0.7, attention_in_multiplier=1.2,
    attention_out_multiplier=0.8, ssm_in_multiplier=1.1, ssm_out_multiplier=0.9, mlp_multipliers=[0.6, 1.3],
    ssm_multipliers=[0.5, 1.5, 0.8, 1.2, 0.7], eos_token_id=[7, 9])

TINY_C = dict(TINY_B, mamba_rms_norm=True, mamba_norm_before_gate=True, sliding_window=40, mamba_conv_bias=True,
              num_key_value_heads=1, mamba_d_conv=2)

# head size 64: the tensor-core attention of prompts; state size 64; query width != hidden size
TINY_D = dict(
    architectures=["FalconH1ForCausalLM"], model_type="falcon_h1",
    vocab_size=320, hidden_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
    head_dim=64, intermediate_size=192, rope_theta=100000.0, max_position_embeddings=512, rms_norm_eps=1e-5,
    tie_word_embeddings=True, mamba_d_ssm=128, mamba_n_heads=2, mamba_d_head=64, mamba_n_groups=1,
    mamba_d_state=64, mamba_d_conv=4, mamba_conv_bias=True, mamba_rms_norm=True, key_multiplier=0.5,
    ssm_multipliers=[1.0, 0.5, 1.0, 1.0, 0.5], eos_token_id=3)

ALL = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D}
