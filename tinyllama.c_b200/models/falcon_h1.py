"""Falcon-H1: every layer runs an attention mixer and a Mamba2 mixer in parallel on the
same normed input, then a SwiGLU feed-forward (CodeClaper/tinyllama.c falcon_h1.c:246-255).

This file only turns a FalconH1Config into data: one LayerSpec per layer (which parts,
with which sizes and constants, under which tensor names) and the tensor names of the
embedding, the final norm and the head.  Tensor names follow the architecture's
checkpoints (the reference binds blk.N.attn_q ... ssm_in ... ffn_gate, core.c:1092-1113).
"""
from __future__ import annotations

from typing import List

from ..config.base import register_architecture
from ..config.falcon_h1 import FalconH1Config
from ..parts.base import LayerSpec, PartSpec
from .model import Model


def layer_specs(cfg: FalconH1Config) -> List[LayerSpec]:
    specs = []
    for l in range(cfg.num_hidden_layers):
        p = f"model.layers.{l}."
        norm = lambda name: PartSpec("norm", "rmsnorm", dict(width=cfg.hidden_size, eps=cfg.rms_norm_eps,
                                                             weight_name=p + name))
        attention = PartSpec("mixer", "attention", dict(
            hidden=cfg.hidden_size, n_heads=cfg.num_attention_heads, n_kv_heads=cfg.num_key_value_heads,
            head_dim=cfg.head_dim, prefix=p + "self_attn.", bias=cfg.attention_bias, window=cfg.sliding_window,
            position=PartSpec("position", "rope_neox", dict(head_dim=cfg.head_dim, theta=cfg.rope_theta)),
            in_scale=cfg.attention_in_multiplier, out_scale=cfg.attention_out_multiplier,
            key_scale=cfg.key_multiplier))
        mamba = PartSpec("mixer", "mamba2", dict(
            hidden=cfg.hidden_size, d_ssm=cfg.mamba_d_ssm, n_heads=cfg.mamba_n_heads, d_head=cfg.mamba_d_head,
            n_groups=cfg.mamba_n_groups, d_state=cfg.mamba_d_state, d_conv=cfg.mamba_d_conv, prefix=p + "mamba.",
            eps=cfg.rms_norm_eps, conv_bias=cfg.mamba_conv_bias, proj_bias=cfg.mamba_proj_bias,
            rms_norm=cfg.mamba_rms_norm, norm_before_gate=cfg.mamba_norm_before_gate,
            slice_scales=cfg.ssm_multipliers, in_scale=cfg.ssm_in_multiplier, out_scale=cfg.ssm_out_multiplier))
        ffn = PartSpec("feed_forward", "swiglu", dict(
            hidden=cfg.hidden_size, intermediate=cfg.intermediate_size, prefix=p + "feed_forward.",
            bias=cfg.mlp_bias, gate_scale=cfg.mlp_multipliers[0], down_scale=cfg.mlp_multipliers[1]))
        # residual order (x + attention) + mamba, falcon_h1.c:372-375
        specs.append(LayerSpec(norm("input_layernorm.weight"), (attention, mamba),
                               norm("pre_ff_layernorm.weight"), ffn))
    return specs


def build(cfg: FalconH1Config) -> Model:
    final_norm = PartSpec("norm", "rmsnorm", dict(width=cfg.hidden_size, eps=cfg.rms_norm_eps,
                                                  weight_name="model.final_layernorm.weight"))
    return Model(cfg, layer_specs(cfg), None, final_norm, embed_name="model.embed_tokens.weight",
                 head_name=None if cfg.tie_word_embeddings else "lm_head.weight", vocab=cfg.vocab_size,
                 hidden=cfg.hidden_size, embed_scale=cfg.embedding_multiplier, head_scale=cfg.lm_head_multiplier)


register_architecture("FalconH1ForCausalLM", FalconH1Config, build)
