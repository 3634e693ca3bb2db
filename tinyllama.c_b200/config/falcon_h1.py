"""Falcon-H1 configuration: every key of the architecture's config.json.

CodeClaper/tinyllama.c reads the attention geometry with fallbacks at core.c:1611-1636
and the Mamba2 geometry at falcon_h1.c:108-128 (inner size, state size, group count,
head count, conv taps, rope base).  It has no field for the norm eps (a constant,
def.h:10), for the muP multipliers or for the bias / norm options; those are keys here.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional, Tuple, Union

from .base import ConfigError, ModelConfig


def _is_int(v: Any) -> bool:
    return isinstance(v, int) and not isinstance(v, bool)


def _is_num(v: Any) -> bool:
    return isinstance(v, (int, float)) and not isinstance(v, bool)


@dataclass(frozen=True)
class FalconH1Config(ModelConfig):
    # sizes without a default are required keys
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    mamba_n_heads: int
    mamba_d_state: int
    num_key_value_heads: Optional[int] = None          # default: num_attention_heads (core.c:1616-1619)
    head_dim: Optional[int] = None                     # default: hidden/heads (core.c:1621-1631)
    max_position_embeddings: int = 8192
    rope_theta: float = 10000.0                        # falcon_h1.c:126-128
    rms_norm_eps: float = 1e-5
    sliding_window: Optional[int] = None               # window of op_attn (cpu_op.c:1019-1022); none = full causal
    tie_word_embeddings: bool = False                  # core.c:1246-1249
    attention_bias: bool = False
    mlp_bias: bool = False
    hidden_act: str = "silu"
    mamba_d_ssm: Optional[int] = None                  # default: mamba_expand * hidden (falcon_h1.c:111)
    mamba_expand: int = 2
    mamba_d_head: Union[int, str, None] = "auto"       # "auto": d_ssm / n_heads (falcon_h1.c:123)
    mamba_n_groups: int = 1
    mamba_d_conv: int = 4
    mamba_chunk_size: int = 128                        # a tiling hint of the chunked scan, not math
    mamba_conv_bias: bool = True
    mamba_proj_bias: bool = False
    mamba_rms_norm: bool = True
    mamba_norm_before_gate: bool = False
    embedding_multiplier: float = 1.0
    lm_head_multiplier: float = 1.0
    key_multiplier: float = 1.0
    attention_in_multiplier: float = 1.0
    attention_out_multiplier: float = 1.0
    ssm_in_multiplier: float = 1.0
    ssm_out_multiplier: float = 1.0
    mlp_multipliers: Tuple[float, float] = (1.0, 1.0)              # (gate pre-activation, down output)
    ssm_multipliers: Tuple[float, float, float, float, float] = (1.0,) * 5   # z, x, B, C, dt slices of in_proj
    bos_token_id: Optional[int] = None
    eos_token_id: Union[int, Tuple[int, ...], None] = None
    pad_token_id: Optional[int] = None
    torch_dtype: str = "bfloat16"
    model_type: str = "falcon_h1"
    initializer_range: float = 0.02

    def validate(self) -> None:
        s = lambda k, v: object.__setattr__(self, k, v)
        bad = []
        for k in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                  "num_attention_heads", "mamba_n_heads", "mamba_d_state", "mamba_n_groups",
                  "mamba_d_conv", "mamba_expand", "max_position_embeddings", "mamba_chunk_size"):
            v = getattr(self, k)
            if not _is_int(v) or v <= 0:
                bad.append(f"'{k}' must be a positive integer, got {v!r}")
        for k in ("num_key_value_heads", "head_dim", "mamba_d_ssm", "sliding_window"):
            v = getattr(self, k)
            if v is not None and (not _is_int(v) or v <= 0):
                bad.append(f"'{k}' must be a positive integer or null, got {v!r}")
        for k in ("rope_theta", "rms_norm_eps", "embedding_multiplier", "lm_head_multiplier",
                  "key_multiplier", "attention_in_multiplier", "attention_out_multiplier",
                  "ssm_in_multiplier", "ssm_out_multiplier"):
            v = getattr(self, k)
            if not _is_num(v):
                bad.append(f"'{k}' must be a number, got {v!r}")
        for k in ("tie_word_embeddings", "attention_bias", "mlp_bias", "mamba_conv_bias",
                  "mamba_proj_bias", "mamba_rms_norm", "mamba_norm_before_gate"):
            if not isinstance(getattr(self, k), bool):
                bad.append(f"'{k}' must be true or false, got {getattr(self, k)!r}")
        for k, n in (("mlp_multipliers", 2), ("ssm_multipliers", 5)):
            v = getattr(self, k)
            if not (isinstance(v, (list, tuple)) and len(v) == n and all(_is_num(x) for x in v)):
                bad.append(f"'{k}' must be a list of {n} numbers, got {v!r}")
            else:
                s(k, tuple(float(x) for x in v))
        if self.hidden_act != "silu":
            bad.append(f"'hidden_act' must be 'silu' (falcon_h1.c:383), got {self.hidden_act!r}")
        e = self.eos_token_id
        if isinstance(e, list):
            s("eos_token_id", tuple(e))
            e = self.eos_token_id
        if e is not None and not _is_int(e) and not (isinstance(e, tuple) and all(_is_int(x) for x in e)):
            bad.append(f"'eos_token_id' must be an integer or a list of integers, got {e!r}")
        if bad:
            raise ConfigError("config.json: " + "; ".join(bad))

        if self.num_key_value_heads is None:
            s("num_key_value_heads", self.num_attention_heads)
        if self.head_dim is None:
            if self.hidden_size % self.num_attention_heads:
                bad.append("'head_dim' is absent and hidden_size is not a multiple of num_attention_heads")
            s("head_dim", self.hidden_size // self.num_attention_heads)
        if self.mamba_d_ssm is None:
            s("mamba_d_ssm", self.mamba_expand * self.hidden_size)
        if self.mamba_d_head in (None, "auto"):
            if self.mamba_d_ssm % self.mamba_n_heads:
                bad.append("'mamba_d_head' is auto and mamba_d_ssm is not a multiple of mamba_n_heads")
            s("mamba_d_head", self.mamba_d_ssm // self.mamba_n_heads)
        elif not _is_int(self.mamba_d_head) or self.mamba_d_head <= 0:
            bad.append(f"'mamba_d_head' must be a positive integer or \"auto\", got {self.mamba_d_head!r}")
        if not bad:
            if self.num_attention_heads % self.num_key_value_heads:
                bad.append(f"num_attention_heads ({self.num_attention_heads}) must be a multiple of "
                           f"num_key_value_heads ({self.num_key_value_heads})")
            if self.mamba_n_heads * self.mamba_d_head != self.mamba_d_ssm:        # cpu_op.c:900
                bad.append(f"mamba_n_heads*mamba_d_head ({self.mamba_n_heads}*{self.mamba_d_head}) "
                           f"must equal mamba_d_ssm ({self.mamba_d_ssm})")
            if self.mamba_n_heads % self.mamba_n_groups:                           # graph.c:332
                bad.append(f"mamba_n_heads ({self.mamba_n_heads}) must be a multiple of "
                           f"mamba_n_groups ({self.mamba_n_groups})")
            if self.mamba_d_ssm % self.mamba_n_groups:
                bad.append("mamba_d_ssm must be a multiple of mamba_n_groups")
            if self.head_dim % 2:
                bad.append(f"head_dim ({self.head_dim}) must be even for the split-half rotation")
            if self.rms_norm_eps <= 0 or self.rope_theta <= 0:
                bad.append("rms_norm_eps and rope_theta must be positive")
        if bad:
            raise ConfigError("config.json: " + "; ".join(bad))

    # ---- derived sizes (falcon_h1.c:123-124, 342) --------------------------------------
    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def mamba_conv_dim(self) -> int:
        return self.mamba_d_ssm + 2 * self.mamba_n_groups * self.mamba_d_state

    @property
    def mamba_proj_dim(self) -> int:
        return self.mamba_d_ssm + self.mamba_conv_dim + self.mamba_n_heads

    @property
    def stop_token_ids(self) -> Tuple[int, ...]:
        e = self.eos_token_id
        if e is None:
            return ()
        return (e,) if isinstance(e, int) else tuple(e)
