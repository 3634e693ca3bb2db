"""Loading a model folder (config.json + safetensors) and writing one with random weights.

CodeClaper/tinyllama.c binds tensors by name against a per-architecture table with
required flags, and stops at the first missing one (core.c:961-1254, 1289-1345).  Here the
table is the model's own ``weight_specs()``; every name and shape is checked before
anything is bound and one error lists all missing and unexpected tensors and all wrong
shapes.  bfloat16 tensors stay bfloat16, tensors stored in 32-bit stay 32-bit, integer
tables become int32; a float32 run widens everything.
"""
from __future__ import annotations

import hashlib
import json
import math
import os
from typing import Dict, Optional, Union

import torch

from ..config.base import ModelConfig, config_from_dict, load_config, lookup_architecture
from ..models.model import Model
from . import safetensors_io as st


class WeightError(ValueError):
    """The tensors in the model folder do not match what the architecture declares."""


_RUN_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
               torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def run_dtype(dtype) -> torch.dtype:
    if dtype not in _RUN_DTYPES:
        raise ValueError(f"dtype must be bfloat16 or float32, got {dtype!r}")
    return _RUN_DTYPES[dtype]


def build_model(config: ModelConfig) -> Model:
    _, builder = lookup_architecture(config.architecture)
    return builder(config)


def check_tensors(model: Model, tensors: Dict[str, torch.Tensor]) -> None:
    specs = {s.name: s for s in model.weight_specs()}
    missing = sorted(n for n in specs if n not in tensors)
    unexpected = sorted(n for n in tensors if n not in specs)
    wrong = []
    for n, s in specs.items():
        if n in tensors and tuple(tensors[n].shape) != tuple(s.shape):
            wrong.append(f"{n}: expected {list(s.shape)}, found {list(tensors[n].shape)}")
    bad_type = sorted(f"{n}: {tensors[n].dtype}" for n in specs
                      if n in tensors and not tensors[n].dtype.is_floating_point)
    if missing or unexpected or wrong or bad_type:
        lines = [f"weights do not match architecture {model.config.architecture}:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            lines.append(f"  wrong shapes ({len(wrong)}): " + "; ".join(wrong))
        if bad_type:
            lines.append(f"  not floating point ({len(bad_type)}): " + "; ".join(bad_type))
        raise WeightError("\n".join(lines))


def normalise(t: torch.Tensor) -> torch.Tensor:
    """Storage types the kernels do not take: half -> bfloat16, double -> float32, integers -> int32."""
    if t.dtype in (torch.float32, torch.bfloat16):
        return t
    if t.dtype == torch.float16:
        return t.to(torch.bfloat16)
    if t.dtype == torch.float64:
        return t.to(torch.float32)
    if not t.dtype.is_floating_point:
        return t.to(torch.int32)
    return t.to(torch.float32)


def load_model(model_dir: str, dtype: Union[str, torch.dtype] = "bfloat16", device="cuda") -> Model:
    """Model folder -> model bound to its weights on `device`, computing in `dtype`."""
    rd = run_dtype(dtype)
    config = load_config(model_dir)
    model = build_model(config)
    try:
        tensors = st.load_model_dir(model_dir)
    except st.SafetensorsError as e:
        raise WeightError(str(e)) from e
    check_tensors(model, tensors)
    model.bind({k: normalise(v) for k, v in tensors.items()}, rd, torch.device(device))
    return model


# ---- random weights ------------------------------------------------------------------------
def _generator(seed: int, name: str) -> torch.Generator:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    g = torch.Generator(device="cpu")
    g.manual_seed(int.from_bytes(h[:8], "little") & ((1 << 63) - 1))
    return g


def draw_tensor(spec, generator: torch.Generator, dtype: torch.dtype, std: float, norm_std: float = 0.1) -> torch.Tensor:
    """One weight by its init rule, drawn from `generator` on the generator's device.  Matrices,
    embeddings, biases and conv taps are N(0, std), norm weights 1 + N(0, norm_std), A_log =
    log U(1, 16), dt_bias the inverse softplus of a log-uniform time step in [1e-3, 0.1], D = 1 +
    N(0, norm_std).  Matrices are stored in `dtype`; the per-head SSM constants in float32."""
    dev, f32 = generator.device, torch.float32
    if spec.init in ("normal", "conv"):
        t = torch.empty(spec.shape, dtype=f32, device=dev).normal_(0.0, std, generator=generator).to(dtype)
    elif spec.init == "ones":
        t = (1.0 + torch.empty(spec.shape, dtype=f32, device=dev).normal_(0.0, norm_std, generator=generator)).to(dtype)
    elif spec.init == "zeros":
        t = torch.zeros(spec.shape, dtype=dtype, device=dev)
    elif spec.init == "a_log":
        t = torch.log(1.0 + 15.0 * torch.rand(spec.shape, generator=generator, dtype=f32, device=dev))
    elif spec.init == "dt_bias":
        u = torch.rand(spec.shape, generator=generator, dtype=f32, device=dev)
        step = torch.exp(u * (math.log(0.1) - math.log(1e-3)) + math.log(1e-3))
        t = step + torch.log(-torch.expm1(-step))
    elif spec.init == "d_skip":
        t = 1.0 + torch.empty(spec.shape, dtype=f32, device=dev).normal_(0.0, norm_std, generator=generator)
    else:
        raise ValueError(f"weight {spec.name}: unknown init rule '{spec.init}'")
    return t.contiguous()


def random_tensors(model: Model, seed: int, dtype: torch.dtype = torch.bfloat16, std: Optional[float] = None,
                   norm_std: float = 0.1) -> Dict[str, torch.Tensor]:
    """One tensor per declared weight (see draw_tensor), each drawn from its own generator keyed by
    (seed, name), so a tensor does not depend on which others exist; std defaults to the config's
    initializer_range, else 0.02."""
    std = float(std if std is not None else getattr(model.config, "initializer_range", 0.02))
    return {s.name: draw_tensor(s, _generator(seed, s.name), dtype, std, norm_std) for s in model.weight_specs()}


def random_model(config: Union[ModelConfig, dict], seed: int = 0, dtype: Union[str, torch.dtype] = "bfloat16",
                 device: str = "cuda:0", std: Optional[float] = None,
                 compute_dtype: Union[str, torch.dtype, None] = None) -> Model:
    """A model bound to random weights drawn on `device` by the rules of draw_tensor (one generator for
    all tensors; no folder is written): for benchmarks of configurations too large to be worth a round
    trip through a file.  `dtype` is what the matrices are stored as, `compute_dtype` (default: the same)
    what the model computes in: bfloat16 weights in a float32 run are widened exactly."""
    if isinstance(config, dict):
        config = config_from_dict(dict(config))
    model = build_model(config)
    rd = run_dtype(dtype)
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    std = float(std if std is not None else getattr(config, "initializer_range", 0.02))
    tensors = {s.name: draw_tensor(s, gen, rd, std) for s in model.weight_specs()}
    model.bind(tensors, rd if compute_dtype is None else run_dtype(compute_dtype), torch.device(device))
    return model


def write_random_model(config: Union[ModelConfig, dict], out_dir: str, seed: int = 0,
                       dtype: Union[str, torch.dtype] = "bfloat16", std: Optional[float] = None,
                       norm_std: float = 0.1) -> str:
    """Writes config.json and model.safetensors for `config` with weights drawn from `seed`."""
    if isinstance(config, dict):
        raw = dict(config)
        config = config_from_dict(raw)
    model = build_model(config)
    tensors = random_tensors(model, seed, run_dtype(dtype), std, norm_std)
    os.makedirs(out_dir, exist_ok=True)
    cfg = config.to_dict()
    cfg["torch_dtype"] = "bfloat16" if run_dtype(dtype) == torch.bfloat16 else "float32"
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(cfg, f, indent=2)
    st.save_file(tensors, os.path.join(out_dir, "model.safetensors"))
    return out_dir
