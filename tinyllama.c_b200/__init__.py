"""tinyllama.c_b200: a small model library with generation for one GPU (NVIDIA B200).

It covers what CodeClaper/tinyllama.c does between a request's tokens and its next
token, for the Falcon-H1 architecture: configuration and registry, weights from
safetensors, layers put together from parts, a paged cache with per-sequence state, one
step function, a generation loop, samplers, and hand-written CUDA kernels for sm_100a.

    import tinyllama_c_b200 as tlc
    llm = tlc.LLM("model_dir", dtype="bfloat16", max_tokens=8192)
    results = llm.generate([[1, 2, 3], [4, 5]], tlc.SamplingParams(temperature=0.0), max_new_tokens=16)
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Union

import torch

from . import models as _models  # noqa: F401  (registers the architectures)
from .cache import Cache, CacheError
from .config import ConfigError, FalconH1Config, load_config, register_architecture, registered_architectures
from .engine import Continuation, EngineBackend, GenerationResult, StepEntry, StepError, generate, step
from .parts import (ChunkRequest, KVRequest, LayerRun, LayerSpec, Part, PartSpec, Position, StateRequest, StepInfo, WeightSpec,
                    register_feed_forward, register_mixer, register_norm, register_position)
from .sampling import GREEDY, Sampler, SamplingParams
from .weights import WeightError, build_model, load_model, write_random_model

__all__ = ["LLM", "SamplingParams", "GREEDY", "load_model", "write_random_model", "Cache", "StepEntry", "step",
           "generate", "GenerationResult", "Continuation", "register_architecture", "register_mixer", "register_feed_forward",
           "register_norm", "register_position", "ConfigError", "WeightError", "CacheError", "StepError"]


class LLM:
    """A loaded model with its cache: the Python entry point.

    max_tokens sizes the key/value cache (positions held by live sequences together, each
    rounded up to 64); max_seqs the number of live sequences (default: as many as max_tokens
    allows, at most 256)."""

    def __init__(self, model_dir, dtype: Union[str, torch.dtype] = "bfloat16", max_tokens: int = 8192,
                 max_seqs: Optional[int] = None, device: str = "cuda:0", use_graphs: bool = True):
        """model_dir: a folder with config.json and model.safetensors, or a model that is
        already bound to its weights on `device` (see random_model)."""
        if not torch.cuda.is_available():
            raise RuntimeError("tinyllama.c_b200 needs a CUDA device (NVIDIA B200); there is no CPU path")
        from . import ops
        ops.library()                                   # build / load the kernels now, loudly
        torch.cuda.set_device(torch.device(device))
        self.model = load_model(model_dir, dtype, device) if isinstance(model_dir, (str, bytes)) else model_dir
        self.config = self.model.config
        self.use_graphs = use_graphs
        self._graphs: dict = {}
        self.last_stats: dict = {}
        n_pages = (int(max_tokens) + 63) // 64
        self.max_seqs = int(max_seqs) if max_seqs else max(1, min(n_pages, 256))
        self.cache = Cache(self.model.cache_requests(), max_tokens, self.max_seqs, self.model.dtype, device)
        self.max_context = min(n_pages * 64, getattr(self.config, "max_position_embeddings", 1 << 30))

    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        return step(self.model, self.cache, entries)

    def generate(self, prompts: Sequence[Sequence[int]], params: SamplingParams = SamplingParams(),
                 max_new_tokens: int = 128, stop_ids: Optional[Sequence[int]] = None, max_batch: int = 64,
                 ignore_eos: bool = False, max_step_tokens: int = 8192,
                 continuations: Optional[Sequence[Optional[Continuation]]] = None, on_token=None) -> List[GenerationResult]:
        """Token ids in, token ids out (host lists).  continuations[i] lets request i go on in a slot the
        caller holds (a further turn of a conversation); on_token(i, token) sees every token as it is made."""
        if stop_ids is None:
            stop_ids = getattr(self.config, "stop_token_ids", ())
        backend = EngineBackend(self.model, self.cache, params, self._graphs, self.use_graphs, max_step_tokens)
        try:
            return generate(backend, prompts, max_new_tokens, stop_ids, max_batch, self.max_context, ignore_eos,
                            continuations, on_token)
        finally:
            self.last_stats = backend.stats


def random_model(config: dict, seed: int = 0, dtype: Union[str, torch.dtype] = "bfloat16", device: str = "cuda:0",
                 std: Optional[float] = None, run_dtype: Union[str, torch.dtype, None] = None):
    """A model with random weights drawn on the device (see weights.loader.random_model)."""
    from .weights.loader import random_model as _random_model
    return _random_model(config, seed, dtype, device, std, run_dtype)
