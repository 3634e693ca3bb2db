"""Sampling parameters with CodeClaper/tinyllama.c's names, meanings and defaults
(SampleParam, def.h:81-90; defaults core.h:6-13, bench.c:68-80)."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.8          # -t/--temp; <= 1e-6 is greedy (sampler.c:146-147)
    top_k: int = 40                   # -tk/--topk; 0 = off
    top_p: float = 0.9                # -tp/--topp; 1.0 = off
    min_p: float = 0.05               # -P/--minp; 0 = off
    repeat_penalty: float = 1.1       # -rp; 1.0 = off
    repeat_last_n: int = 64           # -rl
    frequency_penalty: float = 0.0    # -fp
    presence_penalty: float = 0.0     # -pp
    seed: int = 0                     # the reference seeds from the thread id (sampler.c:13-17); here it is explicit

    def __post_init__(self):
        if self.temperature < 0.0:
            raise ValueError(f"Temperature must be >= 0.0, got {self.temperature:.2f}")       # bench.c:117-120
        if not (0.0 < self.top_p <= 1.0):
            raise ValueError(f"Top-p must be in (0.0, 1.0], got {self.top_p:.2f}")            # bench.c:121-124
        if not (0.0 <= self.min_p <= 1.0):
            raise ValueError(f"Min-p must be in [0.0, 1.0], got {self.min_p:.2f}")            # bench.c:125-128
        if self.top_k < 0 or self.repeat_last_n < 0:
            raise ValueError("top_k and repeat_last_n must be >= 0")

    @property
    def is_greedy(self) -> bool:
        """Greedy when the temperature is ~0, and also when no filter is active (sampler.c:146-151)."""
        no_filter = self.top_k == 0 and self.top_p >= 1.0 and self.min_p <= 1e-6
        return self.temperature <= 1e-6 or no_filter

    @property
    def has_penalties(self) -> bool:
        return (self.repeat_penalty != 1.0 or self.frequency_penalty != 0.0 or self.presence_penalty != 0.0) \
            and self.repeat_last_n > 0


GREEDY = SamplingParams(temperature=0.0, top_k=0, top_p=1.0, min_p=0.0, repeat_penalty=1.0)
