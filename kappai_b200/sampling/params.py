"""Sampling options of a request, with the reference's names, defaults and
meanings (src/config.c:156-172, help text :119-131)."""
from __future__ import annotations

from dataclasses import dataclass

MAX_TOP_K = 1024     # the device sampler keeps at most this many candidates (src/sampler.c:7)


@dataclass
class SamplingParams:
    temperature: float = 0.80      # -t; <= 0 is greedy
    top_k: int = 40                # -k; 0 disables
    top_p: float = 0.90            # -P; 1.0 disables
    min_p: float = 0.10            # -M; 0.0 disables
    repeat_penalty: float = 1.0    # --repeat-penalty; 1.0 disables
    repeat_last_n: int = 64        # --repeat-last-n
    seed: int = 0                  # -s; 0 = random
    n_predict: int = -1            # -n; -1 = until the context is full or EOS

    def validate(self, vocab_size: int) -> None:
        if self.top_k > MAX_TOP_K and self.top_k < vocab_size:
            raise ValueError(f"top_k={self.top_k}: the sampler keeps at most {MAX_TOP_K} candidates "
                             "(use 0 to disable top-k)")
        if self.repeat_penalty <= 0:
            raise ValueError("repeat_penalty must be positive")
        if not (0.0 <= self.min_p <= 1.0) or self.top_p < 0.0:
            raise ValueError("top_p and min_p must lie in [0, 1]")
        if self.repeat_last_n < 0 or self.repeat_last_n > 256:
            raise ValueError("repeat_last_n must lie in 0..256")

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0 or self.top_k == 1


GREEDY = SamplingParams(temperature=0.0, top_k=0, top_p=1.0, min_p=0.0)
