"""Per-request sampling options, with the names and meanings of the reference's
``SamplingConfig`` / ``GenerationConfig`` (infMain/include/serving/generation_config.h:22-63)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List

_MASK64 = (1 << 64) - 1


def request_sample_uniform(seed: int, counter: int) -> float:
    """The request's ``counter``-th uniform draw in [0, 1): SplitMix64 of
    ``seed + phi * (counter + 1)``, top 24 bits.  It depends on the request's seed and on
    how many tokens it has sampled, never on batch order, handles or retries
    (infMain/include/serving/generation_config.h:14-20)."""
    z = (seed + 0x9E3779B97F4A7C15 * (counter + 1)) & _MASK64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK64
    z ^= z >> 31
    return float(z >> 40) * (1.0 / 16777216.0)


@dataclass
class SamplingParams:
    max_new_tokens: int = 128        # stop after this many sampled tokens (>= 1)
    min_new_tokens: int = 0          # EOS is ignored until more than this many are generated
    ignore_eos: bool = False         # never stop on EOS
    temperature: float = 0.0         # 0: greedy; else logits / max(T, 1e-6)
    top_k: int = 0                   # 0: off
    top_p: float = 1.0               # nucleus over the ordered candidates, at least one kept
    repetition_penalty: float = 1.0  # seen tokens: logit / p when positive, logit * p otherwise
    seed: int = 0xC0FFEE
    priority: int = 0                # accepted for compatibility; scheduling is first come first served

    def normalized(self) -> "SamplingParams":
        p = SamplingParams(**self.__dict__)
        p.temperature = max(0.0, float(p.temperature))
        p.top_p = min(1.0, max(0.0, float(p.top_p)))
        p.top_k = max(0, int(p.top_k))
        p.repetition_penalty = max(0.0, float(p.repetition_penalty))
        p.max_new_tokens = max(1, int(p.max_new_tokens))
        p.min_new_tokens = max(0, min(int(p.min_new_tokens), p.max_new_tokens))
        p.seed = int(p.seed) & _MASK64
        return p

    @property
    def is_greedy(self) -> bool:
        """infMain/source/model/qwen2.cpp:104-107."""
        return self.temperature <= 0.0 and self.top_k <= 0 and self.top_p >= 1.0 \
            and self.repetition_penalty == 1.0
