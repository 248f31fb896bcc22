"""Sampling and generation options, named as in wlejon/brolm
(include/brolm/detail/generate.h:29-34 and :57-61)."""
from __future__ import annotations

import dataclasses


@dataclasses.dataclass
class SamplingParams:
    temperature: float = 1.0   # <= 0: greedy (argmax)
    top_k: int = 0             # 0: off; 1: greedy
    top_p: float = 1.0         # >= 1: off
    seed: int = 0

    @property
    def greedy(self) -> bool:
        """Greedy when temperature <= 0 or top_k == 1 (src/detail/generate.cpp:73-76)."""
        return self.temperature <= 0.0 or self.top_k == 1


@dataclasses.dataclass
class GenerateOptions:
    max_new_tokens: int = 64
    sampling: SamplingParams = dataclasses.field(default_factory=SamplingParams)
    stop_on_eos: bool = True       # stop when eos_id is drawn; the eos token is not returned
    stop_ids: tuple = ()           # further stop tokens, treated like eos
