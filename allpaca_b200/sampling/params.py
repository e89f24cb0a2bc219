"""Per-request generation options, with the reference's names, meanings and defaults.

``GenerationParams`` of the reference (crates/allpaca-types/src/generation.rs:4-34):
``max_tokens`` 32, ``temperature`` 0.8, ``top_k`` 40, ``top_p`` 0.95, ``seed`` None,
``stop_token_ids`` [].  ``temperature <= 1e-5`` is greedy
(crates/allpaca-core/src/sampling.rs:36-38); ``top_k`` 0 switches it off (:262-264);
``top_p`` acts only for ``0 <= p < 1`` (:276-279); ``max_tokens`` 0 counts as 1
(crates/allpaca-core/src/engine.rs:3194-3196).  Structured-output options of the reference
(json_mode, json_schema, grammar) are not part of this engine.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

GREEDY_TEMPERATURE = 1e-5


@dataclass
class SamplingParams:
    max_tokens: int = 32
    temperature: float = 0.8
    top_k: int = 40
    top_p: float = 0.95
    seed: Optional[int] = None
    stop_token_ids: List[int] = field(default_factory=list)

    def __post_init__(self):
        if self.max_tokens < 0:
            raise ValueError("max_tokens must not be negative")
        if self.max_tokens == 0:
            self.max_tokens = 1
        if self.top_k < 0:
            raise ValueError("top_k must not be negative (0 switches it off)")
        if self.temperature < 0:
            raise ValueError("temperature must not be negative")
        self.stop_token_ids = [int(t) for t in self.stop_token_ids]

    @property
    def greedy(self) -> bool:
        return self.temperature <= GREEDY_TEMPERATURE

    @classmethod
    def greedy_params(cls, max_tokens: int = 32, stop_token_ids=()) -> "SamplingParams":
        return cls(max_tokens=max_tokens, temperature=0.0, top_k=0, top_p=1.0,
                   stop_token_ids=list(stop_token_ids))
