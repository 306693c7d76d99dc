"""Sampling options of one request, with the reference's names, defaults and
bounds (src/frontend/sampling.rs:12-62)."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

from ..errors import ConfigError


@dataclass
class SamplingParams:
    temperature: float = 0.7          # 0: greedy
    top_p: float = 0.95               # nucleus mass, (0, 1]
    top_k: int = 0                    # 0: no limit
    repetition_penalty: float = 1.0   # > 0; applied once per distinct token of prompt + output
    seed: Optional[int] = None        # None: seeded from the system's entropy
    max_new_tokens: int = 512

    def validate(self) -> None:
        if not math.isfinite(self.temperature) or self.temperature < 0:
            raise ConfigError("temperature must be finite and not negative")
        if not math.isfinite(self.top_p) or self.top_p <= 0 or self.top_p > 1:
            raise ConfigError("top_p must lie in (0, 1]")
        if not isinstance(self.top_k, int) or self.top_k < 0:
            raise ConfigError("top_k must be a non-negative integer")
        if not math.isfinite(self.repetition_penalty) or self.repetition_penalty <= 0:
            raise ConfigError("repetition_penalty must be finite and positive")
        if self.max_new_tokens <= 0:
            raise ConfigError("max_new_tokens must be greater than zero")

    @property
    def is_greedy(self) -> bool:     # src/frontend/sampling.rs:87-89
        return self.temperature == 0.0 and self.repetition_penalty == 1.0
