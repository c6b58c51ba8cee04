"""Per-request generation options, with the reference's names and meanings.

``max_tokens`` (default 128), ``temperature`` (default 1.0; 0 means greedy), ``top_p``
(default 1.0, in (0, 1]), ``seed`` and ``stop`` are the options of the reference's
request type and their validation (src/engine/types.rs:14-37; API defaults
src/api/openai.rs:70-96, 160-167).  ``stop_token_ids`` and ``ignore_eos`` are additions
for a token-ids-in, token-ids-out engine.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional, Sequence, Tuple


@dataclass(frozen=True)
class SamplingParams:
    max_tokens: int = 128
    temperature: float = 1.0
    top_p: float = 1.0
    seed: Optional[int] = None
    stop: Tuple[str, ...] = ()
    stop_token_ids: Tuple[int, ...] = ()
    ignore_eos: bool = False

    def __post_init__(self):
        object.__setattr__(self, "stop", tuple([self.stop] if isinstance(self.stop, str) else self.stop))
        object.__setattr__(self, "stop_token_ids", tuple(self.stop_token_ids))
        self.validate()

    def validate(self) -> None:
        if self.max_tokens <= 0:
            raise ValueError("max_tokens must be positive")
        if not math.isfinite(self.temperature) or self.temperature < 0.0:
            raise ValueError("temperature must be finite and non-negative")
        if not math.isfinite(self.top_p) or not 0.0 < self.top_p <= 1.0:
            raise ValueError("top_p must be in (0, 1]")
        if any(s == "" for s in self.stop):
            raise ValueError("stop strings must not be empty")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0
